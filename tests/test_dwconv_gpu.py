"""Depthwise / transposed compact convolutions and the reference-named fp32 operators against the oracle.
Depthwise results are bit-exact (fp32, fixed tap order); the fp32 GEMM operators are compared with the fp64 product."""
import numpy as np
import pytest
import torch

from oracle import ternary as T

pytestmark = pytest.mark.gpu

GEOMS = [  # C, H, W, kernel, stride, padding, dilation, output_padding
    (20, 9, 11, (3, 3), (1, 1), (1, 1), (1, 1), (0, 0)),
    (33, 12, 10, (3, 5), (2, 1), (1, 2), (1, 1), (1, 0)),
    (16, 8, 8, (5, 5), (2, 2), (2, 2), (1, 1), (1, 1)),
    (7, 10, 9, (3, 3), (1, 2), (2, 1), (2, 1), (0, 1)),
    (64, 28, 28, (3, 3), (1, 1), (1, 1), (1, 1), (0, 0)),
    (5, 6, 7, (1, 1), (1, 1), (0, 0), (1, 1), (0, 0)),
    (48, 5, 5, (7, 7), (1, 1), (3, 3), (1, 1), (0, 0)),
    (8, 20, 130, (5, 5), (1, 1), (2, 2), (1, 1), (0, 0)),      # several tiles in x, tiled kernel
    (3, 17, 70, (3, 3), (1, 1), (0, 0), (1, 1), (0, 0)),       # output width not a multiple of 4
    (4, 33, 65, (7, 7), (1, 1), (1, 2), (1, 1), (0, 0)),
    (40, 12, 12, (5, 5), (1, 1), (0, 0), (1, 1), (0, 0)),      # marching kernel: no padding, width shrinks by 4
    (9, 20, 132, (5, 5), (1, 1), (2, 2), (1, 1), (0, 0)),      # marching kernel: several warps per row
    (48, 8, 8, (7, 7), (1, 1), (3, 3), (1, 1), (0, 0)),
    (6, 10, 16, (3, 3), (1, 1), (0, 0), (1, 1), (0, 0)),
    (130, 7, 4, (3, 3), (1, 1), (1, 1), (1, 1), (0, 0)),       # one chunk per row
    (5, 6, 8, (3, 3), (1, 1), (2, 1), (1, 1), (0, 0)),         # taller padding than "same"
    (24, 56, 56, (3, 3), (2, 2), (1, 1), (1, 1), (1, 1)),      # stride-2 tiles (forward), generic gather (transposed)
    (10, 31, 140, (5, 5), (2, 2), (2, 2), (1, 1), (0, 0)),
]


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


def _case(C, H, W, k, seed, B=3):
    rng = np.random.default_rng(seed)
    Wt = rng.integers(-1, 2, (C, 1) + k).astype(np.float32)
    P = T.pack(Wt)                                       # [1, ky, kx, ceil(C/16)]
    x = rng.standard_normal((B, C, H, W)).astype(np.float32)
    sc = (rng.random(C) + 0.5).astype(np.float32)
    bi = rng.standard_normal(C).astype(np.float32)
    return Wt, P, x, sc, bi


@pytest.mark.parametrize("geom", GEOMS)
def test_dwconv2d_bit_exact(ops, geom):
    C, H, W, k, s, p, d, _ = geom
    Wt, P, x, sc, bi = _case(C, H, W, k, C * 100 + H)
    Pd, xd = torch.from_numpy(P).cuda(), torch.from_numpy(x).cuda()
    y = ops.ternary_dwconv2d(xd, Pd, k, s, p, d, torch.from_numpy(sc), torch.from_numpy(bi))
    assert np.array_equal(y.cpu().numpy().view(np.uint32), T.dwconv2d(x, P, k, s, p, d, sc, bi).view(np.uint32))
    y0 = ops.ternary_dwconv2d(xd, Pd, k, s, p, d)
    assert np.array_equal(y0.cpu().numpy().view(np.uint32), T.dwconv2d(x, P, k, s, p, d).view(np.uint32))
    ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(Wt).double(), None, s, p, d, groups=C)
    assert torch.allclose(y0.cpu().double(), ref, rtol=0, atol=1e-5)


@pytest.mark.parametrize("geom", GEOMS)
def test_dwconvtrans2d_bit_exact(ops, geom):
    C, H, W, k, s, p, d, op = geom
    Wt, P, x, sc, bi = _case(C, H, W, k, C * 77 + W)
    Pd, xd = torch.from_numpy(P).cuda(), torch.from_numpy(x).cuda()
    y = ops.ternary_dwconvtrans2d(xd, Pd, k, s, p, d, op, torch.from_numpy(sc), torch.from_numpy(bi))
    want = T.dwconvtrans2d(x, P, k, s, p, d, op, sc, bi)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))
    y0 = ops.ternary_dwconvtrans2d(xd, Pd, k, s, p, d, op)
    ref = torch.nn.functional.conv_transpose2d(torch.from_numpy(x).double(), torch.from_numpy(Wt).double(), None, s, p, op,
                                               C, d)
    assert torch.allclose(y0.cpu().double(), ref, rtol=0, atol=1e-5)


@pytest.mark.parametrize("C,P_,k", [(20, 50, (3, 3)), (64, 300, (3, 3)), (7, 33, (5, 2)), (130, 65, (1, 1))])
def test_operator_level_forms(ops, C, P_, k):
    """ternary_dwconv_cuda / ternary_dwconvtrans_cuda on the reference operators' own layouts, all ranks, all batches."""
    rng = np.random.default_rng(C + P_)
    nt = k[0] * k[1]
    Wt = rng.integers(-1, 2, (C, 1) + k).astype(np.float32)
    P = T.pack(Wt)
    Pd = torch.from_numpy(P).cuda()
    x = rng.standard_normal((2, P_, nt * C)).astype(np.float32)
    want = T.dwconv_patches(x, P, C, nt).reshape(2, P_, C)
    for view in (x, x[:, None], x[0]):
        y = ops.ternary_dwconv_cuda(torch.from_numpy(np.ascontiguousarray(view)).cuda(), Pd, k[1], k[0], C)
        w = want if view.ndim == 3 else (want[:, None] if view.ndim == 4 else want[0])
        assert y.shape == w.shape
        assert np.array_equal(y.cpu().numpy().view(np.uint32), np.ascontiguousarray(w).view(np.uint32))
    xt = rng.standard_normal((2, P_, C)).astype(np.float32)
    wantt = T.dwconvtrans_patches(xt, P, C, nt)
    for view in (xt, xt[:, None], xt[1]):
        y = ops.ternary_dwconvtrans_cuda(torch.from_numpy(np.ascontiguousarray(view)).cuda(), Pd, k[1], k[0])
        w = wantt if view.ndim == 3 else (wantt[:, None] if view.ndim == 4 else wantt[1])
        assert y.shape == w.shape
        assert np.array_equal(y.cpu().numpy().view(np.uint32), np.ascontiguousarray(w).view(np.uint32))


def test_unfold_operator_fold_equals_direct(ops):
    """The reference's composition (F.unfold -> ternary_dwconv_cuda; ternary_dwconvtrans_cuda -> F.fold) and the direct
    kernels agree: bit-exact forward (same tap order), to rounding for the transposed form (fold sums in its own order)."""
    C, H, W, k = 24, 14, 14, (3, 3)
    Wt, P, x, _, _ = _case(C, H, W, k, 5, B=2)
    Pd, xd = torch.from_numpy(P).cuda(), torch.from_numpy(x).cuda()
    unf = torch.nn.functional.unfold(xd, kernel_size=k, padding=1)                         # [B, C*9, L]
    perm = unf.view(2, C, 3, 3, -1).permute(0, 4, 2, 3, 1).reshape(2, H * W, 9 * C).contiguous()
    conv = ops.ternary_dwconv_cuda(perm, Pd, 3, 3, C)                                       # [B, L, C]
    direct = ops.ternary_dwconv2d(xd, Pd, k, (1, 1), (1, 1))
    assert torch.equal(conv.transpose(1, 2).reshape(2, C, H, W), direct)
    cols = ops.ternary_dwconvtrans_cuda(xd.reshape(2, C, H * W).transpose(1, 2).contiguous(), Pd, 3, 3)
    folded = torch.nn.functional.fold(cols, output_size=(2 * H, 2 * W), kernel_size=k, stride=2, padding=1,
                                      )[:, :, :, :]
    direct_t = ops.ternary_dwconvtrans2d(xd, Pd, k, (2, 2), (1, 1), (1, 1), (1, 1))
    assert torch.allclose(folded, direct_t, rtol=0, atol=1e-5)


@pytest.mark.parametrize("shape", [(1, 64, 128), (5, 300, 200), (1, 3, 40, 72)])
def test_reference_named_gemm_operators(ops, shape):
    """ternary_mmm_cuda / ternary_mvm_cuda: fp32 activations, reference packed layout, any batch rank."""
    *lead, M, K = shape
    N = 200
    rng = np.random.default_rng(M * K)
    Wm = rng.integers(-1, 2, (N, K)).astype(np.float32)
    P = T.pack(Wm)
    Pd = torch.from_numpy(P).cuda()
    x = rng.standard_normal(shape).astype(np.float32)
    y = ops.ternary_mmm_cuda(torch.from_numpy(x).cuda(), Pd, N)
    assert tuple(y.shape) == tuple(shape[:-1]) + (N,)
    ref = x.reshape(-1, K).astype(np.float64) @ Wm.T.astype(np.float64)
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(y.cpu().double().numpy().reshape(-1, N) - ref) <= 2e-6 * np.maximum(np.abs(ref), rms))
    for v in (x.reshape(-1, K)[0], x.reshape(-1, K)[:1], x.reshape(-1, K)[:1][None]):
        yv = ops.ternary_mvm_cuda(torch.from_numpy(np.ascontiguousarray(v)).cuda(), Pd, N)
        assert tuple(yv.shape) == tuple(v.shape[:-1]) + (N,)
        assert np.all(np.abs(yv.cpu().double().numpy().reshape(-1) - ref[0]) <= 2e-6 * np.maximum(np.abs(ref[0]), rms[0]))


def test_compact_layers_depthwise_and_transposed():
    """quantize_model -> compressed_state_dict -> compact inference for a depthwise Conv2d, a depthwise
    ConvTranspose2d and a dense ConvTranspose2d, against the same layers run from their rounded fp32 weights."""
    import tmq_b200 as tmq
    torch.manual_seed(0)
    net = torch.nn.Sequential(
        torch.nn.Conv2d(16, 16, 3, padding=1, groups=16, bias=True),
        torch.nn.ConvTranspose2d(16, 16, 3, stride=2, padding=1, output_padding=1, groups=16, bias=True),
        torch.nn.ConvTranspose2d(16, 24, 4, stride=2, padding=1, bias=True),
    ).cuda()
    ctrl = tmq.QuantizationControl(device="cuda")
    tmq.quantize_model(net, ctrl)
    with torch.no_grad():
        for m in net:
            m.bias.uniform_(-1, 1)
    net.eval()
    tmq.quantize_weights(net)
    ctrl.inference()
    x = torch.randn(2, 16, 10, 12, device="cuda")
    with torch.no_grad():
        w = [m.weight.data.clone() for m in net]
        want = torch.nn.functional.conv2d(x.double(), w[0].double(), net[0].bias.double(), padding=1, groups=16)
        want = torch.nn.functional.conv_transpose2d(want, w[1].double(), net[1].bias.double(), stride=2, padding=1,
                                                    output_padding=1, groups=16)
        want = torch.nn.functional.conv_transpose2d(want, w[2].double(), net[2].bias.double(), stride=2, padding=1)
    sd = tmq.compressed_state_dict(net)
    assert all(m.weight.dtype == torch.int32 for m in net)
    with torch.no_grad():
        got = net(x)
    assert got.shape == want.shape
    assert torch.allclose(got.double(), want, rtol=0, atol=2e-4)
