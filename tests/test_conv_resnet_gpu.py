"""Implicit-GEMM convolution and the ResNet-18 workloads (baseline configuration 4) on the GPU."""
import numpy as np
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


def _conv_case(ops, b, c, h, w, n, k, s, p, d, relu, seed):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(b, c, h, w, generator=gen).to(torch.bfloat16)
    wgt = torch.randint(-1, 2, (n, c, k, k), generator=gen).float()
    scale = torch.rand(n, generator=gen) * 0.09 + 0.01
    bias = torch.randn(n, generator=gen)
    ref = nn.functional.conv2d(x.double(), wgt.double(), None, s, p, d) * scale.double().view(1, -1, 1, 1) \
        + bias.double().view(1, -1, 1, 1)
    if relu:
        ref = torch.relu(ref)
    packed = ops.compactify_ternary(wgt.cuda())                       # [c, k, k, q], rows (c, ky, kx)
    rows = packed.view(c * k * k, -1)
    idx = torch.arange(c * k * k)
    cc, rem = idx // (k * k), idx % (k * k)
    perm = torch.argsort(rem * c + cc).cuda()                          # to (ky, kx, c) order
    wt = ops.prepack(rows.index_select(0, perm).contiguous(), n, ops.FMT_BF16)
    y = ops.ternary_conv2d_nhwc(x.cuda().permute(0, 2, 3, 1).contiguous(), wt, n, (k, k), (s, s), (p, p), (d, d),
                                scale.cuda(), bias.cuda(), relu=relu)
    ops.check_gemm_status()
    got = y.permute(0, 3, 1, 2).double().cpu()
    assert got.shape == ref.shape
    tol = 2.0 ** -7 * ref.abs() + 1e-4 * ref.abs().max()               # one bf16 ulp of the output + accumulation slack
    assert bool(((got - ref).abs() <= tol).all()), float((got - ref).abs().max())


@pytest.mark.parametrize("case", [
    (2, 64, 12, 12, 64, 3, 1, 1, 1, True), (3, 64, 15, 13, 128, 3, 2, 1, 1, False), (2, 128, 9, 9, 128, 3, 1, 1, 1, True),
    (2, 64, 14, 14, 128, 1, 2, 0, 1, False), (1, 256, 7, 7, 512, 3, 2, 1, 1, True), (2, 64, 10, 10, 72, 3, 1, 2, 2, False),
    (5, 128, 28, 28, 256, 3, 1, 1, 1, True), (1, 512, 7, 7, 512, 3, 1, 1, 1, True)])
def test_implicit_conv_matches_conv2d(ops, case):
    b, c, h, w, n, k, s, p, d, relu = case
    _conv_case(ops, b, c, h, w, n, k, s, p, d, relu, seed=sum(case[:9]))


S1_CASES = [
    # b, c, h, w, n, (ky, kx), (py, px), (dy, dx), relu, residual
    (3, 64, 56, 56, 64, (3, 3), (1, 1), (1, 1), True, True),        # two output rows per tile
    (2, 128, 28, 28, 128, (3, 3), (1, 1), (1, 1), True, False),
    (2, 256, 14, 14, 256, (3, 3), (1, 1), (1, 1), False, True),     # two channel tiles, two row tiles per image
    (5, 512, 7, 7, 512, (3, 3), (1, 1), (1, 1), True, True),        # two images side by side in one tile, odd image count
    (1, 64, 7, 7, 72, (3, 3), (1, 1), (1, 1), False, False),        # a single small image, ragged channel count
    (2, 64, 13, 9, 200, (3, 3), (0, 0), (1, 1), False, False),      # no padding
    (2, 64, 11, 150, 64, (3, 3), (1, 1), (1, 1), True, False),      # rows wider than a tile: column pieces
    (2, 64, 20, 20, 64, (3, 3), (2, 2), (2, 2), False, False),      # dilation 2
    (3, 128, 9, 12, 64, (1, 1), (0, 0), (1, 1), True, True),        # 1 x 1
    (2, 64, 10, 17, 96, (3, 1), (1, 0), (1, 1), False, False),      # 3 x 1 kernel, asymmetric padding
    (2, 64, 12, 12, 64, (2, 2), (1, 0), (1, 1), False, False),      # even kernel: output larger / smaller than the input
    # one input slice, <= 64 output channels and enough tiles for two streams per SM: the pixel-major kernel
    (12, 64, 56, 56, 64, (3, 3), (1, 1), (1, 1), True, True),
    (11, 64, 56, 40, 48, (3, 3), (1, 1), (1, 1), False, True),      # 48 channels
    (16, 64, 40, 44, 36, (3, 3), (0, 0), (1, 1), True, False),      # channel count that is no multiple of 8: scalar stores
    (5, 64, 30, 260, 64, (3, 3), (1, 1), (1, 1), False, False),     # column pieces
    (40, 64, 24, 24, 64, (1, 1), (0, 0), (1, 1), True, True),       # 1 x 1
]


@pytest.mark.parametrize("case", S1_CASES)
def test_shifted_window_conv_matches_conv2d(ops, case):
    b, c, h, w, n, (ky, kx), (py, px), (dy, dx), relu, with_res = case
    gen = torch.Generator().manual_seed(b * 1000 + c + h * 7 + w + n)
    x = torch.randn(b, c, h, w, generator=gen).to(torch.bfloat16)
    wgt = torch.randint(-1, 2, (n, c, ky, kx), generator=gen).float()
    scale = torch.rand(n, generator=gen) * 0.09 + 0.01
    bias = torch.randn(n, generator=gen)
    ref = nn.functional.conv2d(x.double(), wgt.double(), None, 1, (py, px), (dy, dx)) * scale.double().view(1, -1, 1, 1) \
        + bias.double().view(1, -1, 1, 1)
    res = None
    if with_res:
        res = torch.randn(ref.shape, generator=gen).to(torch.bfloat16)
        ref = ref + res.double()
    if relu:
        ref = torch.relu(ref)
    packed = ops.compactify_ternary(wgt.cuda())
    wt = ops.prepack(ops.conv_rows_skkc(packed, c, ky, kx), n, ops.FMT_BF16)
    y = ops.ternary_conv2d_s1(x.cuda().permute(0, 2, 3, 1).contiguous(), wt, n, (ky, kx), (py, px), (dy, dx), scale.cuda(),
                              bias.cuda(), relu=relu,
                              residual=None if res is None else res.cuda().permute(0, 2, 3, 1).contiguous())
    ops.check_gemm_status()
    assert y is not None
    got = y.permute(0, 3, 1, 2).double().cpu()
    assert got.shape == ref.shape
    tol = 2.0 ** -7 * ref.abs() + 1e-4 * ref.abs().max()
    bad = (got - ref).abs() > tol
    assert not bool(bad.any()), (int(bad.sum()), float((got - ref).abs().max()))
    # the gather kernel computes the same sums in the same precision: the two agree to the last bf16 bit almost everywhere
    wt2 = ops.prepack(ops.conv_rows_kkc(packed, c, ky, kx), n, ops.FMT_BF16)
    y2 = ops.ternary_conv2d_nhwc(x.cuda().permute(0, 2, 3, 1).contiguous(), wt2, n, (ky, kx), (1, 1), (py, px), (dy, dx),
                                 scale.cuda(), bias.cuda(), relu=relu,
                                 residual=None if res is None else res.cuda().permute(0, 2, 3, 1).contiguous())
    assert float((y.float() != y2.float()).float().mean()) < 1e-3


STEM_CASES = [
    # b, c, h, w, n, (ky, kx), (sy, sx), (py, px), relu
    (2, 3, 224, 224, 64, (7, 7), (2, 2), (3, 3), False),        # the ResNet stem
    (3, 3, 64, 64, 64, (7, 7), (2, 2), (3, 3), True),
    (2, 1, 30, 40, 32, (3, 3), (2, 2), (1, 1), False),          # one channel
    (2, 4, 33, 31, 64, (5, 5), (2, 2), (2, 2), True),           # all four channel slots used, odd sizes
    (2, 3, 21, 50, 40, (3, 5), (1, 2), (0, 2), False),          # vertical stride 1, 40 channels
    (2, 8, 20, 24, 64, (3, 3), (1, 1), (1, 1), True),           # horizontal stride 1: eight channel slots
    (1, 5, 17, 19, 56, (3, 3), (2, 1), (1, 1), False),
    (7, 3, 50, 60, 64, (7, 7), (2, 2), (3, 3), True),           # several images per CTA range: refills at image boundaries
    (300, 2, 9, 12, 20, (3, 3), (2, 2), (1, 1), False),         # many small images, channel count no multiple of 8
]


@pytest.mark.parametrize("case", STEM_CASES)
def test_descriptor_patch_stem_matches_conv2d(ops, case):
    b, c, h, w, n, (ky, kx), (sy, sx), (py, px), relu = case
    gen = torch.Generator().manual_seed(b + 10 * c + h + w + n)
    x = torch.randn(b, c, h, w, generator=gen)
    wgt = torch.randint(-1, 2, (n, c, ky, kx), generator=gen).float()
    scale = torch.rand(n, generator=gen) * 0.09 + 0.01
    bias = torch.randn(n, generator=gen)
    ref = nn.functional.conv2d(x.to(torch.bfloat16).double(), wgt.double(), None, (sy, sx), (py, px)) \
        * scale.double().view(1, -1, 1, 1) + bias.double().view(1, -1, 1, 1)
    if relu:
        ref = torch.relu(ref)
    packed = ops.compactify_ternary(wgt.cuda())
    rows = ops.conv_rows_stem(packed, c, ky, kx, sx)
    assert rows is not None
    y = ops.ternary_conv2d_stem_rows(x.cuda(), ops.prepack(rows, n, ops.FMT_BF16), n, (ky, kx), (sy, sx), (py, px),
                                     scale.cuda(), bias.cuda(), relu=relu)
    ops.check_gemm_status()
    assert y is not None
    got = y.permute(0, 3, 1, 2).double().cpu()
    assert got.shape == ref.shape
    tol = 2.0 ** -7 * ref.abs() + 1e-4 * ref.abs().max()
    bad = (got - ref).abs() > tol
    assert not bool(bad.any()), (int(bad.sum()), float((got - ref).abs().max()))


POOLED_STEM_CASES = [
    # b, c, h, w, (ky, kx), (sy, sx), (py, px): 64 output channels, even output height and width
    (2, 3, 224, 224, (7, 7), (2, 2), (3, 3)),        # the ResNet stem: 112 x 112 -> 56 x 56
    (5, 3, 64, 64, (7, 7), (2, 2), (3, 3)),          # several images per CTA range: image boundaries inside a chunk
    (300, 2, 12, 16, (3, 3), (2, 2), (1, 1)),        # 6 x 8 rows per image: chunks start inside images (recomputed halo row)
    (3, 4, 20, 24, (3, 3), (1, 2), (1, 1)),          # vertical stride 1: 20 x 12 -> 10 x 6
    (1, 3, 8, 8, (3, 3), (2, 2), (1, 1)),            # one tiny image, fewer rows than CTAs
]


@pytest.mark.parametrize("case", POOLED_STEM_CASES)
def test_pooled_stem_equals_stem_then_relu_then_maxpool(ops, case):
    """Convolution + ReLU + 3x3/2/1 max pooling in one kernel: bit-identical to the unfused kernels (stem without
    ReLU, then the pooling kernel with the ReLU folded in) and to torch's max_pool2d of the stem's bf16 output."""
    b, c, h, w, (ky, kx), (sy, sx), (py, px) = case
    n = 64
    gen = torch.Generator().manual_seed(b + c + h + w)
    x = torch.randn(b, c, h, w, generator=gen).cuda()
    wgt = torch.randint(-1, 2, (n, c, ky, kx), generator=gen).float()
    scale = (torch.rand(n, generator=gen) * 0.09 + 0.01).cuda()
    bias = torch.randn(n, generator=gen).cuda()
    rows = ops.conv_rows_stem(ops.compactify_ternary(wgt.cuda()), c, ky, kx, sx)
    wt = ops.prepack(rows, n, ops.FMT_BF16)
    plain = ops.ternary_conv2d_stem_rows(x, wt, n, (ky, kx), (sy, sx), (py, px), scale, bias, relu=False)
    fused = ops.ternary_conv2d_stem_rows(x, wt, n, (ky, kx), (sy, sx), (py, px), scale, bias, relu=True, pool=True)
    ops.check_gemm_status()
    assert plain is not None and fused is not None
    want = ops.maxpool2d_nhwc(plain, 3, 2, 1, relu=True)
    assert fused.shape == want.shape
    assert torch.equal(fused, want)
    ref = nn.functional.max_pool2d(torch.relu(plain.float()).permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)
    assert torch.equal(fused.float(), ref)


def test_pooled_stem_limits(ops):
    x = torch.randn(1, 3, 18, 18).cuda()                      # 9 x 9 output: odd
    wgt = torch.randint(-1, 2, (64, 3, 3, 3)).float()
    rows = ops.conv_rows_stem(ops.compactify_ternary(wgt.cuda()), 3, 3, 3, 2)
    wt = ops.prepack(rows, 64, ops.FMT_BF16)
    assert ops.ternary_conv2d_stem_rows(x, wt, 64, (3, 3), (2, 2), (1, 1), relu=True, pool=True) is None


def test_residual_fusion_and_patch_kernel(ops):
    gen = torch.Generator().manual_seed(77)
    # residual + ReLU inside the epilogue equals conv, then add, then ReLU
    x = torch.randn(2, 64, 10, 10, generator=gen).to(torch.bfloat16).cuda().permute(0, 2, 3, 1).contiguous()
    wgt = torch.randint(-1, 2, (64, 64, 3, 3), generator=gen).float()
    rows = ops.compactify_ternary(wgt.cuda()).view(64 * 9, -1)
    k = torch.arange(64 * 9)
    perm = torch.argsort((k % 9) * 64 + k // 9).cuda()
    wt = ops.prepack(rows.index_select(0, perm).contiguous(), 64, ops.FMT_BF16)
    scale = (torch.rand(64, generator=gen) * 0.05 + 0.01).cuda()
    res = torch.randn(2, 10, 10, 64, generator=gen).to(torch.bfloat16).cuda()
    plain = ops.ternary_conv2d_nhwc(x, wt, 64, (3, 3), (1, 1), (1, 1), (1, 1), scale)
    fused = ops.ternary_conv2d_nhwc(x, wt, 64, (3, 3), (1, 1), (1, 1), (1, 1), scale, relu=True, residual=res)
    want = torch.relu(plain.float() + res.float())
    assert (fused.float() - want).abs().max() <= 2.0 ** -6 * want.abs().max()
    # patch kernel against unfold
    img = torch.randn(3, 3, 20, 17, generator=gen).cuda()
    a, (b, oh, ow) = ops.conv_patches(img, (7, 7), (2, 2), (3, 3), (1, 1))
    unf = torch.nn.functional.unfold(img, (7, 7), padding=3, stride=2)            # [B, C*49, L], (c, ky, kx)
    ref = unf.view(3, 3, 49, -1).permute(0, 3, 2, 1).reshape(b * oh * ow, 147)      # -> (ky, kx, c)
    assert a.shape == (b * oh * ow, 152)
    assert torch.equal(a[:, :147], ref.to(torch.bfloat16)) and float(a[:, 147:].abs().max()) == 0.0
    # other geometries: row-staged kernel (unit dilation) and the generic one (dilation 2)
    for (c, h, w, k, s_, p_, d_) in [(4, 9, 33, (3, 3), (1, 1), (1, 1), (1, 1)), (3, 12, 10, (5, 3), (2, 3), (0, 1), (1, 1)),
                                     (2, 11, 13, (3, 3), (1, 1), (2, 2), (2, 2)), (1, 8, 8, (1, 1), (1, 1), (0, 0), (1, 1))]:
        img = torch.randn(2, c, h, w, generator=gen).cuda()
        a, (b, oh, ow) = ops.conv_patches(img, k, s_, p_, d_)
        unf = torch.nn.functional.unfold(img, k, dilation=d_, padding=p_, stride=s_)
        kk = k[0] * k[1]
        ref = unf.view(2, c, kk, -1).permute(0, 3, 2, 1).reshape(b * oh * ow, kk * c)
        assert torch.equal(a[:, :kk * c], ref.to(torch.bfloat16)), (c, h, w, k, s_, p_, d_)
        assert a.shape[1] == (kk * c + 7) // 8 * 8 and (a.shape[1] == kk * c or float(a[:, kk * c:].abs().max()) == 0.0)


@pytest.mark.parametrize("c,h,w,n,k,s,p", [(3, 40, 36, 64, 7, 2, 3), (3, 224, 224, 64, 7, 2, 3), (4, 17, 30, 72, 3, 1, 1),
                                           (1, 9, 128, 8, 5, 1, 2), (2, 12, 20, 136, 3, 2, 0)])
def test_fused_stem_convolution(c, h, w, n, k, s, p):
    """Few-channel convolution with the patches kept on chip, against torch conv2d on the bf16-rounded image (fp64) and
    against the explicit patch-matrix + GEMM route (same products, same k-block order)."""
    from tmq_b200 import ops
    gen = torch.Generator().manual_seed(c * 100 + n)
    wgt = torch.randint(-1, 2, (n, c, k, k), generator=gen).float()
    img = torch.randn(2, c, h, w, generator=gen)
    scale = torch.rand(n, generator=gen) * 0.05 + 0.01
    bias = torch.randn(n, generator=gen)
    rows = ops.compactify_ternary(wgt.cuda()).view(c * k * k, -1)                    # (c, ky, kx) order
    kk = torch.arange(c * k * k)
    perm = torch.argsort((kk % (k * k)) * c + kk // (k * k)).cuda()                   # -> (ky, kx, c)
    rows = rows.index_select(0, perm).contiguous()
    pad = (-rows.shape[0]) % 8
    if pad:
        rows = torch.nn.functional.pad(rows, (0, 0, 0, pad))
    wt = ops.prepack(rows, n, ops.FMT_BF16)
    y = ops.ternary_conv2d_stem(img.cuda(), wt, n, (k, k), (s, s), (p, p), scale.cuda(), bias.cuda(), relu=True)
    ops.check_gemm_status()
    assert y is not None and y.dtype == torch.bfloat16
    ref = torch.nn.functional.conv2d(img.to(torch.bfloat16).double(), wgt.double(), None, s, p)
    ref = torch.relu(ref * scale.double().view(1, -1, 1, 1) + bias.double().view(1, -1, 1, 1)).permute(0, 2, 3, 1)
    assert y.shape == ref.shape
    err = (y.cpu().double() - ref).abs()
    assert float(err.max()) <= 2.0 ** -7 * float(ref.abs().max()) + 1e-6            # one bf16 rounding of the output
    a, (b, oh, ow) = ops.conv_patches(img.cuda(), (k, k), (s, s), (p, p), (1, 1))
    via_patches = torch.relu(ops.ternary_gemm(a, wt, n, scale.cuda(), bias.cuda()).view(b, oh, ow, n))
    assert torch.equal(y, via_patches)


def test_qat_step_with_fused_optimizer_matches_adam_plus_clamp():
    """One QAT step of a small TMQ model with ops.MultiTensorAdam (clamp fused in) against torch.optim.Adam followed by
    QuantizationControl.clamp, from identical initial states."""
    import copy
    import tmq_b200 as tmq
    from tmq_b200 import workloads
    torch.manual_seed(3)
    net = torch.nn.Sequential(torch.nn.Linear(48, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10)).cuda()
    ctrl = tmq.QuantizationControl(epoch_knots=tmq.QuantizationScheduleBuilder.default_schedule(50),
                                   qpenalty_range=(0.0, 1e-3), device="cuda")
    tmq.quantize_model(net, ctrl)
    for e in range(1, 30):
        ctrl.step(e)
    with torch.no_grad():
        for node in ctrl._registry.values():
            node.weight.mul_(1.3)                      # some weights beyond the clamp range
    net_b = copy.deepcopy(net)                        # copies the controller along with the layers that hold it
    ctrl_b = next(m for m in net_b.modules() if isinstance(m, tmq.TMQLayer))._ctrl
    assert ctrl_b is not ctrl and len(ctrl_b._registry) == len(ctrl._registry)
    x = torch.randn(32, 48, device="cuda")
    y = torch.randint(0, 10, (32,), device="cuda")
    net.train(); net_b.train()
    opt_a = torch.optim.Adam(net.parameters(), lr=1e-2)
    opt_b = workloads.fused_optimizer(net_b, ctrl_b, lr=1e-2)
    for _ in range(3):
        la = workloads.qat_step(net, ctrl, opt_a, x, y)[0]
        lb = workloads.qat_step(net_b, ctrl_b, opt_b, x, y)[0]
        assert abs(float(la) - float(lb)) <= 1e-5 * max(1.0, abs(float(la)))
    for pa, pb in zip(net.parameters(), net_b.parameters()):
        assert torch.allclose(pa, pb, rtol=1e-5, atol=1e-6)
    for node in ctrl_b._registry.values():
        assert float(node.weight.detach().min()) >= -1.0 and float(node.weight.detach().max()) <= 1.0


def test_maxpool_nhwc_matches_torch():
    from tmq_b200 import ops
    gen = torch.Generator().manual_seed(3)
    for (b, h, w, c, k, s, p) in [(2, 13, 11, 64, 3, 2, 1), (1, 8, 8, 8, 2, 2, 0), (3, 7, 9, 24, 3, 1, 1)]:
        x = torch.randn(b, h, w, c, generator=gen).to(torch.bfloat16).cuda()
        want = torch.nn.functional.max_pool2d(x.permute(0, 3, 1, 2).float(), k, s, p).permute(0, 2, 3, 1).to(torch.bfloat16)
        assert torch.equal(ops.maxpool2d_nhwc(x, k, s, p), want.contiguous())
        assert torch.equal(ops.maxpool2d_nhwc(x, k, s, p, relu=True), torch.relu(want).contiguous())


def test_resnet18_qat_step_runs_and_clamps():
    from tmq_b200 import workloads
    torch.manual_seed(0)
    model, ctrl = workloads.build_resnet18(101)
    assert len(ctrl._registry) == 21 and sum(n.weight.numel() for n in ctrl._registry.values()) == 11218624
    model.cuda().train()
    for e in range(1, 45):
        ctrl.step(e)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    x = torch.randn(8, 3, 64, 64, device="cuda")
    y = torch.randint(0, 101, (8,), device="cuda")
    w_before = model.layer1[0].conv1.weight.detach().clone()
    loss, ce, ql = workloads.qat_step(model, ctrl, opt, x, y)
    assert torch.isfinite(loss) and ql.item() > 0
    w_after = model.layer1[0].conv1.weight.detach()
    assert not torch.equal(w_before, w_after)
    for node in ctrl._registry.values():
        assert float(node.weight.min()) >= -1.0 and float(node.weight.max()) <= 1.0
