"""Tensor-core ternary GEMM (tcgen05) against the oracle: int8 activations bit-exact; bf16 activations within
rel 1e-3 of the fp64 result before output rounding (fp32 output), and within one bf16 ulp after it (bf16 output)."""
import numpy as np
import pytest
import torch

from oracle import ternary as T

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


def make_weights(N, K, seed, p=(0.3, 0.4, 0.3)):
    rng = np.random.default_rng(seed)
    u = rng.random((N, K))
    W = np.where(u < p[0], -1.0, np.where(u < p[0] + p[1], 0.0, 1.0)).astype(np.float32)
    return W, T.pack(W)


SHAPES = [(1, 128, 64), (8, 128, 64), (32, 256, 128), (33, 200, 192), (64, 128, 256), (100, 130, 72), (128, 384, 512),
          (129, 128, 64), (256, 256, 1024), (300, 520, 576), (512, 1000, 2304)]


PATHS = ["tiles", "gemv"]


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_i8_exact(ops, M, N, K, path):
    if path == "gemv" and M > 40:
        pytest.skip("the skinny kernels are meant for skinny problems")
    K = (K + 15) // 16 * 16
    W, P = make_weights(N, K, M * 7 + N)
    rng = np.random.default_rng(K)
    X = rng.integers(-127, 128, (M, K)).astype(np.int8)
    wt = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_I8)
    Y = ops.ternary_gemm_i8(torch.from_numpy(X).cuda(), wt, N, path=path)
    ops.check_gemm_status()
    assert np.array_equal(Y.cpu().numpy(), T.gemm_i8_fast(X, P, N))


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_bf16_tolerance(ops, M, N, K, path):
    if path == "gemv" and M > 40:
        pytest.skip("the skinny kernels are meant for skinny problems")
    K = (K + 7) // 8 * 8
    W, P = make_weights(N, K, M * 11 + N)
    gen = torch.Generator().manual_seed(K)
    X = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    scale = (torch.rand(N, generator=gen) * 0.09 + 0.01)
    bias = torch.randn(N, generator=gen)
    wt = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_BF16)
    ref_acc = T.gemm_f64_fast(X.float().numpy(), P, N)                       # exact sum of exact products
    ref = ref_acc * scale.double().numpy()[None, :] + bias.double().numpy()[None, :]
    y32 = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), bias.cuda(), out_dtype=torch.float32, path=path)
    ops.check_gemm_status()
    got = y32.cpu().double().numpy()
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(got - ref) <= 1e-3 * np.maximum(np.abs(ref), rms)), np.abs(got - ref).max()
    # in practice fp32 accumulation of exact products is far tighter than the 1e-3 bar
    assert np.all(np.abs(got - ref) <= 1e-5 * np.maximum(np.abs(ref), rms))
    y16 = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), bias.cuda(), out_dtype=torch.bfloat16, path=path)
    ops.check_gemm_status()
    want16 = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
    ulp = np.abs(want16) * 2.0 ** -7                     # one bf16 ulp, plus the fp32 accumulation slack near zero
    assert np.all(np.abs(y16.cpu().float().numpy() - want16) <= ulp + 1e-5 * rms)


def test_gemm_no_scale_bias_matches_reference_semantics(ops):
    """scale = 1, bias = 0 reproduces the reference kernel's plain X.T product (tmq/tmq_cuda.cu:289-427)."""
    M, N, K = 64, 128, 128
    W, P = make_weights(N, K, 5)
    X = torch.randint(-4, 5, (M, K)).to(torch.bfloat16)            # small integers: every partial sum is exact
    wt = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_BF16)
    y = ops.ternary_gemm(X.cuda(), wt, N, out_dtype=torch.float32)
    ops.check_gemm_status()
    assert np.array_equal(y.cpu().numpy(), T.gemm_f32_seq(X.float().numpy(), P, N))


def test_prepack_is_layout_only(ops):
    """Prepacking twice gives the same words, and both formats decode to the same matrix (checked through GEMMs with
    one-hot activations, which read out single weight columns exactly)."""
    N, K = 144, 128
    W, P = make_weights(N, K, 9)
    Pd = torch.from_numpy(P).cuda()
    a, b = ops.prepack(Pd, N, ops.FMT_BF16), ops.prepack(Pd, N, ops.FMT_BF16)
    assert torch.equal(a, b)
    eye16 = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    eye8 = torch.eye(K, dtype=torch.int8, device="cuda")
    t16 = ops.ternary_gemm(eye16, a, N, out_dtype=torch.float32)                   # [K, N] = T^T
    t8 = ops.ternary_gemm_i8(eye8, ops.prepack(Pd, N, ops.FMT_I8), N)
    ops.check_gemm_status()
    assert np.array_equal(t16.cpu().numpy(), W.T)
    assert np.array_equal(t8.cpu().numpy(), W.T.astype(np.int32))


def test_gemm_argument_checks(ops):
    wt = torch.zeros((128, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError):
        ops.ternary_gemm(torch.zeros((4, 64), dtype=torch.float32, device="cuda"), wt, 128)
    with pytest.raises(RuntimeError):
        ops.ternary_gemm(torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda"), wt, 128)   # K mismatch
    with pytest.raises(RuntimeError):                                                             # K % 8 != 0
        ops.ternary_gemm(torch.zeros((4, 60), dtype=torch.bfloat16, device="cuda"), wt, 128)


@pytest.mark.parametrize("M", [1, 8, 32])
def test_gemv_baseline_shape(ops, M):
    """BASELINE decode-like config: N = 11008, K = 4096, weights at P = 0.3/0.4/0.3, per-channel scale in [0.01, 0.1],
    bf16 activations N(0,1) (rel 1e-3 before output rounding) and int8 activations in [-127, 127] (bit-exact)."""
    N, K = 11008, 4096
    W, P = make_weights(N, K, 0)
    Pd = torch.from_numpy(P).cuda()
    gen = torch.Generator().manual_seed(M)
    X = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    scale = torch.rand(N, generator=gen) * 0.09 + 0.01
    ref = T.gemm_f64_fast(X.float().numpy(), P, N) * scale.double().numpy()[None, :]
    wt = ops.prepack(Pd, N, ops.FMT_BF16)
    y = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), out_dtype=torch.float32)
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(y.cpu().double().numpy() - ref) <= 1e-3 * np.maximum(np.abs(ref), rms))
    assert np.all(np.abs(y.cpu().double().numpy() - ref) <= 1e-5 * np.maximum(np.abs(ref), rms))
    X8 = torch.randint(-127, 128, (M, K), generator=gen, dtype=torch.int8)
    y8 = ops.ternary_gemm_i8(X8.cuda(), ops.prepack(Pd, N, ops.FMT_I8), N)
    assert np.array_equal(y8.cpu().numpy(), T.gemm_i8_fast(X8.numpy(), P, N))
    # deterministic: same bits on a second run
    y2 = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), out_dtype=torch.float32)
    for pth in ("gemv", "tiles"):
        yo = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), out_dtype=torch.float32, path=pth)
        assert np.all(np.abs(yo.cpu().double().numpy() - ref) <= 1e-5 * np.maximum(np.abs(ref), rms)), pth
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M,N,K", [(1, 11000, 4096), (2, 2368, 4096), (3, 4096, 11008), (8, 1000, 1088),
                                   (1, 16, 64), (2, 40, 16384), (1, 12000, 16384), (5, 200, 40000)])
def test_gemv_resident_and_streaming_forms(ops, M, N, K):
    """The skinny kernels in both forms: rows resident in shared memory (byte dot products for int8 with M <= 2, warp
    MMA otherwise; channel counts that are no multiple of 16 or of the CTA count) and, where one SM's share of the
    rows exceeds the shared-memory budget or no status word is passed, the streaming kernels."""
    import ctypes
    from tmq_b200 import _lib
    W, P = make_weights(N, K, N + K + M)
    Pd = torch.from_numpy(P).cuda()
    rng = np.random.default_rng(M)
    X8 = rng.integers(-127, 128, (M, K)).astype(np.int8)
    want8 = T.gemm_i8_fast(X8, P, N)
    wt8 = ops.prepack(Pd, N, ops.FMT_I8)
    y8 = ops.ternary_gemm_i8(torch.from_numpy(X8).cuda(), wt8, N, path="gemv")
    ops.check_gemm_status()
    assert np.array_equal(y8.cpu().numpy(), want8)
    # no status word: the streaming kernel, same bits
    x8d = torch.from_numpy(X8).cuda()
    y8s = torch.empty((M, N), dtype=torch.int32, device="cuda")
    rc = _lib.lib().tmq_ternary_gemv_i8(x8d.data_ptr(), wt8.data_ptr(), y8s.data_ptr(), M, N, K, N, None,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    assert np.array_equal(y8s.cpu().numpy(), want8)
    X = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    scale = torch.from_numpy((rng.random(N) * 0.09 + 0.01).astype(np.float32))
    bias = torch.from_numpy(rng.standard_normal(N).astype(np.float32))
    ref = T.gemm_f64_fast(X.float().numpy(), P, N) * scale.double().numpy()[None, :] + bias.double().numpy()[None, :]
    y = ops.ternary_gemm(X.cuda(), ops.prepack(Pd, N, ops.FMT_BF16), N, scale.cuda(), bias.cuda(),
                         out_dtype=torch.float32, path="gemv")
    ops.check_gemm_status()
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(y.cpu().double().numpy() - ref) <= 1e-5 * np.maximum(np.abs(ref), rms))


def test_full_size_prefill_shape_sampled(ops):
    """BASELINE prefill config (M = 8192, K = 8192, N = 28672) at full size: a random 96 x 96 sample of the outputs
    against fp64 dot products of the same operands (bf16 path: rel 1e-3 bar, 1e-5 expected; int8 path: bit-exact), plus
    one size-independent property: activations with a single one per row read out weight columns exactly."""
    M, K, N = 8192, 8192, 28672
    gen = torch.Generator(device="cuda").manual_seed(0)
    u = torch.rand(N, K, generator=gen, device="cuda")
    W = torch.where(u < 0.3, -1.0, torch.where(u < 0.7, 0.0, 1.0))
    del u
    P = ops.compactify_ternary(W)
    scale = torch.rand(N, generator=gen, device="cuda") * 0.09 + 0.01
    X = torch.randn(M, K, generator=gen, device="cuda").to(torch.bfloat16)
    Y = ops.ternary_gemm(X, ops.prepack(P, N, ops.FMT_BF16), N, scale, out_dtype=torch.float32)
    ops.check_gemm_status()
    rows = torch.randint(0, M, (96,), generator=gen, device="cuda")
    cols = torch.randint(0, N, (96,), generator=gen, device="cuda")
    ref = (X[rows].double() @ W[cols].double().T) * scale[cols].double()
    got = Y[rows][:, cols].double()
    rms = ref.pow(2).mean().sqrt()
    assert bool(((got - ref).abs() <= 1e-5 * torch.maximum(ref.abs(), rms)).all())
    del Y
    X8 = torch.randint(-127, 128, (M, K), generator=gen, device="cuda", dtype=torch.int8)
    wt8 = ops.prepack(P, N, ops.FMT_I8)
    Y8 = ops.ternary_gemm_i8(X8, wt8, N)
    ops.check_gemm_status()
    ref8 = (X8[rows].double() @ W[cols].double().T).to(torch.int32)
    assert torch.equal(Y8[rows][:, cols], ref8)
    del Y8, X8
    # one-hot rows: Y[i] = column k_i of T, exactly
    ks = torch.randint(0, K, (256,), generator=gen, device="cuda")
    E = torch.zeros(256, K, dtype=torch.int8, device="cuda")
    E[torch.arange(256, device="cuda"), ks] = 1
    out = ops.ternary_gemm_i8(E, wt8, N, path="tiles")
    assert torch.equal(out, W[:, ks].T.to(torch.int32))


@pytest.mark.parametrize("n0,width", [(0, 256), (3, 256), (8, 200), (5, 203)])
@pytest.mark.parametrize("M", [8, 100])
def test_gemm_bf16_writes_a_column_block_of_a_wider_output(ops, M, n0, width):
    """Y = base + n0 with ldy = the full width: the 16-byte vector stores are only legal when that address is 16-byte
    aligned and ldy % 8 == 0; every other combination must take the scalar stores and still give the same bits as the
    plain call, without touching the columns outside the block."""
    N, K = 72, 192
    W, P = make_weights(N, K, 31)
    gen = torch.Generator().manual_seed(n0 * 7 + width)
    X = torch.randn(M, K, generator=gen).to(torch.bfloat16).cuda()
    wt = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_BF16)
    plain = ops.ternary_gemm(X, wt, N)
    wide = torch.full((M, width), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.ternary_gemm(X, wt, N, out=wide[:, n0:n0 + N])
    ops.check_gemm_status()
    assert torch.equal(wide[:, n0:n0 + N], plain)
    assert bool((wide[:, :n0] == 7.0).all()) and bool((wide[:, n0 + N:] == 7.0).all())


# Batched skinny form: several matrices of one shape in one launch.  Shapes cover the separate and the overlaid
# reduction area (rows + reduction beyond the shared-memory budget at M = 8 on the decode shape), ragged channel counts
# (N % 16 != 0, fewer 16-channel groups than SMs), an odd and an even number of matrices, and more than one launch's
# worth of matrices.
BATCHED = [(1, 11008, 4096, 3), (2, 11008, 4096, 2), (8, 11008, 4096, 2), (5, 1000, 1088, 5), (1, 520, 256, 1),
           (1, 4096, 4096, 18), (3, 2368, 512, 4)]


@pytest.mark.parametrize("shared", [True, False])
@pytest.mark.parametrize("M,N,K,nmat", BATCHED)
def test_gemv_batched_i8_exact(ops, M, N, K, nmat, shared):
    rng = np.random.default_rng(N + K + nmat)
    X = rng.integers(-127, 128, (M, K) if shared else (nmat, M, K)).astype(np.int8)
    packed = [make_weights(N, K, 31 * j + M)[1] for j in range(nmat)]
    wts = [ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_I8) for P in packed]
    Y = ops.ternary_gemv_batched(torch.from_numpy(X).cuda(), wts, N)
    ops.check_gemm_status()
    for j in range(nmat):
        assert np.array_equal(Y[j].cpu().numpy(), T.gemm_i8_fast(X if shared else X[j], packed[j], N)), j


@pytest.mark.parametrize("shared", [True, False])
@pytest.mark.parametrize("M,N,K,nmat", BATCHED)
def test_gemv_batched_bf16_matches_oracle_and_the_one_matrix_kernel(ops, M, N, K, nmat, shared):
    gen = torch.Generator().manual_seed(N + K + nmat)
    X = torch.randn((M, K) if shared else (nmat, M, K), generator=gen).to(torch.bfloat16)
    packed = [make_weights(N, K, 17 * j + M)[1] for j in range(nmat)]
    wts = [ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_BF16) for P in packed]
    scales = [torch.rand(N, generator=gen) * 0.09 + 0.01 if j % 2 == 0 else None for j in range(nmat)]
    biases = [torch.randn(N, generator=gen) if j % 3 != 1 else None for j in range(nmat)]
    Xc = X.cuda()
    Y = ops.ternary_gemv_batched(Xc, wts, N, scales, biases, out_dtype=torch.float32)
    ops.check_gemm_status()
    for j in range(nmat):
        xj = X if shared else X[j]
        acc = T.gemm_f64_fast(xj.float().numpy(), packed[j], N)
        ref = acc * (scales[j].double().numpy()[None, :] if scales[j] is not None else 1.0)
        if biases[j] is not None:
            ref = ref + biases[j].double().numpy()[None, :]
        got = Y[j].double().cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max(), j
        one = ops.ternary_gemm(Xc if shared else Xc[j], wts[j], N, scales[j], biases[j], torch.float32, path="gemv")
        # same products; the K slices are summed by 8 warps here and 16 there, so only fp32 summation order differs
        assert float((one - Y[j]).abs().max()) <= 2e-6 * float(one.abs().max()), j


def test_gemv_batched_argument_checks(ops):
    N, K = 64, 128
    wt = ops.prepack(torch.from_numpy(make_weights(N, K, 1)[1]).cuda(), N, ops.FMT_BF16)
    x = torch.zeros(9, K, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.ternary_gemv_batched(x, [wt], N)                       # more than 8 rows
    with pytest.raises(RuntimeError):
        ops.ternary_gemv_batched(x[:2].reshape(2, 1, K), [wt], N)  # two activation blocks, one matrix
    assert ops.ternary_gemv_batched(x[:1], [], N) == []


@pytest.mark.parametrize("M,N,K,ldy,off", [(300, 256, 1024, 512, 128), (1000, 520, 576, 520, 0), (100, 256, 1024, 256, 0),
                                           (8192, 1024, 2048, 4096, 1024), (513, 130, 640, 130, 0)])
def test_gemm_bcast_writes_every_destination(ops, M, N, K, ldy, off):
    """The all-gather form of the GEMM on one GPU: the same column block goes into several buffers (here all local;
    across GPUs they are peer mappings).  Tall, vector-friendly shapes take the kernel that parks the tile and writes
    whole rows; the others the ordinary epilogue.  Every destination must equal the plain GEMM, other columns untouched."""
    W, P = make_weights(N, K, M + N)
    gen = torch.Generator().manual_seed(K)
    X = torch.randn(M, K, generator=gen).to(torch.bfloat16).cuda()
    scale = (torch.rand(N, generator=gen) * 0.09 + 0.01).cuda()
    bias = torch.randn(N, generator=gen).cuda()
    wt = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_BF16)
    want = ops.ternary_gemm(X, wt, N, scale, bias, path="tiles")
    bufs = [torch.full((M, ldy), 7.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    ops.ternary_gemm_bcast(X, wt, N, [b.data_ptr() + off * 2 for b in bufs], ldy, scale, bias)
    ops.check_gemm_status()
    for b in bufs:
        assert torch.equal(b[:, off:off + N], want)
        rest = torch.cat([b[:, :off], b[:, off + N:]], dim=1)
        assert bool((rest == 7.0).all())


# Skinny problems with fewer output tiles than SMs: K is split over several CTAs per tile and a second kernel sums the
# partial results in split order (ops takes that route on its own whenever the C library reports a workspace size).
SPLIT_K = [(64, 4096, 4096), (17, 1000, 2048), (100, 2304, 1024), (256, 640, 8192), (1, 512, 4096)]


@pytest.mark.parametrize("M,N,K", SPLIT_K)
def test_split_k_gemm_matches_oracle(ops, M, N, K):
    from tmq_b200 import _lib
    assert _lib.lib().tmq_ternary_gemm_workspace_bytes(M, N, K, 0) > 0          # these shapes are split
    W, P = make_weights(N, K, M + N + K)
    rng = np.random.default_rng(K + M)
    X8 = rng.integers(-127, 128, (M, K)).astype(np.int8)
    wt8 = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_I8)
    Y8 = ops.ternary_gemm_i8(torch.from_numpy(X8).cuda(), wt8, N, path="tiles")
    assert np.array_equal(Y8.cpu().numpy(), T.gemm_i8_fast(X8, P, N))
    gen = torch.Generator().manual_seed(K)
    X = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    scale = torch.rand(N, generator=gen) * 0.09 + 0.01
    bias = torch.randn(N, generator=gen)
    wt = ops.prepack(torch.from_numpy(P).cuda(), N, ops.FMT_BF16)
    ref = T.gemm_f64_fast(X.float().numpy(), P, N) * scale.double().numpy()[None, :] + bias.double().numpy()[None, :]
    y32 = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), bias.cuda(), out_dtype=torch.float32, path="tiles")
    ybf = ops.ternary_gemm(X.cuda(), wt, N, scale.cuda(), bias.cuda(), out_dtype=torch.bfloat16, path="tiles")
    ops.check_gemm_status()
    assert np.abs(y32.double().cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    assert torch.equal(ybf, y32.to(torch.bfloat16))
