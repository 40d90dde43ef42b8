"""Fused quantisation-aware Linear forward (soft staircase evaluated inside the tensor-core GEMM's operand producers)
against the oracle: Y = X . S(W)^T + b with S the oracle's bit-exact fp32 staircase, the sum formed in fp64.
Bar: the two-term bf16 split carries S to 2^-17 relative and accumulation is fp32, so |error| <= 1e-5 * max|Y| (the
north-star bound for floating-point GEMMs is rel 1e-3).  The layer-level test checks that the module route gives the
gradients of SoftStep.apply + F.linear."""
import numpy as np
import pytest
import torch

from oracle import softstep as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


def reference(x_bf16, w, b, d):
    S = O.forward(w, d).astype(np.float64)
    y = x_bf16.float().double().numpy() @ S.T
    return y if b is None else y + b.astype(np.float64)[None, :]


# (M, N, K): one tile, ragged rows / channels / K tail, both activation-tile widths (M <= 128 and M > 128), several
# tiles per CTA (more tiles than SMs) so that the stage ring and the accumulator hand-over wrap many times
SHAPES = [(1, 128, 64), (7, 100, 72), (128, 256, 512), (129, 130, 200), (300, 384, 1000), (64, 4096, 1024),
          (520, 5000, 328)]


@pytest.mark.parametrize("d", [1.0, 4.0, 6.5, 40.0])
@pytest.mark.parametrize("M,N,K", SHAPES[:5])
def test_fused_forward_matches_oracle(ops, M, N, K, d):
    rng = np.random.default_rng(M + N + K)
    w = (rng.random((N, K), dtype=np.float32) * 3.0 - 1.5).astype(np.float32)
    w[0, :8] = [0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 1.4999999, -1.5]           # steps, mid-points, range ends
    b = rng.standard_normal(N).astype(np.float32)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    y = ops.qat_linear_forward(x.cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda(), d)
    ops.check_gemm_status()
    ref = reference(x, w, b, d)
    assert y.shape == (M, N) and y.dtype == torch.float32
    assert np.abs(y.double().cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("M,N,K", SHAPES[5:])
def test_fused_forward_many_tiles(ops, M, N, K):
    rng = np.random.default_rng(N)
    w = (rng.random((N, K), dtype=np.float32) * 2.5 - 1.25).astype(np.float32)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    y = ops.qat_linear_forward(x.cuda(), torch.from_numpy(w).cuda(), None, 5.0)
    ops.check_gemm_status()
    ref = reference(x, w, None, 5.0)
    assert np.abs(y.double().cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()


def test_fused_forward_equals_elementwise_staircase_then_matmul(ops):
    """The producers evaluate the same staircase as the elementwise kernel: with activations that pick single weights
    (one-hot rows) the result is S(w) itself, up to the 2^-17 relative split."""
    rng = np.random.default_rng(3)
    N, K = 256, 128
    w = torch.from_numpy((rng.random((N, K), dtype=np.float32) * 3.0 - 1.5).astype(np.float32)).cuda()
    x = torch.eye(K, dtype=torch.bfloat16, device="cuda")
    y = ops.qat_linear_forward(x, w, None, 7.0)                 # [K, N] = S(w)^T
    s = ops.fwd_softstep(w, 7.0)
    assert float((y.t() - s).abs().max()) <= 2.0 ** -16 * float(s.abs().max())


def test_fused_forward_leading_dimensions_and_checks(ops):
    w = torch.zeros(64, 128, device="cuda")
    x = torch.zeros(2, 3, 128, dtype=torch.bfloat16, device="cuda")
    assert ops.qat_linear_forward(x, w, None, 2.0).shape == (2, 3, 64)
    with pytest.raises(RuntimeError):
        ops.qat_linear_forward(x.float(), w, None, 2.0)
    with pytest.raises(RuntimeError):
        ops.qat_linear_forward(x[..., :100].contiguous(), w[:, :100].contiguous(), None, 2.0)   # K % 8 != 0
    with pytest.raises(RuntimeError):
        ops.qat_linear_forward(x, w, None, 1e9)                                                   # hardness out of range


def test_layer_route_and_gradients(ops):
    """tmq.Linear in training mode with bf16 activations takes the fused kernel; loss and gradients agree with the
    unfused route (SoftStep.apply + F.linear on the same bf16-representable activations in fp32)."""
    from tmq_b200 import tmq
    torch.manual_seed(5)
    ctrl = tmq.QuantizationControl(epoch_knots=(15, 40, 43, 46, 50), device="cuda")
    ctrl.digamma = 3.0
    layer = tmq.Linear(256, 192, True, ctrl=ctrl, device="cuda", quant_mode=tmq.QuantMode.TERNARY)
    layer.train()
    with torch.no_grad():
        layer.bias.copy_(torch.randn(192, device="cuda"))
    x = torch.randn(40, 256, device="cuda").to(torch.bfloat16)
    xa = x.clone().requires_grad_(True)
    ya = layer(xa)
    assert ya.dtype == torch.float32
    ga = torch.randn_like(ya)
    ya.backward(ga)
    ya = ya.detach()
    gw_a, gb_a, gx_a = layer.weight.grad.clone(), layer.bias.grad.clone(), xa.grad.clone()
    layer.weight.grad = None
    layer.bias.grad = None
    xb = x.float().requires_grad_(True)
    yb = layer(xb)                                   # fp32 activations: staircase kernel + F.linear
    yb.backward(ga)
    yb = yb.detach()
    assert float((ya - yb).abs().max()) <= 1e-4 * float(yb.abs().max())
    assert float((gw_a - layer.weight.grad).abs().max()) <= 1e-4 * float(layer.weight.grad.abs().max())
    assert float((gb_a - layer.bias.grad).abs().max()) <= 1e-5 * float(layer.bias.grad.abs().max())
    assert float((gx_a.float() - xb.grad).abs().max()) <= 1e-2 * float(xb.grad.abs().max())   # gx is rounded to bf16
