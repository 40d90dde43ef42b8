"""Parity of the CUDA soft-step kernels (through the C ABI) with the oracle and the reference-generated fixtures.
Bar: bit-exact fp32 for every elementwise output; rel 1e-9 for the fp64 loss sum against the fp64 sum of the
bit-exact integrand (reduction order is the only freedom), rel 1e-6 against the reference's fp32 torch.mean."""
import numpy as np
import pytest
import torch

from conftest import bits
from oracle import softstep as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same_bits(t, ref):
    got = bits(t.detach().cpu().numpy())
    want = bits(ref)
    nan = np.isnan(ref)
    ok = (got == want) | (nan & np.isnan(t.detach().cpu().numpy()))
    return bool(ok.all())


def test_golden_all_digammas(ops, gold_softstep):
    G = gold_softstep
    w, g = dev(G["w"]), dev(G["g"])
    s = float(G["strength"])
    for i, d in enumerate(G["digammas"].tolist()):
        assert same_bits(ops.fwd_softstep(w, d), G[f"fwd_{i}"]), d
        assert same_bits(ops.bwd_softstep(w, d, 1.0, g), G[f"bwd_{i}"]), d
        assert same_bits(ops.fwd_softstep_derivative(w, d, s), G[f"dfwd_{i}"]), d
        assert same_bits(ops.bwd_softstep_derivative(w, d, s, g), G[f"dbwd_{i}"]), d
    assert same_bits(ops.clamp(w, -1.0, 1.0), G["clamp"])
    assert same_bits(ops.clamp(w, -1.25, 1.25), G["clamp_slack"])
    mean = float(ops.qloss_sum(w, 5.0, s).item()) / w.numel()
    assert abs(mean - float(G["qloss_mean"])) <= 1e-6 * abs(float(G["qloss_mean"]))


def test_const_div_fast_path_is_exact(ops):
    for d in (0.05, 0.1, 0.5, 0.9, 1.0, 2.275, 5.0, 6.0, 20.0):
        assert ops.selftest_const_div(d) == 0, d


def test_ranged_division_is_exact(ops):
    # every denominator of the nine binades against 4096 pseudo-random numerators each (3e11 quotients) ...
    assert ops.selftest_div(4096) == 0
    # ... and a slab of 2048 denominators per binade against EVERY numerator mantissa (1.5e11 quotients)
    for binade in range(9):
        assert ops.selftest_div(1 << 23, (binade << 23) + 12345 * (binade + 1), 2048) == 0, binade


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 255, 1023, 4096, 4097, 1 << 20, (1 << 20) + 7])
def test_sizes_and_tails(ops, n):
    rng = np.random.default_rng(n)
    w = (rng.random(n, dtype=np.float32) * 3 - 1.5).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    d = 0.9
    wd, gd = dev(w), dev(g)
    assert same_bits(ops.fwd_softstep(wd, d), O.forward(w, d))
    assert same_bits(ops.bwd_softstep(wd, d, 1.0, gd), O.backward(w, g, d))
    assert same_bits(ops.fwd_softstep_derivative(wd, 5.0, 1e-3), O.deriv_forward(w, 5.0, 1e-3))
    assert same_bits(ops.bwd_softstep_derivative(wd, 5.0, 1e-3, gd), O.deriv_backward(w, g, 5.0, 1e-3))
    assert same_bits(ops.clamp(wd, -1, 1), O.clamp(w, -1, 1))
    if n:
        s = float(ops.qloss_sum(wd, 5.0, 1e-3).item())
        ref = O.qloss_sum_f64(w, 5.0, 1e-3)
        assert abs(s - ref) <= 2.5e-7 * abs(ref)      # fp32 partial sums of 4 terms inside a vector


def test_unaligned_views_take_the_scalar_path(ops):
    rng = np.random.default_rng(5)
    base = (rng.random(10001, dtype=np.float32) * 3 - 1.5).astype(np.float32)
    wd = dev(base)[1:]                      # 4-byte aligned only
    assert wd.data_ptr() % 16 != 0
    assert same_bits(ops.fwd_softstep(wd, 1.35), O.forward(base[1:], 1.35))


@pytest.mark.parametrize("d", [0.1, 0.5, 0.9, 1.0, 3.0, 6.0, 10.0])
def test_fused_step_matches_composition(ops, d):
    n = (1 << 18) + 3
    gen = torch.Generator().manual_seed(0)
    w = (torch.rand(n, generator=gen) * 3 - 1.5)
    g = torch.randn(n, generator=gen)
    y, gw, wc, loss = ops.fused_step(w.cuda(), g.cuda(), d, 5.0, 5e-4, -1.0, 1.0)
    ye, ge, wce, ls = O.fused_step(w.numpy(), g.numpy(), d, 5.0, 5e-4, -1.0, 1.0)
    assert same_bits(y, ye)
    assert same_bits(gw, ge)
    assert same_bits(wc, wce)
    assert abs(float(loss.item()) - ls) <= 1e-9 * abs(ls)


def test_fused_step_zero_strength_and_repeatable(ops):
    n = 100000
    gen = torch.Generator().manual_seed(1)
    w = (torch.rand(n, generator=gen) * 3 - 1.5).cuda()
    g = torch.randn(n, generator=gen).cuda()
    y, gw, wc, loss = ops.fused_step(w, g, 6.0, 5.0, 0.0, -1.0, 1.0)
    ye, ge, wce, ls = O.fused_step(w.cpu().numpy(), g.cpu().numpy(), 6.0, 5.0, 0.0, -1.0, 1.0)
    assert same_bits(gw, ge) and float(loss.item()) == 0.0
    a = ops.fused_step(w, g, 0.9, 5.0, 5e-4, -1.0, 1.0)[3].item()
    b = ops.fused_step(w, g, 0.9, 5.0, 5e-4, -1.0, 1.0)[3].item()
    assert a == b                              # deterministic reduction, scratch re-armed by the kernel


def test_nan_inf_inputs(ops):
    w = np.array([np.nan, np.inf, -np.inf, 0.25, -0.0, 7.5, -7.5, 1e30], dtype=np.float32)
    g = np.ones_like(w)
    wd, gd = dev(w), dev(g)
    assert same_bits(ops.fwd_softstep(wd, 1.0), O.forward(w, 1.0))
    assert same_bits(ops.bwd_softstep(wd, 1.0, 1.0, gd), O.backward(w, g, 1.0))
    assert same_bits(ops.clamp(wd, -1, 1), O.clamp(w, -1, 1))


def test_full_size_properties(ops):
    """BASELINE size (2^26 elements): properties that need no CPU replay of the whole tensor."""
    n = 1 << 26
    gen = torch.Generator(device="cuda").manual_seed(0)
    w = torch.rand(n, generator=gen, device="cuda") * 3 - 1.5
    g = torch.randn(n, generator=gen, device="cuda")
    d = 0.9
    y, gw, wc, loss = ops.fused_step(w, g, d, 5.0, 5e-4, -1.0, 1.0)
    # (1) the fusion equals the separate kernels bit for bit
    assert torch.equal(y, ops.fwd_softstep(w, d))
    gq = torch.full((1,), 1.0, device="cuda") / torch.full((1,), float(n), device="cuda")
    g2 = ops.bwd_softstep_derivative(w, 5.0, 5e-4, gq.expand(n))
    assert torch.equal(gw, ops.bwd_softstep(w, d, 1.0, g) + g2)
    assert torch.equal(wc, torch.clamp(w, -1.0, 1.0))
    # (2) the staircase maps integer+u to integer+s(u): shifting the input by one shifts the output by one
    sub = w[: 1 << 20]
    assert torch.equal(ops.fwd_softstep(torch.floor(sub) + 0.25, d), torch.floor(sub) + ops.fwd_softstep(
        torch.full_like(sub, 0.25), d))
    # (3) loss: fused sum == fp64 sum of the materialised integrand; mean close to strength (integral of S' is 1)
    o = ops.fwd_softstep_derivative(w, 5.0, 5e-4)
    ref = o.double().sum().item()
    assert abs(loss.item() - ref) <= 1e-9 * abs(ref)
    assert abs(loss.item() / n - 5e-4) < 5e-6
    # (4) a random 1M sample is bit-exact against the oracle
    idx = torch.randint(0, n, (1 << 20,), generator=gen, device="cuda")
    ws, gs = w[idx].cpu().numpy(), g[idx].cpu().numpy()
    assert same_bits(y[idx], O.forward(ws, d))
    assert same_bits(ops.bwd_softstep(w, d, 1.0, g)[idx], O.backward(ws, gs, d))


def test_multi_tensor_forms(ops):
    gen = torch.Generator().manual_seed(3)
    shapes = [(64, 3, 7, 7), (64, 64, 3, 3), (101, 512), (5,), (4097,)]
    ws = [(torch.rand(s, generator=gen) * 3 - 1.5).cuda() for s in shapes]
    plan = ops.MultiTensorPlan(ws)
    loss = plan.qloss(5.0, 1e-3).item()
    ref = sum(O.qloss_sum_f64(w.cpu().numpy(), 5.0, 1e-3) / w.numel() for w in ws)
    assert abs(loss - ref) <= 2.5e-7 * abs(ref)
    up = torch.tensor(0.75, device="cuda")
    grads = plan.qloss_bwd(5.0, 1e-3, up)
    for w, gr in zip(ws, grads):
        wn = w.cpu().numpy()
        ginv = np.full(wn.shape, np.float32(0.75) / np.float32(wn.size), dtype=np.float32)
        assert same_bits(gr, O.deriv_backward(wn, ginv, 5.0, 1e-3))
    before = [w.clone() for w in ws]
    plan.clamp_(-1.0, 1.0)
    for w, b in zip(ws, before):
        assert torch.equal(w, torch.clamp(b, -1.0, 1.0))


def test_fused_step_host_matches_device_call():
    """The pipelined host-buffer entry point: elementwise outputs bit-equal to the device call, loss sum equal to fp64
    rounding (the chunks' sums are added in order), odd sizes and a chunk size that does not divide the length."""
    from tmq_b200 import ops
    gen = torch.Generator().manual_seed(11)
    for n, chunk in ((1 << 20) + 12345, 1 << 18), (70000, 1 << 16), (1 << 16, 1 << 20):
        hw = (torch.rand(n, generator=gen) * 3 - 1.5).pin_memory()
        hg = torch.randn(n, generator=gen).pin_memory()
        hy, hgw, hwc = (torch.empty(n).pin_memory() for _ in range(3))
        for d in (0.5, 3.0):
            loss = ops.fused_step_host(hw, hg, hy, hgw, hwc, d, 5.0, 5e-4, -1.0, 1.0, chunk_elems=chunk)
            y, gw, wc, want = ops.fused_step(hw.cuda(), hg.cuda(), d, 5.0, 5e-4, -1.0, 1.0)
            assert torch.equal(hy, y.cpu()) and torch.equal(hgw, gw.cpu()) and torch.equal(hwc, wc.cpu())
            assert abs(loss - float(want.item())) <= 1e-12 * abs(float(want.item()))


def test_multi_tensor_adam_with_clamp_matches_torch_adam():
    """Fused Adam + clamp over several tensors (ragged sizes) against torch.optim.Adam on the CPU followed by
    torch.clamp, six steps with fresh gradients each: parameters and both moments to a few fp32 ulps."""
    from tmq_b200 import ops
    gen = torch.Generator().manual_seed(5)
    shapes = [(64, 33), (128,), (7, 3, 3, 3), (4099,), (1,)]
    ref = [torch.nn.Parameter(torch.rand(s, generator=gen) * 2.4 - 1.2) for s in shapes]
    dev = [torch.nn.Parameter(p.detach().clone().cuda()) for p in ref]
    opt_ref = torch.optim.Adam(ref, lr=0.05, betas=(0.9, 0.999), eps=1e-8, foreach=False)
    clamp_idx = (0, 2, 3)
    opt = ops.MultiTensorAdam(dev, lr=0.05, betas=(0.9, 0.999), eps=1e-8, clamp_params=[dev[i] for i in clamp_idx],
                              clamp=(-1.0, 1.0))
    for step in range(6):
        grads = [torch.randn(s, generator=gen) * (0.1 if step % 2 else 3.0) for s in shapes]
        opt.zero_grad()
        for p, q, g in zip(ref, dev, grads):
            p.grad = g.clone()
            q.grad.copy_(g)                                   # .grad views the flat buffer
        opt_ref.step()
        with torch.no_grad():
            for i in clamp_idx:
                ref[i].copy_(torch.clamp(ref[i], -1.0, 1.0))
        opt.step()
        for i, (p, q) in enumerate(zip(ref, dev)):
            assert torch.allclose(q.detach().cpu(), p.detach(), rtol=2e-6, atol=1e-7), (step, i)
    for i, p in enumerate(ref):
        st = opt_ref.state[p]
        a, b = opt.offsets[i], opt.offsets[i] + p.numel()
        assert torch.allclose(opt.exp_avg[a:b].cpu().view_as(p), st["exp_avg"], rtol=1e-5, atol=1e-6)     # O(1) values, cancellation
        assert torch.allclose(opt.exp_avg_sq[a:b].cpu().view_as(p), st["exp_avg_sq"], rtol=1e-5, atol=1e-9)
    for i in clamp_idx:
        assert float(dev[i].min()) >= -1.0 and float(dev[i].max()) <= 1.0
