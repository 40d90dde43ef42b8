"""The Python API end to end on the GPU: the MLP QAT step of the baseline configuration against the reference's CPU
run (golden: mlp_step.npz), compact inference of Linear / Conv2d layers against F.linear / F.conv2d on the expanded
weights, and the compressed state-dict round trip."""
import io

import numpy as np
import pytest
import torch
from torch import nn

from oracle import softstep as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tmq():
    import tmq_b200
    return tmq_b200


def _mlp():
    return nn.Sequential(nn.Linear(256, 128), nn.BatchNorm1d(128), nn.ReLU(), nn.Linear(128, 10), nn.BatchNorm1d(10))


@pytest.mark.parametrize("tag,epochs", [("warm", [5]), ("late", list(range(1, 45)))])
def test_mlp_qat_step_matches_reference(tmq, gold_mlp, tag, epochs):
    G = gold_mlp
    model = _mlp()
    ctrl = tmq.QuantizationControl(epoch_knots=tmq.QuantizationScheduleBuilder.default_schedule(50),
                                   qpenalty_range=(0.0, 1e-3))
    tmq.quantize_model(model, ctrl)
    init = {k[len(tag) + 6:]: torch.from_numpy(G[k]) for k in G.files if k.startswith(f"{tag}_init/")}
    model.load_state_dict(init)
    model.cuda()
    for e in epochs:
        ctrl.step(e)
    assert ctrl.digamma == float(G[f"{tag}_digamma"]) and ctrl.qpenalty == float(G[f"{tag}_qpenalty"])
    x, y = torch.from_numpy(G[f"{tag}_x"]).cuda(), torch.from_numpy(G[f"{tag}_y"]).cuda()
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    model.train()
    opt.zero_grad()
    logits = model(x)
    ce = nn.functional.cross_entropy(logits, y)
    ql = ctrl.quantization_loss()
    (ce + ql).backward()
    np.testing.assert_allclose(logits.detach().cpu().numpy(), G[f"{tag}_logits"], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(ce.item(), float(G[f"{tag}_ce"]), rtol=1e-5)
    np.testing.assert_allclose(ql.item(), float(G[f"{tag}_qloss"]), rtol=1e-5, atol=1e-12)
    for n, p in model.named_parameters():
        key = f"{tag}_grad/{n}"
        if key in G.files:
            ref = G[key]
            scale = np.abs(ref).max() + 1e-12
            # a bias in front of a BatchNorm has a mathematically zero gradient: only rounding noise, hence the floor
            assert np.abs(p.grad.cpu().numpy() - ref).max() <= 2e-4 * scale + 1e-8, n
    opt.step()
    ctrl.clamp()
    post = {k[len(tag) + 6:]: G[k] for k in G.files if k.startswith(f"{tag}_post/")}
    for k, v in model.state_dict().items():
        if v.dtype.is_floating_point:
            # Adam's first step moves every weight by about lr; a sign flip of a near-zero gradient costs 2*lr
            assert np.abs(v.cpu().numpy() - post[k]).max() <= 2.5e-3, k
    for name in ("0.weight", "3.weight"):
        w = model.state_dict()[name]
        assert float(w.min()) >= -1.0 and float(w.max()) <= 1.0
        close = np.abs(w.cpu().numpy() - post[name]) <= 1e-5
        assert close.mean() > 0.999, name


def test_all_layer_loss_equals_per_layer_losses_and_oracle(tmq):
    torch.manual_seed(1)
    model = nn.Sequential(nn.Conv2d(3, 8, 3), nn.Conv2d(8, 16, 3), nn.Flatten(), nn.Linear(16, 5))
    ctrl = tmq.QuantizationControl(epoch_knots=(15, 40, 43, 46, 50), qpenalty_range=(0.0, 1e-3))
    tmq.quantize_model(model, ctrl)
    model.cuda()
    fused = ctrl.quantization_loss(7e-4)
    per_layer = sum(node.quantization_loss(7e-4, ctrl.qpenalty_sharpness) for node in ctrl._registry.values())
    ref = sum(O.qloss_sum_f64(n.weight.detach().cpu().numpy(), 5.0, 7e-4) / n.weight.numel()
              for n in ctrl._registry.values())
    assert abs(fused.item() - ref) <= 1e-6 * abs(ref) and abs(per_layer.item() - ref) <= 1e-6 * abs(ref)
    fused.backward()
    for node in ctrl._registry.values():
        w = node.weight.detach().cpu().numpy()
        ginv = np.full(w.shape, np.float32(1.0) / np.float32(w.size), dtype=np.float32)
        want = O.deriv_backward(w, ginv, 5.0, 7e-4)
        assert np.array_equal(node.weight.grad.cpu().numpy().view(np.uint32), want.view(np.uint32))
    before = [n.weight.detach().clone() * 1.7 for n in ctrl._registry.values()]
    with torch.no_grad():
        for n, b in zip(ctrl._registry.values(), before):
            n.weight.copy_(b)
    ctrl.clamp(slack=0.25)
    for n, b in zip(ctrl._registry.values(), before):
        assert torch.equal(n.weight.detach(), torch.clamp(b, -1.25, 1.25))


def _small_convnet():
    return nn.Sequential(nn.Conv2d(3, 16, 3, padding=1, bias=False), nn.BatchNorm2d(16), nn.ReLU(),
                         nn.Conv2d(16, 40, 3, stride=2, padding=1, bias=True), nn.ReLU(),
                         nn.Conv2d(40, 24, 1, stride=2, bias=False), nn.AdaptiveAvgPool2d(1), nn.Flatten(),
                         nn.Linear(24, 11))


def _ternary_reference_model(tmq, seed):
    torch.manual_seed(seed)
    model = _small_convnet()
    ctrl = tmq.QuantizationControl()               # no schedule -> inference mode, weights used as they are
    tmq.quantize_model(model, ctrl)
    with torch.no_grad():
        for node in ctrl._registry.values():
            node.weight.mul_(1.4)
            if getattr(node, "bias", None) is not None:
                node.bias.normal_()
    tmq.quantize_weights(model)
    with torch.no_grad():
        for node in ctrl._registry.values():
            node.weight.clamp_(-1, 1)
    model.cuda().eval()
    return model, ctrl


@pytest.mark.parametrize("strong", [False, True])
def test_compressed_state_dict_roundtrip_and_compact_inference(tmq, strong):
    model, ctrl = _ternary_reference_model(tmq, 3)
    x = torch.randn(6, 3, 20, 20, device="cuda")
    with torch.no_grad():
        want = model(x)                           # F.conv2d / F.linear on the fp32 ternary weights
    state = tmq.compressed_state_dict(model, strong=strong)
    for name, node in ctrl._registry.items():
        assert node.compact and node.weight.dtype == torch.int32 and not node.training
    key = "0.weight"
    assert state[key].dtype == (torch.int8 if strong else torch.int32)
    assert state._metadata["0"]["tmq.tensor_type"] == (3 if strong else 2)
    assert tuple(state._metadata["0"]["tmq.shape"]) == (16, 3, 3, 3) and state._metadata["0"]["tmq.quant"] == 1
    with torch.no_grad():
        got = model(x)                            # packed weights, tensor-core GEMM, exact fp32 split
    scale = want.abs().max()
    assert (got - want).abs().max() <= 1e-5 * scale
    # through a file and into a fresh model
    buf = io.BytesIO()
    torch.save(state, buf)
    buf.seek(0)
    loaded = torch.load(buf, weights_only=False)
    fresh = _small_convnet()
    tmq.quantize_model(fresh, tmq.QuantizationControl())
    tmq.load_compressed_state_dict(fresh, loaded)
    fresh.cuda().eval()
    with torch.no_grad():
        again = fresh(x)
    assert (again - want).abs().max() <= 1e-5 * scale
    # back to fp32 weights
    tmq.expand_compact_layers(fresh)
    with torch.no_grad():
        expanded = fresh(x)
    assert (expanded - want).abs().max() <= 1e-5 * scale


def test_linear_compact_forward_shapes_and_dtypes(tmq):
    torch.manual_seed(5)
    ctrl = tmq.QuantizationControl(post_scale=True)
    lin = tmq.Linear(200, 77, bias=True, ctrl=ctrl, quant_mode=tmq.QuantMode.TERNARY, post_scale=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randint(-1, 2, (77, 200)).float())
        lin.bias.normal_()
    holder = nn.Sequential(lin).cuda().eval()
    W, b, ps = lin.weight.detach().clone(), lin.bias.detach().clone(), lin.post_scale_imm
    tmq.compressed_state_dict(holder)
    for shape in [(200,), (1, 200), (9, 200), (2, 33, 200), (1, 1, 3, 200)]:
        x = torch.randn(*shape, device="cuda")
        want = ps * (x @ W.T) + b
        got = lin(x)
        assert got.shape == want.shape and got.dtype == torch.float32
        assert (got - want).abs().max() <= 2e-6 * want.abs().max()
    xb = torch.randn(40, 200, device="cuda").to(torch.bfloat16)
    got = lin(xb)
    want = (ps * (xb.float() @ W.T) + b)
    assert got.dtype == torch.bfloat16
    assert (got.float() - want).abs().max() <= 2 ** -7 * want.abs().max()
    xi = torch.randint(-127, 128, (5, 200), device="cuda", dtype=torch.int8)
    assert torch.equal(lin(xi), (xi.double() @ W.double().T).to(torch.int32))


def test_conv_geometries(tmq):
    torch.manual_seed(9)
    cases = [(3, 64, 7, 2, 3, 1, 32), (64, 64, 3, 1, 1, 1, 14), (64, 128, 1, 2, 0, 1, 14), (8, 24, 3, 2, 1, 1, 9),
             (5, 7, (3, 2), (1, 2), (1, 0), 1, 11), (4, 6, 3, 1, 2, 2, 12)]
    for (cin, cout, k, s, p, d, hw) in cases:
        conv = tmq.Conv2d(cin, cout, k, stride=s, padding=p, dilation=d, bias=False, ctrl=tmq.QuantizationControl(),
                          quant_mode=tmq.QuantMode.TERNARY)
        with torch.no_grad():
            conv.weight.copy_(torch.randint(-1, 2, conv.weight.shape).float())
        holder = nn.Sequential(conv).cuda().eval()
        W = conv.weight.detach().clone()
        x = torch.randn(3, cin, hw, hw + 1, device="cuda")
        want = nn.functional.conv2d(x.double(), W.double(), None, s, p, d).float()   # fp64: cuDNN fp32 may use TF32
        tmq.compressed_state_dict(holder)
        got = conv(x)
        assert got.shape == want.shape
        assert (got - want).abs().max() <= 1e-5 * want.abs().max(), (cin, cout, k, s, p, d)
