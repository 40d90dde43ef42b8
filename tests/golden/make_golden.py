"""Generates the committed golden fixtures by RUNNING THE REFERENCE on CPU.

Needs the reference checkout (its path in the environment variable TMQ_REFERENCE_DIR) and the compiled reference
extension oracle/_ref/tmq_native.so (python oracle/build_ref.py).  Run from the repository root:

    TMQ_REFERENCE_DIR=<path to the mtnwrw/tmq checkout> python tests/golden/make_golden.py

Outputs (all small, committed):
  softstep.npz   reference tmq.SoftStep / SoftStepDerivative forward+backward (PyTorch CPU eager) on seeded inputs
  schedule.npz   QuantizationControl.step traces
  pack.npz       compactify_ternary / expand_ternary known answers (2-D, 4-D, ragged, int inputs)
  codec.npz      compress_ternary / decompress_ternary streams
  mlp_step.npz   the reference MLP QAT step (logits, loss, grads, post-step weights)
  resnet_qat_step.npz   the reference ResNet-18 (101 classes) QAT step on CPU, batch 8 of 64 x 64 images: logits, loss
                 terms, gradients of three layers (parameters are filled from one seeded generator in state_dict order,
                 so the fixture does not have to carry the 45 MB of initial weights)
"""
import contextlib
import io
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
REFERENCE = os.environ.get("TMQ_REFERENCE_DIR")
assert REFERENCE and os.path.isdir(REFERENCE), "set TMQ_REFERENCE_DIR to the reference checkout"
OUT = os.path.dirname(os.path.abspath(__file__))

from oracle import build_ref  # noqa: E402

build_ref.build_native()
native = build_ref.load_native()
assert native is not None, "oracle/_ref/tmq_native.so missing"
# make the reference package see its own compiled native helper, exactly as an installed copy would
sys.modules["tmq.tmq_native"] = native
sys.path.insert(0, REFERENCE)
with contextlib.redirect_stdout(io.StringIO()):
    import tmq as ref  # noqa: E402
assert ref.NATIVE_EXT_AVAILABLE and not ref.CUDA_EXT_AVAILABLE

DIGAMMAS = [0.05, 0.1, 0.4625, 0.5, 0.9, 1.0, 1.35, 3.0, 4.8, 5.0, 6.0, 10.0, 20.0]


class _Ctrl:
    def __init__(self, d):
        self.digamma = d


def softstep_inputs(n, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.rand(n, generator=g) * 3.0 - 1.5
    # sprinkle the awkward points: integers, half-integers, tiny values, just-below-integer values, signed zero
    special = torch.tensor([0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 1.5, -1.5, 2.0, -2.0, 1e-8, -1e-8, 1e-30, -1e-30,
                            0.99999994, -0.99999994, 1.0000001, -1.0000001, 0.49999997, 0.50000006,
                            3.75, -3.75, 100.25, -100.25, 1e6 + 0.5, -1e6 - 0.5], dtype=torch.float32)
    w[: special.numel()] = special
    grad = torch.randn(n, generator=g)
    return w, grad


def make_softstep():
    n = 8192
    w, g = softstep_inputs(n, 20250101)
    out = {"w": w.numpy(), "g": g.numpy(), "digammas": np.array(DIGAMMAS, dtype=np.float64),
           "strength": np.float64(5e-4)}
    for i, d in enumerate(DIGAMMAS):
        ctrl = _Ctrl(d)
        wp = w.clone().requires_grad_(True)
        y = ref.SoftStep.apply(wp, 1.0, ctrl)
        y.backward(g)
        out[f"fwd_{i}"] = y.detach().numpy()
        out[f"bwd_{i}"] = wp.grad.numpy()
        wq = w.clone().requires_grad_(True)
        o = ref.SoftStepDerivative.apply(wq, d, 5e-4)
        o.backward(g)
        out[f"dfwd_{i}"] = o.detach().numpy()
        out[f"dbwd_{i}"] = wq.grad.numpy()
    # layer loss exactly as Linear.quantization_loss composes it (mean + autograd), sharpness 5.0
    wl = w.clone().requires_grad_(True)
    loss = torch.mean(ref.SoftStepDerivative.apply(wl, 5.0, 5e-4))
    loss.backward()
    out["qloss_mean"] = loss.detach().numpy()
    out["qloss_grad"] = wl.grad.numpy()
    out["clamp"] = torch.clamp(w, -1.0, 1.0).numpy()
    out["clamp_slack"] = torch.clamp(w, -1.0 - 0.25, 1.0 + 0.25).numpy()
    np.savez_compressed(os.path.join(OUT, "softstep.npz"), **out)


def make_schedule():
    out = {}
    for tag, epochs, qp in (("e50", 50, (0.0, 1e-3)), ("e150", 150, (1e-4, 2e-3))):
        knots = ref.QuantizationScheduleBuilder.default_schedule(epochs)
        ctrl = ref.QuantizationControl(epoch_knots=knots, qpenalty_range=qp)
        dg, qpn = [], []
        for e in range(1, epochs + 1):
            ctrl.step(e)
            dg.append(ctrl.digamma)
            qpn.append(ctrl.qpenalty)
        out[f"{tag}_knots"] = np.array(knots)
        out[f"{tag}_digamma"] = np.array(dg, dtype=np.float64)
        out[f"{tag}_qpenalty"] = np.array(qpn, dtype=np.float64)
    np.savez_compressed(os.path.join(OUT, "schedule.npz"), **out)


def make_pack_and_codec():
    g = torch.Generator().manual_seed(1234)
    lin = torch.randint(-1, 2, (37, 50), generator=g).float()
    conv = torch.randint(-1, 2, (20, 3, 3, 3), generator=g).float()
    soft = (torch.rand(33, 47, generator=g) * 3.0 - 1.5)            # needs rounding + clamping
    soft[0, :8] = torch.tensor([0.5, -0.5, 1.5, -1.5, 0.49999997, -0.49999997, 2.5, -2.5])
    wide = torch.randint(-1, 2, (130, 64), generator=g).float()
    conv1x1 = torch.randint(-1, 2, (48, 16, 1, 1), generator=g).float()
    ints = torch.randint(-3, 4, (19, 21), generator=g, dtype=torch.int32)
    bytes_ = torch.randint(-3, 4, (17, 40), generator=g, dtype=torch.int32).to(torch.int8)
    pk, cd = {}, {}
    for name, t in (("lin", lin), ("conv", conv), ("soft", soft), ("wide", wide), ("conv1x1", conv1x1),
                    ("ints", ints), ("bytes", bytes_)):
        p = native.compactify_ternary(t.contiguous())
        pk[f"{name}_in"] = t.numpy()
        pk[f"{name}_packed"] = p.numpy()
        if t.dim() == 4:
            pk[f"{name}_expanded"] = native.expand_ternary(p, list(t.shape), False).numpy()
        if t.dtype == torch.float32:
            c_plain = native.compress_ternary(t.contiguous(), list(t.shape), False)
            c_compact = native.compress_ternary(p, list(t.shape), True)
            assert torch.equal(c_plain, c_compact)
            back = native.decompress_ternary(c_plain, list(t.shape))
            assert torch.equal(back, p)
            cd[f"{name}_shape"] = np.array(t.shape)
            cd[f"{name}_packed"] = p.numpy()
            cd[f"{name}_stream"] = c_plain.numpy()
    # a skewed and a larger matrix for the coder
    u = torch.rand(333, 200, generator=g)
    skew = torch.where(u < 0.05, -1.0, torch.where(u < 0.9, 0.0, 1.0))
    big = torch.where(u < 0.3, -1.0, torch.where(u < 0.7, 0.0, 1.0))
    for name, t in (("skew", skew), ("big", big)):
        p = native.compactify_ternary(t.contiguous())
        c = native.compress_ternary(p, list(t.shape), True)
        assert torch.equal(native.decompress_ternary(c, list(t.shape)), p)
        cd[f"{name}_shape"] = np.array(t.shape)
        cd[f"{name}_packed"] = p.numpy()
        cd[f"{name}_stream"] = c.numpy()
    np.savez_compressed(os.path.join(OUT, "pack.npz"), **pk)
    np.savez_compressed(os.path.join(OUT, "codec.npz"), **cd)


def make_mlp_step():
    """BASELINE config 1: the reference MLP QAT step on CPU (README usage pattern, tmq/tmq.py:85-310)."""
    from torch import nn
    ref.Linear.forward = ref.Linear.forward_wrap          # skip the debug dump to /tmp (tmq/tmq.py:624-635)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 128), nn.BatchNorm1d(128), nn.ReLU(), nn.Linear(128, 10), nn.BatchNorm1d(10))
    knots = ref.QuantizationScheduleBuilder.default_schedule(50)
    out = {}
    for tag, epoch_seq in (("warm", [5]), ("late", list(range(1, 45)))):
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(256, 128), nn.BatchNorm1d(128), nn.ReLU(), nn.Linear(128, 10),
                              nn.BatchNorm1d(10))
        ctrl = ref.QuantizationControl(epoch_knots=knots, qpenalty_range=(0.0, 1e-3))
        ref.quantize_model(model, ctrl)
        g = torch.Generator().manual_seed(7)
        x = torch.randn(256, 256, generator=g)
        y = torch.randint(0, 10, (256,), generator=g)
        for e in epoch_seq:
            ctrl.step(e)
        init = {k: v.detach().clone().numpy() for k, v in model.state_dict().items()}
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
        model.train()
        opt.zero_grad()
        logits = model(x)
        ce = nn.functional.cross_entropy(logits, y)
        ql = ctrl.quantization_loss()
        loss = ce + ql
        loss.backward()
        grads = {n: p.grad.detach().clone().numpy() for n, p in model.named_parameters() if p.grad is not None}
        opt.step()
        ctrl.clamp()
        post = {k: v.detach().clone().numpy() for k, v in model.state_dict().items()}
        out[f"{tag}_x"] = x.numpy()
        out[f"{tag}_y"] = y.numpy()
        out[f"{tag}_digamma"] = np.float64(ctrl.digamma)
        out[f"{tag}_qpenalty"] = np.float64(ctrl.qpenalty)
        out[f"{tag}_logits"] = logits.detach().numpy()
        out[f"{tag}_ce"] = ce.detach().numpy()
        out[f"{tag}_qloss"] = ql.detach().numpy()
        for k, v in init.items():
            out[f"{tag}_init/{k}"] = v
        for k, v in grads.items():
            out[f"{tag}_grad/{k}"] = v
        for k, v in post.items():
            out[f"{tag}_post/{k}"] = v
    np.savez_compressed(os.path.join(OUT, "mlp_step.npz"), **out)


def seeded_fill(model, seed):
    """Deterministic parameters and buffers, independent of either implementation's own initialisation: every
    state_dict entry, in key order, from one generator.  Quantized layers' weights U(-1.2, 1.2) (some outside the clamp
    range), BatchNorm scale U(0.5, 1.5), everything else small.  tests/test_conv_api_gpu.py repeats this on the GPU side."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for key, t in model.state_dict().items():
            if not t.is_floating_point() or key.endswith("post_scale"):
                continue
            if key.endswith("running_var"):
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            elif key.endswith("running_mean"):
                t.copy_(torch.randn(t.shape, generator=g) * 0.1)
            elif t.dim() >= 2:
                t.copy_(torch.rand(t.shape, generator=g) * 2.4 - 1.2)
            elif "bn" in key.split(".")[-2] and key.endswith("weight"):
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            elif key.endswith("weight") and t.dim() == 1:
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            else:
                t.copy_(torch.randn(t.shape, generator=g) * 0.1)


RESNET_GRAD_LAYERS = ("conv1.weight", "layer1.0.conv1.weight", "layer2.0.downsample.0.weight", "fc.weight")


def make_resnet_qat_step():
    """BASELINE config 4a at test size: torchvision ResNet-18 (101 classes), every conv / fc layer quantized, the
    sample's fc set-up (samples/resnet_train.py:344-358), one forward + CE + quantization loss + backward on CPU."""
    import torchvision
    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=101)
    knots = ref.QuantizationScheduleBuilder.default_schedule(50)
    ctrl = ref.QuantizationControl(epoch_knots=knots, qpenalty_range=(0.0, 1e-3))
    with contextlib.redirect_stdout(io.StringIO()):
        ref.quantize_model(model, ctrl)
    model.fc.disable_bias()
    model.fc.implicit_bn()
    ref.Linear.forward = ref.Linear.forward_wrap
    seeded_fill(model, 4242)
    for e in range(1, 45):
        ctrl.step(e)
    g = torch.Generator().manual_seed(99)
    x = torch.randn(8, 3, 64, 64, generator=g)
    y = torch.randint(0, 101, (8,), generator=g)
    model.train()
    logits = model(x)
    ce = torch.nn.functional.cross_entropy(logits, y)
    ql = ctrl.quantization_loss()
    (ce + ql).backward()
    params = dict(model.named_parameters())
    out = {"x": x.numpy(), "y": y.numpy(), "digamma": np.float64(ctrl.digamma), "qpenalty": np.float64(ctrl.qpenalty),
           "logits": logits.detach().numpy(), "ce": ce.detach().numpy(), "qloss": ql.detach().numpy(),
           "n_registered": np.int64(len(ctrl._registry))}
    for name in RESNET_GRAD_LAYERS:
        out["grad/" + name] = params[name].grad.detach().numpy()
    ctrl.clamp()
    out["clamped/layer1.0.conv1.weight"] = params["layer1.0.conv1.weight"].detach().numpy()
    np.savez_compressed(os.path.join(OUT, "resnet_qat_step.npz"), **out)


if __name__ == "__main__":
    torch.set_num_threads(1)
    make_softstep()
    make_schedule()
    make_pack_and_codec()
    make_mlp_step()
    make_resnet_qat_step()
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(OUT, f)))
