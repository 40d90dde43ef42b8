"""Host-side behaviour of the Python API that needs no GPU: the schedule (against the reference's trace), module
surgery, registry naming, argument checks."""
import numpy as np
import pytest
import torch
from torch import nn

import tmq_b200 as tmq


def test_public_names():
    for name in ["QuantMode", "TensorType", "QuantizationScheduleBuilder", "QuantizationControl", "SoftStep",
                 "SoftStepDerivative", "TMQLayer", "Linear", "Conv2d", "ConvTranspose2d", "quantize_weights",
                 "quantize_model", "compressed_state_dict", "prepare_compressed_load", "load_compressed_state_dict",
                 "expand_compact_layers", "CUDA_EXT_AVAILABLE", "NATIVE_EXT_AVAILABLE"]:
        assert hasattr(tmq, name), name
    assert tmq.TensorType.COMPRESSED_TERNARY_32BIT.value == 3 and tmq.QuantMode.EIGHT_BIT.value == 8


def test_default_schedule():
    assert tmq.QuantizationScheduleBuilder.default_schedule(50) == (15, 40, 43, 46, 50)
    assert tmq.QuantizationScheduleBuilder.default_schedule(150) == (45, 120, 131, 139, 150)
    with pytest.raises(AssertionError):
        tmq.QuantizationScheduleBuilder.default_schedule(20)


@pytest.mark.parametrize("tag,epochs,qp", [("e50", 50, (0.0, 1e-3)), ("e150", 150, (1e-4, 2e-3))])
def test_schedule_trace_matches_reference(gold_schedule, tag, epochs, qp):
    knots = tmq.QuantizationScheduleBuilder.default_schedule(epochs)
    assert list(knots) == gold_schedule[f"{tag}_knots"].tolist()
    ctrl = tmq.QuantizationControl(epoch_knots=knots, qpenalty_range=qp)
    dg, qpn = [], []
    for e in range(1, epochs + 1):
        ctrl.step(e)
        dg.append(ctrl.digamma)
        qpn.append(ctrl.qpenalty)
    assert np.array_equal(np.array(dg), gold_schedule[f"{tag}_digamma"])
    assert np.array_equal(np.array(qpn), gold_schedule[f"{tag}_qpenalty"])


def test_controller_argument_checks():
    with pytest.raises(AssertionError):
        tmq.QuantizationControl(digamma_range=(0.01, 6))
    with pytest.raises(AssertionError):
        tmq.QuantizationControl(digamma_range=(0.1, 25))
    with pytest.raises(AssertionError):
        tmq.QuantizationControl(epoch_knots=(5, 40, 43, 46, 50))
    c = tmq.QuantizationControl()
    assert c.inference_mode and c.clamp_values == (-1.0, 1.0) and c.qpenalty == 0 and c.qpenalty_sharpness == 5.0
    c.step(3)                                    # no schedule: a no-op
    assert c.digamma == 0.1


def test_quantize_model_swaps_layers_and_names_them_like_the_reference():
    torch.manual_seed(0)
    model = nn.Sequential()
    model.add_module("conv1", nn.Conv2d(3, 8, 3, padding=1, bias=False))
    block = nn.Sequential()
    block.add_module("conv", nn.Conv2d(8, 8, 3, padding=1))
    block.add_module("up", nn.ConvTranspose2d(8, 4, 2, stride=2))
    model.add_module("layer1", block)
    model.add_module("skipme", nn.Linear(4, 4))
    model.add_module("fc", nn.Linear(4, 2))
    ctrl = tmq.QuantizationControl(epoch_knots=(15, 40, 43, 46, 50))
    tmq.quantize_model(model, ctrl, exclude=["skipme"])
    assert isinstance(model.conv1, tmq.Conv2d) and isinstance(model.layer1.conv, tmq.Conv2d)
    assert isinstance(model.layer1.up, tmq.ConvTranspose2d) and isinstance(model.fc, tmq.Linear)
    assert type(model.skipme) is nn.Linear
    assert sorted(ctrl._registry) == sorted([".conv1", "layer1.conv", "layer1.up", ".fc"])
    w = model.conv1.weight
    assert w.shape == (8, 3, 3, 3) and float(w.min()) >= -1.0 and float(w.max()) < 1.0
    assert model.conv1.bias is None and torch.count_nonzero(model.layer1.conv.bias) == 0
    assert model.layer1.up.weight.shape == (8, 4, 2, 2)
    # wildcard exclusion
    m2 = nn.Sequential(nn.Linear(4, 4), nn.Sequential(nn.Linear(4, 4)))
    tmq.quantize_model(m2, tmq.QuantizationControl(), prefix="model", exclude=["*1.0"])
    assert isinstance(m2[0], tmq.Linear) and type(m2[1][0]) is nn.Linear


def test_cpu_tensors_are_refused_loudly():
    ctrl = tmq.QuantizationControl(epoch_knots=(15, 40, 43, 46, 50))
    lin = tmq.Linear(8, 4, ctrl=ctrl, quant_mode=tmq.QuantMode.TERNARY)
    lin.train()
    with pytest.raises(RuntimeError, match="CUDA"):
        lin(torch.randn(2, 8))
    ctrl.register_node("x", lin)
    with pytest.raises(RuntimeError, match="CUDA"):
        ctrl.quantization_loss()
