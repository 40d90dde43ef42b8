"""The numpy oracle must reproduce the reference's PyTorch-CPU-eager results bit for bit (golden: softstep.npz)."""
import numpy as np
import torch

from conftest import bits
from oracle import softstep as O
from oracle import softstep_torch as OT


def test_forward_backward_bit_exact(gold_softstep):
    G = gold_softstep
    w, g = G["w"], G["g"]
    s = float(G["strength"])
    for i, d in enumerate(G["digammas"].tolist()):
        assert np.array_equal(bits(O.forward(w, d)), bits(G[f"fwd_{i}"])), d
        assert np.array_equal(bits(O.backward(w, g, d, 1.0)), bits(G[f"bwd_{i}"])), d
        assert np.array_equal(bits(O.deriv_forward(w, d, s)), bits(G[f"dfwd_{i}"])), d
        assert np.array_equal(bits(O.deriv_backward(w, g, d, s)), bits(G[f"dbwd_{i}"])), d


def test_known_answers():
    # fp32 hex known answers of the reference's eager path
    w = np.array([-1.25, -0.25, 0.25, 0.75, 1.25], dtype=np.float32)
    y1 = O.forward(w, 1.0)
    assert [float(v).hex() for v in y1] == ["-0x1.3c8c880000000p+0", "-0x1.e464480000000p-3", "0x1.e464480000000p-3",
                                            "0x1.86e6ee0000000p-1", "0x1.3c8c880000000p+0"]
    d1 = O.backward(w, np.ones(5, np.float32), 1.0)
    assert all(float(v).hex() == "0x1.0409b80000000p+0" for v in d1)
    mid = O.backward(np.array([0.5, -0.5, 1.5], np.float32), np.ones(3, np.float32), 6.0)
    assert all(float(v) == 3.0 for v in mid)
    at_int = O.backward(np.array([0.0, 1.0, -1.0], np.float32), np.ones(3, np.float32), 6.0)
    assert all(float(v) == 0.0 for v in at_int)


def test_loss_and_clamp(gold_softstep):
    G = gold_softstep
    w = G["w"]
    n = w.size
    s = float(G["strength"])
    mean = O.qloss_sum_f64(w, 5.0, s) / n
    assert abs(mean - float(G["qloss_mean"])) <= 1e-6 * abs(float(G["qloss_mean"]))
    ginv = np.full(n, np.float32(1.0) / np.float32(n), dtype=np.float32)
    assert np.array_equal(bits(O.deriv_backward(w, ginv, 5.0, s)), bits(G["qloss_grad"]))
    assert np.array_equal(bits(O.clamp(w, -1.0, 1.0)), bits(G["clamp"]))
    assert np.array_equal(bits(O.clamp(w, -1.25, 1.25)), bits(G["clamp_slack"]))


def test_torch_baseline_matches_numpy_oracle(gold_softstep):
    G = gold_softstep
    w, g = G["w"], G["g"]
    y, grad, wc, loss = OT.qat_element_pass(torch.from_numpy(w.copy()), torch.from_numpy(g.copy()), 0.9, 5.0, 5e-4,
                                            -1.0, 1.0)
    ye, ge, wce, ls = O.fused_step(w, g, 0.9, 5.0, 5e-4, -1.0, 1.0)
    assert np.array_equal(bits(y.numpy()), bits(ye))
    assert np.array_equal(bits(grad.numpy()), bits(ge))
    assert np.array_equal(bits(wc.numpy()), bits(wce))
    assert abs(float(loss) - ls / w.size) <= 1e-6 * abs(ls / w.size)


def test_nan_inf_propagate():
    w = np.array([np.nan, np.inf, -np.inf], dtype=np.float32)
    assert np.isnan(O.forward(w, 1.0)).all()
    assert np.isnan(O.backward(w, np.ones(3, np.float32), 1.0)).all()
