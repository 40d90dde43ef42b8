"""CPU oracle for the soft-staircase transfer function (TEST INFRASTRUCTURE, not product code).

Restates, in numpy fp32 with one IEEE rounding per line, the PyTorch-CPU-eager branches of the
reference's autograd Functions:

  * forward         tmq/tmq.py:417-419  (SoftStep.forward, sigmoid at tmq/tmq.py:358-360)
  * backward        tmq/tmq.py:434-438  (SoftStep.backward, dsigmoid at tmq/tmq.py:368-370)
  * deriv forward   tmq/tmq.py:469-472  (SoftStepDerivative.forward)
  * deriv backward  tmq/tmq.py:488-492  (SoftStepDerivative.backward, d2sigmoid at tmq/tmq.py:378-381)
  * host scalars    tmq/tmq.py:384-391  (scalar_sigmoid, evaluated in Python doubles)
  * clamp           tmq/tmq.py:696, :879 (torch.clamp on the weights)
  * layer loss      tmq/tmq.py:698-699  (torch.mean of the derivative output)

Parity of this restatement is pinned by tests/golden/softstep_*.npz, which were produced by importing the
reference's own tmq.py on CPU (tests/golden/make_golden.py) and are compared bit for bit.

Only tests/, the smoke check and the cpu_baseline leg of bench.py may import this module.
"""
import numpy as np

F = np.float32


def scalar_sigmoid(v: float) -> float:
    """tmq/tmq.py:384-391 in Python doubles."""
    x = min(3.0, max(-3.0, v))
    x2 = x * x
    return x * (x2 + 27.0) / (27.0 + x2 * 9.0)


def host_scalars(digamma: float):
    """The three fp32 scalars every formula uses: d, d/2 and 2*sigma(d/2) (double math, then one cast)."""
    d32 = F(digamma)
    h32 = F(digamma / 2.0)
    D32 = F(2.0 * scalar_sigmoid(digamma / 2.0))
    return d32, h32, D32


def _arg(w, digamma):
    d32, h32, D32 = host_scalars(digamma)
    w = np.asarray(w, dtype=F)
    fw = np.floor(w)
    fr = w - fw
    t = d32 * fr
    a = t - h32
    # torch.clamp propagates NaN; np.clip does too
    x = np.clip(a, F(-3.0), F(3.0))
    x2 = x * x
    return fw, x, x2, d32, D32


def forward(w, digamma):
    with np.errstate(all="ignore"):
        fw, x, x2, d32, D32 = _arg(w, digamma)
        p = x2 + F(27.0)
        q = x * p
        r = x2 * F(9.0)
        s = F(27.0) + r
        z = q / s
        u = z / D32
        v = u + F(0.5)
        return (v + fw).astype(F)


def _dsig(x2):
    e = x2 - F(9.0)
    n = e * e
    b = F(3.0) + x2
    c = F(9.0) * b
    m = c * b
    return n / m


def backward(w, g, digamma, scale=1.0):
    with np.errstate(all="ignore"):
        fw, x, x2, d32, D32 = _arg(w, digamma)
        ds = _dsig(x2)
        k = d32 * ds
        G = k / D32
        gs = F(scale) * np.asarray(g, dtype=F)
        return (gs * G).astype(F)


def deriv_forward(w, digamma, strength):
    with np.errstate(all="ignore"):
        fw, x, x2, d32, D32 = _arg(w, digamma)
        ds = _dsig(x2)
        sd32 = F(strength * digamma)
        return ((sd32 * ds) / D32).astype(F)


def deriv_backward(w, g, digamma, strength):
    with np.errstate(all="ignore"):
        fw, x, x2, d32, D32 = _arg(w, digamma)
        A = x2 + F(3.0)
        i = F(16.0) * x
        j = x2 - F(9.0)
        N2 = i * j
        B = F(3.0) * A
        Cc = B * A
        Dd = Cc * A
        d2 = N2 / Dd
        sdd32 = F(strength * digamma * digamma)
        gr = (sdd32 * d2) / D32
        return (np.asarray(g, dtype=F) * gr).astype(F)


def clamp(w, lo, hi):
    return np.clip(np.asarray(w, dtype=F), F(lo), F(hi)).astype(F)


def qloss_sum_f64(w, sharpness, strength) -> float:
    """Exact-order-free reference for the layer loss numerator: fp64 sum of the fp32 integrand."""
    return float(deriv_forward(w, sharpness, strength).astype(np.float64).sum())


def fused_step(w, g, digamma, sharpness, strength, lo, hi, scale=1.0):
    """One fused pass as the QAT step composes it (tmq/tmq.py:637-659, :298-310, :263-272):
    y = forward(w); grad = backward(w, g) + deriv_backward(w, 1/n); loss = mean(deriv_forward(w)); wc = clamp(w).
    Returns (y, grad, w_clamped, loss_sum_f64)."""
    w = np.asarray(w, dtype=F)
    n = w.size
    y = forward(w, digamma)
    g1 = backward(w, g, digamma, scale)
    ginv = np.full(w.shape, F(1.0) / F(n), dtype=F)
    g2 = deriv_backward(w, ginv, sharpness, strength)
    with np.errstate(all="ignore"):
        grad = (g1 + g2).astype(F)
    return y, grad, clamp(w, lo, hi), qloss_sum_f64(w, sharpness, strength)
