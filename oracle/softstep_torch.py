"""The soft-staircase QAT element pass as PyTorch CPU eager ops (TEST INFRASTRUCTURE / timed CPU baseline).

This is the op sequence the reference executes when its CUDA extension is absent: autograd Functions whose
forward/backward are the eager formulas of tmq/tmq.py:417-419, :434-438, :469-473, :488-493, followed by
torch.mean (tmq/tmq.py:698-699) and torch.clamp (tmq/tmq.py:696).  bench.py times it on the host cores.
"""
import torch

from . import softstep as _np_oracle


def _sig(x):
    x = torch.clamp(x, -3.0, 3.0)
    x2 = x * x
    return x * (x2 + 27.0) / (27.0 + x2 * 9.0)


def _dsig(x):
    x = torch.clamp(x, -3.0, 3.0)
    x2 = x * x
    return ((x2 - 9) * (x2 - 9)) / (9 * (3 + x2) * (3 + x2))


def _d2sig(x):
    x = torch.clamp(x, -3.0, 3.0)
    x2 = x * x
    a = x2 + 3
    return 16 * x * (x2 - 9) / (3 * a * a * a)


class _Step(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, d):
        ctx.d = d
        ctx.save_for_backward(w)
        fw = torch.floor(w)
        return _sig(d * (w - fw) - d / 2.0) / (2.0 * _np_oracle.scalar_sigmoid(d / 2.0)) + 0.5 + fw

    @staticmethod
    def backward(ctx, g):
        (w,) = ctx.saved_tensors
        d = ctx.d
        arg = d * (w - torch.floor(w)) - d / 2
        return 1.0 * g * (d * _dsig(arg) / (2.0 * _np_oracle.scalar_sigmoid(d / 2.0))), None


class _StepDeriv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, d, strength):
        ctx.d, ctx.s = d, strength
        ctx.save_for_backward(w)
        arg = d * (w - torch.floor(w)) - d / 2
        return strength * d * _dsig(arg) / (2.0 * _np_oracle.scalar_sigmoid(d / 2.0))

    @staticmethod
    def backward(ctx, g):
        (w,) = ctx.saved_tensors
        d, s = ctx.d, ctx.s
        arg = d * (w - torch.floor(w)) - d / 2
        return g * (s * d * d * _d2sig(arg) / (2.0 * _np_oracle.scalar_sigmoid(d / 2.0))), None, None


def qat_element_pass(w, g, digamma, sharpness, strength, lo, hi):
    """forward + quantization loss + backward of both + clamp on one weight tensor; returns (y, grad, w_clamped, loss)."""
    w = w.detach().requires_grad_(True)
    y = _Step.apply(w, digamma)
    loss = torch.mean(_StepDeriv.apply(w, sharpness, strength))
    torch.autograd.backward([y, loss], [g, torch.ones_like(loss)])
    with torch.no_grad():
        wc = torch.clamp(w, lo, hi)
    return y.detach(), w.grad, wc, loss.detach()
