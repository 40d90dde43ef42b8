"""The allocation-free loss-sum entry point (tmq_qloss_sum_noalloc), called straight through the C ABI.

It exists for hosts that cannot allocate device memory and therefore cannot supply the scratch buffer that
tmq_qloss_sum wants; its scratch is a fixed array inside the library.  The check: on two calls in a row (different
data, so leftovers of the first call would show in the second) it must agree with tmq_qloss_sum AND with the CPU
oracle's fp64 sum of the bit-exact integrand (oracle.softstep.qloss_sum_f64) to the tolerance the loss tests use
(rel 2.5e-7: partial sums of four terms are fp32, everything above that fp64).

This file sorts last on purpose: a run that stops at the first failure has then already covered everything else.
It passes on its own in a fresh process as well as after the other tests.
"""
import ctypes

import pytest
import torch


def _lib():
    from tmq_b200 import _lib
    return _lib.lib()


def test_rejects_oversized_and_bad_arguments_without_touching_the_gpu():
    L = _lib()
    p = ctypes.c_void_p(256)
    too_many = 33554432 + 1
    assert L.tmq_qloss_sum_noalloc(p, too_many, 5.0, 1e-3, p, None) == -5          # beyond the built-in scratch
    assert L.tmq_status_string(-5) == b"scratch buffer too small"
    assert L.tmq_qloss_sum_noalloc(p, 16, 5.0, 1e-3, None, None) == -1              # no output pointer
    assert L.tmq_qloss_sum_noalloc(None, 16, 5.0, 1e-3, p, None) == -1              # no input
    assert L.tmq_qloss_sum_noalloc(p, 16, float("nan"), 1e-3, p, None) == -1        # bad hardness
    assert L.tmq_qloss_sum_noalloc(ctypes.c_void_p(258), 16, 5.0, 1e-3, p, None) == -2


@pytest.mark.gpu
def test_matches_the_scratch_taking_entry_point_twice_in_a_row():
    from oracle.softstep import qloss_sum_f64
    L = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    scratch = torch.zeros(L.tmq_reduce_scratch_bytes(), dtype=torch.uint8, device=dev)
    gen = torch.Generator(device=dev).manual_seed(11)
    # sizes: several blocks plus a ragged tail, then a different, smaller tensor; the second also misaligned by 4 B
    cases = [((1 << 21) + 13, 0), (300001, 1)]
    for n, offset in cases:
        base = torch.rand(n + offset, generator=gen, device=dev) * 3 - 1.5
        w = base[offset:]
        ref = torch.full((), -1.0, dtype=torch.float64, device=dev)
        got = torch.full((), -2.0, dtype=torch.float64, device=dev)
        rc = L.tmq_qloss_sum(ctypes.c_void_p(w.data_ptr()), n, 5.0, 5e-4, ctypes.c_void_p(ref.data_ptr()),
                             ctypes.c_void_p(scratch.data_ptr()), scratch.numel(), stream)
        assert rc == 0
        rc = L.tmq_qloss_sum_noalloc(ctypes.c_void_p(w.data_ptr()), n, 5.0, 5e-4, ctypes.c_void_p(got.data_ptr()),
                                     stream)
        assert rc == 0, L.tmq_status_string(rc)
        torch.cuda.synchronize()
        r, g = ref.item(), got.item()
        assert r > 0
        assert abs(g - r) <= 2.5e-7 * abs(r), (n, g, r)
        want = qloss_sum_f64(w.cpu().numpy(), 5.0, 5e-4)
        assert abs(g - want) <= 2.5e-7 * abs(want), (n, g, want)
    # empty input: the sum is zero and the call still succeeds
    got = torch.full((), 7.0, dtype=torch.float64, device=dev)
    assert L.tmq_qloss_sum_noalloc(None, 0, 5.0, 5e-4, ctypes.c_void_p(got.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert got.item() == 0.0
