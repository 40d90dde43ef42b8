"""The bounded-wait failure path of the tensor-core kernels, exercised without faulting or hanging anything.

Every device-side wait in the GEMM / GEMV / convolution kernels is bounded: when it runs out the kernel stores
TMQ_ERR_TIMEOUT in a status word and returns.  The word is sticky, and later launches that see it non-zero skip their
work.  Two things are checked here: (1) the wait itself gives up, on a barrier that nothing completes, with a budget
of about a millisecond; (2) a pre-set status word makes every kernel family return promptly with its output
untouched, and the Python layer raises and re-arms the word."""
import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TIMEOUT = -4


@pytest.fixture(scope="module")
def ops():
    from tmq_b200 import ops
    return ops


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_a_wait_that_nothing_completes_gives_up_and_reports(ops):
    from tmq_b200 import _lib
    L = _lib.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    budget = 2_000_000                                   # about a millisecond of SM clock
    t0 = time.perf_counter()
    assert L.tmq_selftest_wait_timeout(budget, status.data_ptr(), waited.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0                # returned promptly; the context is still usable
    assert int(status.item()) == TIMEOUT
    assert budget < int(waited.item()) < 100 * budget   # the clock is read every 1024 polls of the barrier
    # a second waiter that finds the word already set leaves early instead of spending its own budget (~2 s)
    waited.zero_()
    assert L.tmq_selftest_wait_timeout(4_000_000_000, status.data_ptr(), waited.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert 0 < int(waited.item()) < 200_000_000
    # bad arguments are refused on the host
    assert L.tmq_selftest_wait_timeout(0, status.data_ptr(), None, _stream()) == -1
    assert L.tmq_selftest_wait_timeout(1000, None, None, _stream()) == -1
    # and the device still computes
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0


def test_a_set_status_word_makes_every_kernel_family_skip_and_the_check_raises(ops):
    from tmq_b200 import _lib
    from oracle import ternary as T
    rng = np.random.default_rng(3)
    N, K = 128, 256
    W = rng.integers(-1, 2, (N, K)).astype(np.float32)
    P = torch.from_numpy(T.pack(W)).cuda()
    word = ops.gemm_status_word("cuda")
    ops.check_gemm_status()
    word.fill_(TIMEOUT)
    sentinel = 1234.0
    # tiled GEMM, skinny kernel and implicit convolution through the C ABI, each into a pre-filled output
    L = _lib.lib()
    wt = ops.prepack(P, N, ops.FMT_BF16)
    for M in (64, 4):
        X = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        Y = torch.full((M, N), sentinel, dtype=torch.float32, device="cuda")
        fn = L.tmq_ternary_gemm_bf16 if M > 8 else L.tmq_ternary_gemv_bf16
        t0 = time.perf_counter()
        assert fn(X.data_ptr(), wt.data_ptr(), None, None, Y.data_ptr(), M, N, K, N, 1, word.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0
        if M > 8:
            assert bool((Y == sentinel).all()), "the tiled GEMM must not write while the status word is set"
    wc = rng.integers(-1, 2, (64, 64, 3, 3)).astype(np.float32)
    rows = torch.from_numpy(T.pack(wc.reshape(64, -1))).cuda()
    xc = torch.randn(2, 8, 8, 64, device="cuda").to(torch.bfloat16)
    yc = torch.full((2, 8, 8, 64), sentinel, dtype=torch.bfloat16, device="cuda")
    wtc = ops.prepack(rows, 64, ops.FMT_BF16)
    assert L.tmq_ternary_conv2d_bf16(xc.data_ptr(), wtc.data_ptr(), None, None, None, yc.data_ptr(), 2, 8, 8, 64, 64, 3, 3,
                                     1, 1, 1, 1, 1, 1, 0, word.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    assert bool((yc.float() == torch.tensor(sentinel).to(torch.bfloat16).float()).all())
    # the Python layer: the synchronising check raises and re-arms ...
    with pytest.raises(_lib.TmqError):
        ops.check_gemm_status()
    assert int(word.item()) == 0
    # ... and so does the non-blocking watch, within a bounded number of operator calls
    word.fill_(TIMEOUT)
    X = torch.randn(32, K, device="cuda").to(torch.bfloat16)
    with pytest.raises(_lib.TmqError):
        for _ in range(4 * ops._StatusWatch.EVERY + 4):
            ops.ternary_gemm(X, wt, N)
            torch.cuda.synchronize()
    assert int(word.item()) == 0
    good = ops.ternary_gemm(X, wt, N, out_dtype=torch.float32)
    ops.check_gemm_status()
    ref = T.gemm_f64_fast(X.float().cpu().numpy(), P.cpu().numpy(), N)
    assert np.abs(good.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
