"""The product range coder (host code in libtmq_b200.so) against the reference's streams (golden: codec.npz)
and the oracle.  Runs without a GPU: the coder is host-only."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ternary as T


def _encode(P, rows, cols):
    from tmq_b200 import _lib
    L = _lib.lib()
    p = np.ascontiguousarray(P).reshape(rows, -1).astype(np.int32)
    cap = L.tmq_rc_encode_bound(rows, cols)
    out = np.zeros(cap, dtype=np.int8)
    n = ctypes.c_size_t(0)
    rc = L.tmq_rc_encode(p.ctypes.data, rows, cols, out.ctypes.data, cap, ctypes.byref(n))
    return rc, out[: n.value]


def _decode(stream, rows, cols):
    from tmq_b200 import _lib
    L = _lib.lib()
    s = np.ascontiguousarray(stream)
    out = np.zeros((rows, (cols + 15) // 16), dtype=np.int32)
    rc = L.tmq_rc_decode(s.ctypes.data, s.size, out.ctypes.data, rows, cols)
    return rc, out


@pytest.mark.parametrize("name", ["lin", "conv", "soft", "wide", "conv1x1", "skew", "big"])
def test_streams_are_byte_identical_to_the_reference(gold_codec, name):
    shape = gold_codec[f"{name}_shape"].tolist()
    P = gold_codec[f"{name}_packed"]
    cols, rows = shape[0], int(np.prod(shape[1:]))
    rc, stream = _encode(P, rows, cols)
    assert rc == 0
    assert np.array_equal(stream, gold_codec[f"{name}_stream"])
    rc, back = _decode(gold_codec[f"{name}_stream"], rows, cols)
    assert rc == 0 and np.array_equal(back.reshape(P.shape), P)


def test_random_matrices_roundtrip_and_match_oracle():
    rng = np.random.default_rng(4)
    for (N, K, p) in [(1, 1, (0.3, 0.4)), (16, 16, (0.1, 0.8)), (77, 33, (0.45, 0.1)), (300, 129, (0.3, 0.4))]:
        u = rng.random((N, K))
        W = np.where(u < p[0], -1.0, np.where(u < p[0] + p[1], 0.0, 1.0)).astype(np.float32)
        P = T.pack(W)
        rc, stream = _encode(P, K, N)
        assert rc == 0
        assert np.array_equal(stream, T.rc_encode(P, K, N))
        rc, back = _decode(stream, K, N)
        assert rc == 0 and np.array_equal(back, P)


def test_rejects_illegal_code_and_short_streams():
    P = np.array([[0xC0000000 - (1 << 32)]], dtype=np.int64).astype(np.int32)      # code 11
    rc, _ = _encode(P, 1, 16)
    assert rc == -1
    rc, _ = _decode(np.zeros(10, dtype=np.int8), 1, 16)
    assert rc == -1
