"""oracle.c against the compiled reference's outputs (golden: pack.npz, codec.npz) and against itself."""
import numpy as np
import pytest

from oracle import ternary as T


def test_kat_tiny():
    W = np.array([[1, -1], [0, 1], [-1, 0]], dtype=np.float32)
    P = T.pack(W)
    assert P.shape == (2, 1)
    assert [int(v) & 0xFFFFFFFF for v in P.flatten()] == [0x48000000, 0x90000000]


@pytest.mark.parametrize("name", ["lin", "conv", "soft", "wide", "conv1x1", "ints", "bytes"])
def test_pack_matches_reference(gold_pack, name):
    W = gold_pack[f"{name}_in"]
    P = T.pack(W)
    ref = gold_pack[f"{name}_packed"]
    assert P.shape == ref.shape and P.dtype == ref.dtype
    assert np.array_equal(P, ref)


@pytest.mark.parametrize("name", ["conv", "conv1x1"])
def test_unpack_matches_reference_4d(gold_pack, name):
    P = gold_pack[f"{name}_packed"]
    ref = gold_pack[f"{name}_expanded"]
    out = T.unpack(P, ref.shape)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))


def test_unpack_2d_is_true_inverse(gold_pack):
    W = gold_pack["lin_in"]
    out = T.unpack(gold_pack["lin_packed"], W.shape)
    assert np.array_equal(out, W)
    soft = gold_pack["soft_in"]
    out = T.unpack(gold_pack["soft_packed"], soft.shape)
    s64 = soft.astype(np.float64)
    want = np.clip(np.where(s64 >= 0, np.floor(s64 + 0.5), np.ceil(s64 - 0.5)), -1, 1)   # half away from zero
    assert np.array_equal(out, want.astype(np.float32))


def test_first_row_words(gold_pack):
    P = gold_pack["lin_packed"]
    assert P.shape == (50, 3)
    assert [int(v) & 0xFFFFFFFF for v in P[0]] == [0x9A101621, 0x45641148, 0x14800000]


@pytest.mark.parametrize("name", ["lin", "conv", "soft", "wide", "conv1x1", "skew", "big"])
def test_codec_matches_reference(gold_codec, name):
    shape = gold_codec[f"{name}_shape"].tolist()
    P = gold_codec[f"{name}_packed"]
    cols = shape[0]
    rows = int(np.prod(shape[1:]))
    stream = T.rc_encode(P, rows, cols)
    ref = gold_codec[f"{name}_stream"]
    assert stream.shape == ref.shape
    assert np.array_equal(stream, ref)
    back = T.rc_decode(ref, rows, cols)
    assert np.array_equal(back.reshape(P.shape), P)


def test_codec_header_layout(gold_codec):
    s = gold_codec["lin_stream"].view(np.uint8)
    assert s.size == 397
    assert int.from_bytes(s[0:8].tobytes(), "big") == 37 * 50
    assert int.from_bytes(s[16:20].tobytes(), "big") == 397
    assert int.from_bytes(s[8:16].tobytes(), "big") == (397 - 26 - 1) * 8


def test_gemm_variants_agree():
    rng = np.random.default_rng(3)
    N, K, M = 45, 70, 5
    W = rng.integers(-1, 2, (N, K)).astype(np.float32)
    P = T.pack(W)
    X = rng.standard_normal((M, K)).astype(np.float32)
    assert np.allclose(T.gemm_f32_seq(X, P, N), X @ W.T, rtol=1e-5, atol=1e-5)
    assert np.allclose(T.gemm_f64(X, P, N), X.astype(np.float64) @ W.T.astype(np.float64), rtol=1e-12, atol=1e-12)
    assert np.allclose(T.gemm_f64_fast(X, P, N), T.gemm_f64(X, P, N), rtol=1e-12, atol=1e-12)
    Xi = rng.integers(-127, 128, (M, K)).astype(np.int8)
    want = Xi.astype(np.int64) @ W.T.astype(np.int64)
    assert np.array_equal(T.gemm_i8(Xi, P, N), want.astype(np.int32))
    assert np.array_equal(T.gemm_i8_fast(Xi, P, N), want.astype(np.int32))
    assert np.array_equal(T.decode_i8(P, N), W.astype(np.int8))


def test_nonfinite_pack_follows_x86_conversion():
    W = np.array([[np.inf, -np.inf, np.nan, 3e9, -3e9, 2.5, -2.5, 0.4]], dtype=np.float32).T.copy()  # [8,1]
    P = T.pack(W)
    vals = T.unpack(P, W.shape).flatten().tolist()
    assert vals == [-1.0, -1.0, -1.0, -1.0, -1.0, 1.0, -1.0, 0.0]


@pytest.mark.parametrize("C,H,W,k,s,p,d,op", [(20, 9, 11, (3, 3), (1, 1), (1, 1), (1, 1), (0, 0)),
                                              (33, 12, 10, (3, 5), (2, 1), (1, 2), (1, 1), (1, 0)),
                                              (16, 8, 8, (5, 5), (2, 2), (2, 2), (1, 1), (1, 1)),
                                              (7, 10, 9, (3, 3), (1, 2), (2, 1), (2, 1), (0, 1))])
def test_depthwise_restatements_match_torch(C, H, W, k, s, p, d, op):
    """The depthwise oracle (fixed tap order, fp32) against torch's conv2d / conv_transpose2d in fp64 on the unpacked
    weights: equal up to fp32 rounding of at most ky*kx additions."""
    import torch
    rng = np.random.default_rng(C)
    Wt = rng.integers(-1, 2, (C, 1) + k).astype(np.float32)
    P = T.pack(Wt)
    assert P.shape == (1,) + k + ((C + 15) // 16,)
    x = rng.standard_normal((2, C, H, W)).astype(np.float32)
    sc, bi = rng.random(C).astype(np.float32), rng.standard_normal(C).astype(np.float32)
    ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(Wt).double(), None, s, p, d, groups=C)
    ref = ref.numpy() * sc[None, :, None, None] + bi[None, :, None, None]
    got = T.dwconv2d(x, P, k, s, p, d, sc, bi)
    assert got.shape == ref.shape and np.abs(got - ref).max() < 1e-5
    reft = torch.nn.functional.conv_transpose2d(torch.from_numpy(x).double(), torch.from_numpy(Wt).double(), None, s, p, op,
                                                C, d).numpy()
    gott = T.dwconvtrans2d(x, P, k, s, p, d, op)
    assert gott.shape == reft.shape and np.abs(gott - reft).max() < 1e-5
    # operator-level forms: unfold -> patches form == image form, bit for bit
    unf = torch.nn.functional.unfold(torch.from_numpy(x), kernel_size=k, dilation=d, stride=s, padding=p)
    L = unf.shape[-1]
    perm = unf.view(2, C, k[0], k[1], L).permute(0, 4, 2, 3, 1).reshape(2, L, -1).numpy()
    pat = T.dwconv_patches(perm, P, C, k[0] * k[1]).reshape(2, L, C).transpose(0, 2, 1)
    assert np.array_equal(pat.reshape(got.shape), T.dwconv2d(x, P, k, s, p, d))
