"""ctypes front end of oracle.c (TEST INFRASTRUCTURE): packing, unpacking, GEMM restatements, range coder.

Layout contract restated from tmq/tmq_native.cpp:152-208, :303-319: a weight W[N][K] (Linear [out][in], or a conv
kernel [O][I*ky*kx] flattened in (c,ky,kx) order) becomes P[K][ceil(N/16)] int32, element i of a word in bits
[31-2i : 30-2i], codes 0 -> 00, +1 -> 01, -1 -> 10.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")
_SO = os.path.join(BUILD, "liboracle.so")
_SRC = os.path.join(HERE, "oracle.c")
_lib = None


def build(force=False):
    os.makedirs(BUILD, exist_ok=True)
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-shared", "-fPIC", _SRC, "-o", _SO, "-lm"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        i64, vp = ctypes.c_int64, ctypes.c_void_p
        for name in ("oracle_pack_f32", "oracle_pack_i32", "oracle_pack_i8", "oracle_unpack_f32", "oracle_unpack_i8"):
            getattr(L, name).argtypes = [vp, vp, i64, i64]
            getattr(L, name).restype = None
        for name in ("oracle_gemm_f32_seq", "oracle_gemm_i8", "oracle_gemm_f64"):
            getattr(L, name).argtypes = [vp, vp, vp, i64, i64, i64]
            getattr(L, name).restype = None
        L.oracle_rc_encode.argtypes = [vp, i64, i64, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint32)]
        L.oracle_rc_encode.restype = ctypes.c_int
        L.oracle_rc_decode.argtypes = [vp, ctypes.c_size_t, vp, i64, i64]
        L.oracle_rc_decode.restype = i64
        L.oracle_free.argtypes = [vp]
        L.oracle_free.restype = None
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def pack(W):
    """W: [N, K] (or [O, I, ky, kx]) float32 / int32 / int8 -> int32 [K, ceil(N/16)] (or [I, ky, kx, ceil(O/16)])."""
    W = np.ascontiguousarray(W)
    shape4 = W.shape if W.ndim == 4 else None
    W2 = W.reshape(W.shape[0], -1)
    N, K = W2.shape
    P = np.zeros((K, (N + 15) // 16), dtype=np.uint32)
    fn = {np.dtype(np.float32): "oracle_pack_f32", np.dtype(np.int32): "oracle_pack_i32",
          np.dtype(np.int8): "oracle_pack_i8"}[W2.dtype]
    getattr(lib(), fn)(_p(W2), _p(P), N, K)
    P = P.view(np.int32)
    if shape4 is not None:
        P = P.reshape(shape4[1], shape4[2], shape4[3], -1)
    return P


def unpack(P, shape):
    """Packed int32 -> float32 tensor of the original `shape` ([N,K] or [O,I,ky,kx])."""
    N = int(shape[0])
    K = int(np.prod(shape[1:]))
    P2 = np.ascontiguousarray(P).reshape(K, -1).view(np.uint32)
    W = np.zeros((N, K), dtype=np.float32)
    lib().oracle_unpack_f32(_p(P2), _p(W), N, K)
    return W.reshape(shape)


def decode_i8(P, N):
    """Packed [K, ceil(N/16)] -> T int8 [N, K]."""
    P2 = np.ascontiguousarray(P).reshape(-1, (N + 15) // 16).view(np.uint32)
    K = P2.shape[0]
    T = np.zeros((N, K), dtype=np.int8)
    lib().oracle_unpack_i8(_p(P2), _p(T), N, K)
    return T


def gemm_f32_seq(X, P, N):
    X = np.ascontiguousarray(X, dtype=np.float32)
    M, K = X.shape
    P2 = np.ascontiguousarray(P).reshape(K, -1).view(np.uint32)
    Y = np.zeros((M, N), dtype=np.float32)
    lib().oracle_gemm_f32_seq(_p(X), _p(P2), _p(Y), M, N, K)
    return Y


def gemm_i8(X, P, N):
    X = np.ascontiguousarray(X, dtype=np.int8)
    M, K = X.shape
    P2 = np.ascontiguousarray(P).reshape(K, -1).view(np.uint32)
    Y = np.zeros((M, N), dtype=np.int32)
    lib().oracle_gemm_i8(_p(X), _p(P2), _p(Y), M, N, K)
    return Y


def gemm_f64(X, P, N):
    X = np.ascontiguousarray(X, dtype=np.float32)
    M, K = X.shape
    P2 = np.ascontiguousarray(P).reshape(K, -1).view(np.uint32)
    Y = np.zeros((M, N), dtype=np.float64)
    lib().oracle_gemm_f64(_p(X), _p(P2), _p(Y), M, N, K)
    return Y


def gemm_f64_fast(X, P, N):
    """Same value as gemm_f64 up to fp64 summation order (BLAS on the decoded matrix); for large cases."""
    T = decode_i8(P, N).astype(np.float64)
    return np.asarray(X, dtype=np.float64) @ T.T


def gemm_i8_fast(X, P, N):
    """Exact integer result via fp64 BLAS (all partial sums stay far below 2^53)."""
    T = decode_i8(P, N).astype(np.float64)
    return np.rint(np.asarray(X, dtype=np.float64) @ T.T).astype(np.int32)


def rc_encode(P, rows, cols):
    """Range-code packed P [rows, ceil(cols/16)] -> int8 stream (26-byte big-endian header + payload)."""
    P2 = np.ascontiguousarray(P).reshape(rows, -1).view(np.uint32)
    out = ctypes.c_void_p()
    n = ctypes.c_uint32()
    rc = lib().oracle_rc_encode(_p(P2), rows, cols, ctypes.byref(out), ctypes.byref(n))
    if rc != 0:
        raise RuntimeError(f"oracle_rc_encode failed with {rc}")
    buf = np.frombuffer(ctypes.string_at(out, n.value), dtype=np.int8).copy()
    lib().oracle_free(out)
    return buf


def rc_decode(stream, rows, cols):
    s = np.ascontiguousarray(stream).view(np.uint8)
    P = np.zeros((rows, (cols + 15) // 16), dtype=np.uint32)
    rc = lib().oracle_rc_decode(_p(s), s.size, _p(P), rows, cols)
    if rc < 0:
        raise RuntimeError("oracle_rc_decode: malformed stream")
    return P.view(np.int32)


# ---- depthwise convolutions (numpy fp32, one rounding per line as the reference kernels do) ---------------------------

def _taps(P, C, ntaps):
    """Packed depthwise kernel int32 [ntaps][ceil(C/16)] (or [1][ky][kx][Q]) -> T [ntaps][C] in {-1, 0, +1}, the
    coefficient the reference kernels fetch as coeffs[chan/16 + ceil(C/16)*tap] (tmq/tmq_cuda.cu:141, :189)."""
    P = np.ascontiguousarray(P, dtype=np.int32).reshape(ntaps, (C + 15) // 16).view(np.uint32)
    c = np.arange(C)
    code = (P[:, c >> 4] >> (2 * (15 - (c & 15))).astype(np.uint32)) & 3
    return np.where(code == 1, 1.0, np.where(code == 2, -1.0, 0.0)).astype(np.float32)


def dwconv_patches(X, P, C, ntaps):
    """ternaryDWConvFP32 (tmq/tmq_cuda.cu:163-238): X [rows][ntaps][C] -> Y [rows][C], accu += x * t over taps in
    order, fp32 (the product with {-1,0,1} is exact, so the kernel's fused multiply-add rounds like this add)."""
    T = _taps(P, C, ntaps)
    X = np.asarray(X, dtype=np.float32).reshape(-1, ntaps, C)
    acc = np.zeros((X.shape[0], C), dtype=np.float32)
    for t in range(ntaps):
        acc = acc + X[:, t, :] * T[t][None, :]
    return acc


def dwconvtrans_patches(X, P, C, ntaps):
    """ternaryDWConvTransFP32 (tmq/tmq_cuda.cu:118-159): X [B][P][C] -> Y [B][C*ntaps][P] with
    Y[b][c*ntaps + t][p] = X[b][p][c] * T[t][c]."""
    T = _taps(P, C, ntaps)
    X = np.asarray(X, dtype=np.float32)
    Y = X.transpose(0, 2, 1)[:, :, None, :] * T.T[None, :, :, None]       # [B][C][ntaps][P]
    return Y.reshape(X.shape[0], C * ntaps, X.shape[1]).astype(np.float32)


def _finish(acc, scale, bias):
    if scale is not None:
        acc = acc * np.asarray(scale, dtype=np.float32)[None, :, None, None]
    if bias is not None:
        acc = acc + np.asarray(bias, dtype=np.float32)[None, :, None, None]
    return acc.astype(np.float32)


def dwconv2d(X, P, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), scale=None, bias=None):
    """Depthwise Conv2d.compact_forward (tmq/tmq.py:849-854 around ternaryDWConvFP32), restated on the image itself:
    taps accumulate in (ky, kx) order from +0 with x = 0 outside the image; output size as torch conv2d."""
    X = np.asarray(X, dtype=np.float32)
    B, C, H, W = X.shape
    (ky, kx), (sy, sx), (py, px), (dy, dx) = kernel, stride, padding, dilation
    T = _taps(P, C, ky * kx)
    OH = (H + 2 * py - dy * (ky - 1) - 1) // sy + 1
    OW = (W + 2 * px - dx * (kx - 1) - 1) // sx + 1
    Xp = np.zeros((B, C, H + 2 * py + sy, W + 2 * px + sx), dtype=np.float32)
    Xp[:, :, py:py + H, px:px + W] = X
    acc = np.zeros((B, C, OH, OW), dtype=np.float32)
    for i in range(ky):
        for j in range(kx):
            v = Xp[:, :, i * dy:i * dy + (OH - 1) * sy + 1:sy, j * dx:j * dx + (OW - 1) * sx + 1:sx]
            acc = acc + v * T[i * kx + j][None, :, None, None]
    return _finish(acc, scale, bias)


def dwconvtrans2d(X, P, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1), output_padding=(0, 0), scale=None,
                  bias=None):
    """Depthwise ConvTranspose2d.compact_forward (tmq/tmq.py:1025-1029: ternaryDWConvTransFP32 + F.fold) in gather
    form: output (oy, ox) sums, in (ky, kx) order from +0, the taps whose source pixel (oy + py - i*dy) / sy is integral
    and inside the input (x = 0 otherwise); output size as torch conv_transpose2d."""
    X = np.asarray(X, dtype=np.float32)
    B, C, H, W = X.shape
    (ky, kx), (sy, sx), (py, px), (dy, dx), (opy, opx) = kernel, stride, padding, dilation, output_padding
    T = _taps(P, C, ky * kx)
    OH = (H - 1) * sy - 2 * py + dy * (ky - 1) + 1 + opy
    OW = (W - 1) * sx - 2 * px + dx * (kx - 1) + 1 + opx
    oy, ox = np.arange(OH), np.arange(OW)
    acc = np.zeros((B, C, OH, OW), dtype=np.float32)
    for i in range(ky):
        ty = oy + py - i * dy
        iy = ty // sy
        oky = (ty >= 0) & (iy * sy == ty) & (iy < H)
        for j in range(kx):
            tx = ox + px - j * dx
            ix = tx // sx
            okx = (tx >= 0) & (ix * sx == tx) & (ix < W)
            v = X[:, :, np.clip(iy, 0, H - 1)][:, :, :, np.clip(ix, 0, W - 1)]
            v = np.where((oky[:, None] & okx[None, :])[None, None], v, np.float32(0.0))
            acc = acc + v * T[i * kx + j][None, :, None, None]
    return _finish(acc, scale, bias)
