"""Entropy-coded ("strong") storage of ternary weights: compress_ternary / decompress_ternary with the reference's
names and argument meaning (tmq/tmq_native.cpp:439-503), byte-compatible streams.

The range coder is sequential host code inside libtmq_b200.so (csrc/rangecoder.cu); packing before it and any
expansion after it run on the GPU through tmq_b200.ops."""
import ctypes

import torch

from ._lib import check, lib
from . import ops


def _rows_cols(orig_shape):
    orig_shape = [int(s) for s in orig_shape]
    cols = orig_shape[0]
    rows = 1
    for s in orig_shape[1:]:
        rows *= s
    return rows, cols


def compress_ternary(tensor, orig_shape, from_compact):
    """tensor: fp32 weight (from_compact False) or packed int32 (True) -> int8 stream [total bytes] on the CPU."""
    orig_shape = [int(s) for s in orig_shape]
    if from_compact:
        if tensor.dtype != torch.int32 or tensor.dim() not in (2, 4):
            raise RuntimeError("compress_ternary: expected a 2-D or 4-D int32 packed tensor")
        packed = tensor
    else:
        if tensor.dtype != torch.float32 or tensor.dim() not in (2, 4):
            raise RuntimeError("compress_ternary: expected a 2-D or 4-D float32 tensor")
        packed = ops.compactify_ternary(tensor)
    rows, cols = _rows_cols(orig_shape)
    p = packed.detach().cpu().contiguous()
    if p.numel() != rows * ((cols + 15) // 16):
        raise RuntimeError("compress_ternary: packed tensor does not match the original shape")
    cap = lib().tmq_rc_encode_bound(rows, cols)
    out = torch.empty(cap, dtype=torch.int8)
    n = ctypes.c_size_t(0)
    rc = lib().tmq_rc_encode(ctypes.c_void_p(p.data_ptr()), rows, cols, ctypes.c_void_p(out.data_ptr()), cap,
                             ctypes.byref(n))
    if rc == -1:
        raise RuntimeError("Illegal data encountered")
    check(rc, "compress_ternary")
    return out[: n.value].clone()


def decompress_ternary(stream, orig_shape):
    """int8 stream -> packed int32 [K, ceil(N/16)] (or [I, ky, kx, ceil(O/16)]) on the stream's device."""
    orig_shape = [int(s) for s in orig_shape]
    if stream.dtype != torch.int8 or stream.dim() != 1 or stream.numel() < 26:
        raise RuntimeError("decompress_ternary: expected a 1-D int8 stream with a 26-byte header")
    rows, cols = _rows_cols(orig_shape)
    q = (cols + 15) // 16
    s = stream.detach().cpu().contiguous()
    out = torch.empty((rows, q), dtype=torch.int32)
    rc = lib().tmq_rc_decode(ctypes.c_void_p(s.data_ptr()), s.numel(), ctypes.c_void_p(out.data_ptr()), rows, cols)
    check(rc, "decompress_ternary")
    if len(orig_shape) == 4:
        out = out.view(orig_shape[1], orig_shape[2], orig_shape[3], q)
    return out.to(stream.device)
