"""The C-ABI library builds, loads and exports exactly what include/tmq_b200.h declares (no compute, no GPU)."""
import os
import re
import subprocess

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "tmq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tmq_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    from tmq_b200 import build
    path = build.build()
    out = subprocess.check_output(["nm", "-D", "--defined-only", path], text=True)
    exported = sorted(set(re.findall(r" T (tmq_[a-z0-9_]+)$", out, flags=re.M)))
    assert exported == _declared()


def test_ctypes_signatures_cover_the_header():
    from tmq_b200 import _lib
    assert _lib.exported_symbols() == _declared()
    L = _lib.lib()
    assert L.tmq_abi_version() >= 1
    assert L.tmq_status_string(0) == b"ok"
    assert L.tmq_reduce_scratch_bytes() >= 256 + 8 * 1024


def test_argument_validation_needs_no_gpu():
    """Host-side validation returns error codes before anything is launched."""
    import ctypes
    from tmq_b200 import _lib
    L = _lib.lib()
    assert L.tmq_softstep_fwd(None, None, 16, 1.0, None) == -1
    assert L.tmq_softstep_fwd(ctypes.c_void_p(2), ctypes.c_void_p(64), 16, 1.0, None) == -2
    assert L.tmq_softstep_fwd(ctypes.c_void_p(64), ctypes.c_void_p(64), 16, float("nan"), None) == -1
    assert L.tmq_softstep_fwd(ctypes.c_void_p(64), ctypes.c_void_p(64), 0, 1.0, None) == 0
    assert L.tmq_clamp(ctypes.c_void_p(64), ctypes.c_void_p(64), 8, 1.0, -1.0, None) == -1
    assert L.tmq_qloss_sum(ctypes.c_void_p(64), 8, 5.0, 1e-3, ctypes.c_void_p(64), ctypes.c_void_p(256), 16, None) == -5
    assert L.tmq_pack2b_f32(None, None, 4, 4, None) == -1
    assert L.tmq_pack2b_f32(None, None, 0, 4, None) == 0
