"""Builds libtmq_b200.so (the C-ABI library of hand-written sm_100a kernels) in-tree with nvcc.

    python -m tmq_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The shared object lands in tmq_b200/_build/ and is what the
ctypes shim (tmq_b200/_lib.py) loads; there is no fallback if it is missing.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(OUT, "libtmq_b200.so")

SOURCES = ["capi.cu", "softstep.cu", "pack.cu", "qloss_noalloc.cu", "ternary_gemm.cu", "ternary_gemv.cu", "ternary_conv.cu", "ternary_conv_sw.cu", "ternary_conv_pm.cu", "layout.cu", "qat_linear.cu", "ternary_dwconv.cu", "rangecoder.cu"]

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--fmad=false",
              "-I", os.path.join(ROOT, "include"), "-I", CSRC]
# --fmad=false: contraction is a per-kernel decision here (explicit fmaf where wanted), never the compiler's.


def _headers():
    hs = [os.path.join(ROOT, "include", "tmq_b200.h")]
    hs += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return hs


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, force, verbose, extra=(), out=None):
    obj = os.path.join(out or OUT, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if force or _stale(obj, [path, __file__] + _headers()):
        cmd = ["nvcc", *NVCC_FLAGS, *extra, "-Xptxas", "-v", "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        with open(obj + ".log", "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force=False, verbose=False, extra_flags=(), out_dir=None):
    """Compile and link; `extra_flags` / `out_dir` produce tuning variants (-DTMQ_... macros) beside the product build."""
    out = out_dir or OUT
    lib = os.path.join(out, "libtmq_b200.so")
    os.makedirs(out, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose, tuple(extra_flags), out), SOURCES))
    if force or _stale(lib, objs):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib, *objs,
               "-cudart", "static", "-Xlinker", "--exclude-libs,ALL"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
