"""Build recipe for oracle/_ref/: the reference's own extension sources compiled where they lie.

TEST INFRASTRUCTURE. Nothing is copied: the compiler reads the sources from the read-only reference
checkout and only the resulting shared objects land in oracle/_ref/ (git-ignored).

  tmq_native   <-  <reference>/tmq/tmq_native.cpp (+ rangecoder.h, bitstream.h)   g++, CPU only
  tmq_cuda     <-  <reference>/tmq/tmq_cuda.cu                                     nvcc, sm_100a (optional, slow)

Both are torch/pybind11 extension modules, so they are importable as plain Python modules afterwards
(`import tmq_native` with oracle/_ref on sys.path). When the reference checkout is absent (for instance on a
GPU box) this script does nothing and the prebuilt files are used as they are.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# the reference checkout: TMQ_REFERENCE_DIR, else a checkout placed beside this repository
REFERENCE = os.environ.get("TMQ_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, libdir, abi


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_native(verbose=False):
    src = os.path.join(REFERENCE, "tmq", "tmq_native.cpp")
    if not os.path.exists(src):
        return None
    os.makedirs(OUT, exist_ok=True)
    target = os.path.join(OUT, "tmq_native.so")
    deps = [src, os.path.join(REFERENCE, "tmq", "rangecoder.h"), os.path.join(REFERENCE, "tmq", "bitstream.h")]
    if not _stale(target, deps):
        return target
    inc, libdir, abi = _torch_flags()
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           "-DTORCH_EXTENSION_NAME=tmq_native", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, src, "-o", target,
           f"-L{libdir}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python", f"-Wl,-rpath,{libdir}"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return target


def build_cuda(verbose=False):
    """The reference's CUDA extension for sm_100a (takes minutes). Used only as a same-box comparison."""
    src = os.path.join(REFERENCE, "tmq", "tmq_cuda.cu")
    if not os.path.exists(src):
        return None
    os.makedirs(OUT, exist_ok=True)
    target = os.path.join(OUT, "tmq_cuda.so")
    if not _stale(target, [src]):
        return target
    inc, libdir, abi = _torch_flags()
    cmd = ["nvcc", "-O2", "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-w",
           "-gencode", "arch=compute_100a,code=sm_100a",
           "-DTORCH_EXTENSION_NAME=tmq_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *inc, src, "-o", target,
           f"-L{libdir}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python",
           "-Xlinker", f"-rpath={libdir}"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return target


def load_native():
    """Import the compiled reference module (None when it was never built)."""
    target = os.path.join(OUT, "tmq_native.so")
    if not os.path.exists(target):
        return None
    import torch  # noqa: F401  (its shared libraries must be resident first)
    if OUT not in sys.path:
        sys.path.insert(0, OUT)
    import tmq_native
    return tmq_native


def load_cuda():
    target = os.path.join(OUT, "tmq_cuda.so")
    if not os.path.exists(target):
        return None
    import torch  # noqa: F401
    if OUT not in sys.path:
        sys.path.insert(0, OUT)
    import tmq_cuda
    return tmq_cuda


if __name__ == "__main__":
    print("tmq_native:", build_native(verbose=True))
    if "--cuda" in sys.argv:
        print("tmq_cuda:", build_cuda(verbose=True))
