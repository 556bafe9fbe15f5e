"""In-tree build of the native pieces (no JIT cache: the built files sit next
to the sources so they travel with the tree).

``libkivi_cuda.so``  hand-written sm_100a kernels behind the C ABI of
                     include/kivi_cuda.h (nvcc only, no torch).
``_C.*.so``          the torch extension mirroring the reference's pybind module
                     (g++ only; links libkivi_cuda.so through $ORIGIN).
"""
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libkivi_cuda.so")
EXT = os.path.join(PKG, "_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _cuda_sources():
    cu = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdr.append(os.path.join(ROOT, "include", "kivi_cuda.h"))
    return cu, hdr


def build_cuda_lib(force=False, verbose=False):
    cu, hdr = _cuda_sources()
    if not force and _newer(LIB, cu + hdr):
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + ["-I" + os.path.join(ROOT, "include"), "-I" + CSRC, "-o", LIB] + cu
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


def build_torch_ext(force=False, verbose=False):
    src = os.path.join(CSRC, "torch_ext.cpp")
    if not os.path.exists(src):
        return None
    build_cuda_lib(force=False, verbose=verbose)
    if not force and _newer(EXT, [src, LIB, os.path.join(ROOT, "include", "kivi_cuda.h")]):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce
    inc = ce.include_paths("cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(True)
    lib_dirs = ce.library_paths("cuda") if "device_type" in ce.library_paths.__code__.co_varnames else ce.library_paths(True)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w",
           "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I" + os.path.join(ROOT, "include"), "-I" + sysconfig.get_paths()["include"]]
    cmd += ["-I" + p for p in inc]
    cmd += [src, "-o", EXT, "-L" + PKG, "-l:libkivi_cuda.so", "-Wl,-rpath,$ORIGIN"]
    for d in lib_dirs:
        cmd += ["-L" + d, "-Wl,-rpath," + d]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return EXT


def build_all(force=False, verbose=False):
    build_cuda_lib(force, verbose)
    build_torch_ext(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
