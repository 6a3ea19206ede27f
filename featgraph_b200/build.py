"""In-tree build of the native libraries (no build system beyond nvcc / g++).

``build_all()`` compiles
  * ``_lib/libfeatgraph_b200.so`` - the sm_100a CUDA kernels behind the C ABI declared in
    ``include/featgraph_b200.h`` (nvcc, static CUDA runtime, no torch linkage);
  * ``_lib/libfg_graphgen.so``    - the host-side synthetic graph / feature generators.
Both land inside the package so that they travel with a copy of the tree.
"""
import os
import shutil
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_PKG, "csrc")
LIBDIR = os.path.join(_PKG, "_lib")
CUDA_LIB = os.path.join(LIBDIR, "libfeatgraph_b200.so")
GEN_LIB = os.path.join(LIBDIR, "libfg_graphgen.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",  # products and sums round separately, as in the x86 path being matched
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _host_cxx():
    # an environment CXX may point at a compiler without libgomp; prefer the system one
    for c in ("/usr/bin/g++", shutil.which("g++")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("no g++ found")


def _nvcc():
    for c in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def cuda_sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def build_graphgen(force=False, verbose=False):
    src = os.path.join(CSRC, "graphgen.cpp")
    os.makedirs(LIBDIR, exist_ok=True)
    if force or _newer(GEN_LIB, [src]):
        cmd = [_host_cxx(), "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c++17",
               "-o", GEN_LIB, src]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return GEN_LIB


def build_cuda(force=False, verbose=False, extra=()):
    srcs = cuda_sources()
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(_ROOT, "include", "featgraph_b200.h"))
    os.makedirs(LIBDIR, exist_ok=True)
    if force or _newer(CUDA_LIB, srcs + hdrs):
        cmd = [_nvcc(), *NVCC_FLAGS, "-ccbin", _host_cxx(), "-I", os.path.join(_ROOT, "include"),
               "-I", CSRC, *extra, "-o", CUDA_LIB, *srcs]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return CUDA_LIB


def build_all(force=False, verbose=False):
    return build_cuda(force, verbose), build_graphgen(force, verbose)


if __name__ == "__main__":
    import sys
    build_all(force="--force" in sys.argv, verbose=True)
