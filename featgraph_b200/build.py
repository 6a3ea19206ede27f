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


def _locked(path):
    """Exclusive lock on ``path`` for the life of the returned file object: several ranks of one job
    import the package at the same moment and must not build the same files side by side."""
    import fcntl
    f = open(path, "w")
    fcntl.flock(f, fcntl.LOCK_EX)
    return f


def cuda_stale():
    """True if the CUDA library is missing or older than any of its sources / headers."""
    return _newer(CUDA_LIB, cuda_sources() + _cuda_headers())


def _cuda_headers():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(_ROOT, "include", "featgraph_b200.h"))
    return hdrs


def build_cuda(force=False, verbose=False, extra=(), target=None):
    """Compile every .cu under csrc/ (one object per source, in parallel; an object is rebuilt when
    its source or any header is newer) and link them into the shared library.  Does nothing when
    the library is up to date.  ``extra``: more nvcc flags (forces a full rebuild); ``target``:
    write the library somewhere else (a variant build; also a full rebuild, objects kept apart)."""
    from concurrent.futures import ThreadPoolExecutor
    srcs = cuda_sources()
    hdrs = _cuda_headers()
    out = target or CUDA_LIB
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
    variant = bool(extra) or target is not None
    if not (force or variant or _newer(out, srcs + hdrs)):
        return out
    if variant:  # objects of a variant build are of no further use
        import tempfile
        objdir = tempfile.mkdtemp(prefix="fg_obj_")
    else:
        objdir = os.path.join(LIBDIR, "obj")
        os.makedirs(objdir, exist_ok=True)
    lock = _locked(os.path.join(LIBDIR, ".build.lock"))
    try:
        if not (force or variant or _newer(out, srcs + hdrs)):
            return out  # another process built it while this one waited for the lock
        nvcc, cxx = _nvcc(), _host_cxx()
        compile_flags = [f for f in NVCC_FLAGS if f not in ("-shared", "-cudart", "static")]
        jobs = []
        objs = []
        for src in srcs:
            obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
            objs.append(obj)
            if force or variant or _newer(obj, [src] + hdrs):
                jobs.append([nvcc, *compile_flags, "-ccbin", cxx, "-I", os.path.join(_ROOT, "include"),
                             "-I", CSRC, *extra, "-c", "-o", obj, src])

        def run(cmd):
            if verbose:
                print(" ".join(cmd), flush=True)
            r = subprocess.run(cmd, capture_output=True, text=True)
            return cmd, r

        with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
            results = list(pool.map(run, jobs))
        for cmd, r in results:
            if verbose or r.returncode != 0:
                if r.stdout:
                    print(r.stdout, end="")
                if r.stderr:
                    print(r.stderr, end="")
            if r.returncode != 0:
                raise subprocess.CalledProcessError(r.returncode, cmd, r.stdout, r.stderr)
        tmp = out + ".tmp.%d" % os.getpid()
        link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-shared",
                "-cudart", "static", "-ccbin", cxx, "-o", tmp, *objs]
        if verbose:
            print(" ".join(link), flush=True)
        subprocess.run(link, check=True)
        os.replace(tmp, out)  # a process that has the old file mapped keeps it; new loads see the new one
    finally:
        lock.close()
        if variant:
            shutil.rmtree(objdir, ignore_errors=True)
    return out


def build_all(force=False, verbose=False):
    return build_cuda(force, verbose), build_graphgen(force, verbose)


if __name__ == "__main__":
    import sys
    build_all(force="--force" in sys.argv, verbose=True)
