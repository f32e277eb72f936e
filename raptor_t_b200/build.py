"""Builds the CUDA library of this package in-tree with nvcc for sm_100a.

    python -m raptor_t_b200.build [--force]

Output: raptor_t_b200/lib/libraptor_b200.so - the C-ABI library - and
raptor_t_b200/lib/raptor_t.so - the pybind11 module `raptor_t` with the reference's operator
classes on top of it (both git-ignored).  nvcc cross-compiles without a GPU, so this also
works on a CPU-only build machine.
"""
import contextlib
import fcntl
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libraptor_b200.so")

SOURCES = [
    "runtime.cpp", "metadata.cpp", "tma_host.cpp", "elementwise.cu", "gemm_sm100.cu", "gemm_pair_sm100.cu", "gemm_ln_sm100.cu", "attention_sm100.cu",
    "encoder.cu", "no_alloc.cu", "selftest.cu", "pooler.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
    "-DRT_BUILD",
]


def _nvcc():
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "raptor_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


@contextlib.contextmanager
def _build_lock():
    """Serialises builds between processes (the ranks of a multi-GPU launch import the package at the same
    time): whoever comes second finds the library fresh and returns."""
    os.makedirs(LIB_DIR, exist_ok=True)
    with open(os.path.join(LIB_DIR, ".build.lock"), "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


SHIM = os.path.join(LIB_DIR, "raptor_t.so")
SHIM_SRC = os.path.join(CSRC, "pybind_shim.cpp")


def build_shim(force=False):
    """Compile the pybind11 module `raptor_t` (csrc/pybind_shim.cpp) against torch's headers and
    link it to libraptor_b200.so; returns its path."""
    def fresh():
        return os.path.exists(SHIM) and os.path.getmtime(SHIM) >= max(
            os.path.getmtime(SHIM_SRC), os.path.getmtime(LIB),
            os.path.getmtime(os.path.join(HERE, "..", "include", "raptor_b200.h")))
    if not force and fresh():
        return SHIM
    with _build_lock():
        if not force and fresh():
            return SHIM
        return _build_shim_locked()


def _build_shim_locked():
    import sysconfig

    import torch
    tdir = os.path.dirname(torch.__file__)
    cuda_home = os.path.dirname(os.path.dirname(_nvcc())) if os.path.isabs(_nvcc()) else "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", SHIM_SRC, "-o", SHIM, "-DTORCH_EXTENSION_NAME=raptor_t",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           f"-I{tdir}/include", f"-I{tdir}/include/torch/csrc/api/include", f"-I{sysconfig.get_paths()['include']}",
           f"-I{cuda_home}/include", f"-L{tdir}/lib", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-lc10_cuda",
           "-ltorch_cuda", f"-L{cuda_home}/lib64", "-lcudart", f"-L{LIB_DIR}", "-lraptor_b200", "-Wl,-rpath,$ORIGIN",
           f"-Wl,-rpath,{tdir}/lib"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("raptor_t_b200: building the pybind11 module failed")
    return SHIM


def build(force=False, verbose=False):
    """Compile every CUDA/C++ source into one shared library; returns its path."""
    if not force and not _stale():
        return LIB
    with _build_lock():
        if not force and not _stale():
            return LIB
        return _build_locked(verbose)


def _build_locked(verbose):
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in _sources():
        obj = os.path.join(LIB_DIR, os.path.basename(src) + ".o")
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("raptor_t_b200: CUDA build failed")
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs + ["-lpthread"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_shim(force="--force" in sys.argv))
