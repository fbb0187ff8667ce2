"""Build the CPU checkers.

TEST INFRASTRUCTURE (see oracle.py).  Two shared libraries:

* ``oracle/_build/libmellin_oracle.so`` -- the plain-C restatement
  (``mellin_oracle.c``), always built.
* ``oracle/_ref/libmellin_ref.so`` -- the reference's own header-only CPU
  library behind a C shim (``ref_shim.cpp``), built only where a checkout of
  the reference is present (its sources are compiled where they lie and are
  never copied).  ``-O3 -fopenmp`` so that its OpenMP loops use every host core.

* ``oracle/_ref/mconv_cuda_profiling`` -- the reference's own CUDA timing harness,
  compiled for sm_100a where a checkout is present: the GPU incumbent of the benchmark.

Run ``python oracle/build_oracle.py`` or call :func:`build`.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "_build", "libmellin_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libmellin_ref.so")
REF_INCLUDE_CANDIDATES = [
    os.environ.get("MELLIN_REFERENCE_INCLUDE", ""),
    "/root/reference/ext/include",
]


def _newer(target, sources):
    if not os.path.isfile(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))


def build_port(force=False):
    srcs = [os.path.join(HERE, "mellin_oracle.c"), os.path.join(HERE, "mellin_oracle_impl.inc")]
    if not force and _newer(PORT_SO, srcs):
        return PORT_SO
    os.makedirs(os.path.dirname(PORT_SO), exist_ok=True)
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("no C compiler found for the oracle")
    _run([cc, "-O2", "-std=c11", "-fopenmp", "-Wall", "-shared", "-fPIC", "-o", PORT_SO, srcs[0]])
    return PORT_SO


def reference_include_dir():
    for cand in REF_INCLUDE_CANDIDATES:
        if cand and os.path.isfile(os.path.join(cand, "cdrobert", "mellin", "mconv.h")):
            return cand
    return None


def build_reference(force=False):
    """Returns the path of the built library, or None when no reference
    checkout is reachable and no prebuilt library exists."""
    inc = reference_include_dir()
    src = os.path.join(HERE, "ref_shim.cpp")
    if inc is None:
        return REF_SO if os.path.isfile(REF_SO) else None
    if not force and _newer(REF_SO, [src, os.path.join(inc, "cdrobert", "mellin", "mconv.h")]):
        return REF_SO
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found for the reference shim")
    _run([cxx, "-O3", "-fopenmp", "-std=c++14", "-shared", "-fPIC", "-I", inc, "-o", REF_SO, src])
    return REF_SO


REF_GPU_PROFILER = os.path.join(HERE, "_ref", "mconv_cuda_profiling")


def build_reference_gpu_profiler(force=False):
    """The reference's own CUDA timing harness (c/performance/mconv_cuda_profiling.cu: its stock
    thread-per-output kernels behind a command line), compiled for sm_100a from the sources where
    they lie.  It is the GPU incumbent the benchmark quotes beside this library's kernels.  Returns
    the binary's path, or None when neither a checkout nor a prebuilt binary is there."""
    inc = reference_include_dir()
    if inc is None:
        return REF_GPU_PROFILER if os.path.isfile(REF_GPU_PROFILER) else None
    root = os.path.dirname(os.path.dirname(inc))  # .../ext/include -> checkout root
    perf = os.path.join(root, "c", "performance")
    srcs = [os.path.join(perf, "mconv_cuda_profiling.cu"), os.path.join(perf, "OptionParser.cpp")]
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not all(os.path.isfile(s) for s in srcs) or not os.path.isfile(nvcc):
        return REF_GPU_PROFILER if os.path.isfile(REF_GPU_PROFILER) else None
    if not force and _newer(REF_GPU_PROFILER, srcs):
        return REF_GPU_PROFILER
    os.makedirs(os.path.dirname(REF_GPU_PROFILER), exist_ok=True)
    _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++14",
          "-I", os.path.join(root, "c", "cuda", "include"), "-I", os.path.join(root, "c", "cpu", "include"), "-I", inc,
          "-o", REF_GPU_PROFILER] + srcs + ["-lcublas"])
    return REF_GPU_PROFILER


def build(force=False):
    return build_port(force), build_reference(force), build_reference_gpu_profiler(force)


if __name__ == "__main__":
    port, ref, gpu = build(force="--force" in sys.argv)
    print("port:", port)
    print("reference:", ref)
    print("reference GPU profiler:", gpu)
