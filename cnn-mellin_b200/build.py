"""Build the native parts of the package in-tree.

``lib/libmellin_b200.so``   the C-ABI CUDA library (nvcc, sm_100a only)
``lib/mellin_torch.so``     the torch binding that registers the ``mellin::``
                            operators on top of it (g++, links the above)

    python build.py [--force] [--no-torch]

Nothing is installed outside this directory.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
CAPI_SO = os.path.join(LIBDIR, "libmellin_b200.so")
TORCH_SO = os.path.join(LIBDIR, "mellin_torch.so")

CAPI_SOURCES = ["capi.cu", "kernels.cu", "tc_direct.cu", "tc_direct_taps.cu", "tc_direct_masked.cu", "tc_gradw.cu", "batch_inner.cu", "gradw_rows.cu", "direct_rows.cu", "tc_scatter.cu", "tc_few_in.cu", "tc_gradw_few_in.cu", "few_in_rows.cu", "prologue.cu", "static_scratch.cu", "table_cache.cu", "peaks.cu", "index_map.cpp"]
CAPI_HEADERS = ["mellin_internal.h", "index_map.h", "tc_ptx.cuh", "tuning_hooks.h"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _run(cmd, **kw):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))
    return proc.stdout


def _fresh(target, deps):
    if not os.path.isfile(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def nvcc_path():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _compile_object(args):
    src, obj, flags = args
    _run([nvcc_path()] + flags + ["-c", src, "-o", obj])
    return obj


def build_capi(force=False, verbose_ptxas=False):
    """Compile every source to its own object (in parallel) and link them."""
    from concurrent.futures import ThreadPoolExecutor

    srcs = [os.path.join(CSRC, s) for s in CAPI_SOURCES]
    headers = [os.path.join(CSRC, h) for h in CAPI_HEADERS] + [os.path.join(INCLUDE, "mellin_b200.h")]
    if not force and _fresh(CAPI_SO, srcs + headers):
        return CAPI_SO
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if f != "-shared"] + (["-Xptxas", "-v"] if verbose_ptxas else [])
    jobs, objs = [], []
    for src in srcs:
        obj = os.path.join(OBJDIR, os.path.splitext(os.path.basename(src))[0] + ".o")
        objs.append(obj)
        # tc_direct_taps.cu / tc_direct_masked.cu include tc_direct.cu
        deps = [src] + headers + ([os.path.join(CSRC, "tc_direct.cu")] if "tc_direct_" in src else [])
        if force or not _fresh(obj, deps):
            jobs.append((src, obj, flags))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(_compile_object, jobs))
    _run([nvcc_path(), "-shared", "-o", CAPI_SO] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return CAPI_SO


def build_torch_binding(force=False):
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "mellin_torch.cpp")
    if not os.path.isfile(src):
        return None
    deps = [src, os.path.join(INCLUDE, "mellin_b200.h"), CAPI_SO]
    if not force and _fresh(TORCH_SO, deps):
        return TORCH_SO
    cxx = shutil.which("g++") or shutil.which("c++")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = cpp_extension.CUDA_HOME or "/usr/local/cuda"
    includes = cpp_extension.include_paths() + [os.path.join(cuda_home, "include"), INCLUDE]
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=mellin_torch",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in includes:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", TORCH_SO, "-L" + LIBDIR, "-lmellin_b200", "-Wl,-rpath,$ORIGIN",
            "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
            "-L" + os.path.join(cuda_home, "lib64"), "-lcudart"]
    _run(cmd)
    return TORCH_SO


def build(force=False, with_torch=True):
    capi = build_capi(force)
    binding = build_torch_binding(force) if with_torch else None
    return capi, binding


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, with_torch="--no-torch" not in sys.argv))
