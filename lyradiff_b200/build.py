"""Builds liblyraq.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a, and liblyradiff_classes.so (host C++ that
registers the torch custom classes over that C ABI) with g++.

Usage: python -m lyradiff_b200.build [--force] [--verbose]
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liblyraq.so")
CLASSES_LIB = os.path.join(HERE, "liblyradiff_classes.so")
CLASSES_SRC = os.path.join(CSRC, "torch_classes.cpp")

SOURCES = ["api.cu", "quant_kernels.cu", "gemm_dense.cu", "gemm_w4a4.cu", "lora_down.cu", "block_kernels.cu", "attention.cu", "linear_layers.cu", "noalloc.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if not f.endswith((".o", ".cpp"))]
    deps.append(os.path.join(HERE, "..", "include", "lyraq.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ into lyradiff_b200/liblyraq.so.  Returns the library path."""
    if not force and not _stale():
        return LIB
    objs = []
    procs = []
    for src in _sources():
        obj = src[:-3] + ".o"
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (os.path.basename(src), out))
        failed = failed or pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.check_call(cmd)
    return LIB


def build_classes(force=False):
    """Compile csrc/torch_classes.cpp (no device code) against torch's headers and link it to liblyraq.so, found at load time
    beside it ($ORIGIN).  Returns the library path."""
    build(force=force)
    deps = [CLASSES_SRC, LIB, os.path.join(HERE, "..", "include", "lyraq.h")]
    if not force and os.path.exists(CLASSES_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(CLASSES_LIB) for d in deps):
        return CLASSES_LIB
    import torch
    from torch.utils import cpp_extension
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cmd += ["-I" + p for p in cpp_extension.include_paths()] + ["-I" + cuda_inc]
    cmd += [CLASSES_SRC, "-o", CLASSES_LIB, "-L" + HERE, "-llyraq", "-L" + torch_lib,
            "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-Wl,-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    return CLASSES_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_classes(force="--force" in sys.argv))
