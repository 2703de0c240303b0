"""Build libgemq_b200.so from the CUDA sources in this directory with nvcc (sm_100a only).

    python -m gemq_b200.csrc.build [--verbose]

The library lands next to the Python package (gemq_b200/libgemq_b200.so).  It is
rebuilt only when a source or header is newer than the library.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libgemq_b200.so")
SOURCES = ["pack.cu", "tma.cu", "gemv.cu", "gemv_stream.cu", "route.cu", "layer.cu", "decode_fused.cu", "gemm_sm100.cu", "expert_parallel.cu", "no_alloc.cu"]
HEADERS = ["common.cuh", "gemv.cuh", "ptx.cuh", os.path.join(ROOT, "include", "gemq_b200.h")]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; gemq_b200 has no CPU fallback and cannot be built without it")
    return nvcc


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, s) for s in SOURCES] + [h if os.path.isabs(h) else os.path.join(HERE, h) for h in HEADERS]
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not is_stale():
        return LIB
    nvcc = find_nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    common = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS,
              "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for s in SOURCES:
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        objs.append(obj)
        procs.append((s, subprocess.Popen(common + ["-c", os.path.join(HERE, s), "-o", obj],
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {s} ---\n{out}\n")
        failed = failed or p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([nvcc, "-shared", *ARCH_FLAGS, "-o", LIB, *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
