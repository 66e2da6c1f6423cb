"""Builds libb200moe.so (the C-ABI product library) in-tree with nvcc for sm_100a.

Usage: python -m gfx1151_engine_b200.build [--force]
The library is plain CUDA C++: no PyTorch, no Python headers.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200moe.so")
SOURCES = ["api.cu", "repack.cu", "route.cu", "expert_simt.cu", "expert_gemv.cu", "expert_tc.cu", "combine.cu", "route_static.cu", "router_gemm.cu", "files.cu", "decode.cu", "ep_host.cu", "rotate.cu"]
HEADERS = ["common.cuh", "kernels.h", "tc.h", "route_small.cuh", os.path.join("..", "..", "include", "b200moe.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    # the environment may point nvcc's host compiler elsewhere; use the system one
    "-ccbin", "/usr/bin/g++",
] + os.environ.get("B200MOE_NVCC_FLAGS", "").split()


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every .cu to an object and link the shared library. Returns its path."""
    if not force and not _stale():
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for s in SOURCES:
        obj = os.path.join(objdir, s.replace(".cu", ".o"))
        cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, s), "-o", obj]
        procs.append((s, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for s, obj, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (s, out))
        if verbose:
            print(out)
        objs.append(obj)
    cmd = [NVCC, "-shared", "-o", LIB, "-ccbin", "/usr/bin/g++"] + objs + ["-lcudart", "-ldl"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
