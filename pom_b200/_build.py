"""Build libpom_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

Run as ``python -m pom_b200._build`` or call :func:`build`.  The shared object is
written next to this file so it travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libpom_b200.so")
SOURCES = ["pom_gemm.cu", "pom_gemm_rope.cu", "pom_gemm_causal.cu", "pom_ops.cu", "pom_peer.cu", "pom_layer.cu", "pom_heads.cu"]
HEADERS = ["ptx_sm100.cuh", "pom_math.cuh", "gemm_sm100.cuh", "gemm2_sm100.cuh", "epilogues.cuh", "epilogues_rope.cuh", "epilogues_causal.cuh", "gemm_launch.cuh", "common.cuh", os.path.join("..", "..", "include", "pom_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libpom_b200.so cannot be built")


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    files = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    files += [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(f) > t for f in files if os.path.exists(f))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu translation unit and link the shared library. Returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    procs = []
    flags = list(NVCC_FLAGS)
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [nvcc, *flags, "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    # link beside the target and rename: a reader of the tree never sees a half-written library
    tmp = LIB_PATH + ".tmp"
    link = [nvcc, "-shared", "-o", tmp, *objs, "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link of libpom_b200.so failed")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
