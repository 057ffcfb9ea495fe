"""Builds libhomura_b200.so in-tree with nvcc for sm_100a (no torch involved).

    python -m homura_b200.build [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhomura_b200.so")
SOURCES = ["gemv_bf16.cu", "gemm_tc.cu", "attention.cu", "quant.cu", "kquant.cu", "kquant_gemm.cu", "sampler.cu", "misc_kernels.cu", "engine.cu", "capi.cu", "loaders.cpp", "launch_attrs.cpp"]
HEADERS = ["common.cuh", "engine.h", "gemm_tc.h", "mbarrier.cuh", "kquant.h", "sampler.h", "loaders.h", "launch_attrs.h", os.path.join("..", "..", "include", "homura_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--threads", "4",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """trace=True: a second library with -DHM_PHASE_TRACE (phase stamps inside the decode kernels), written next to
    the product library as libhomura_b200_trace.so; HOMURA_B200_LIB=<path> makes the package load it."""
    if trace:
        return _build(os.path.join(HERE, "libhomura_b200_trace.so"), os.path.join(HERE, "build", "trace"), ["-DHM_PHASE_TRACE"], verbose)
    if not force and not stale():
        return LIB
    return _build(LIB, os.path.join(HERE, "build"), [], verbose)


def _build(LIB: str, bdir: str, extra_flags, verbose: bool) -> str:
    objs = []
    env = dict(os.environ)
    # the image exports CC/CXX that point at a compiler without libgomp; nvcc should use the system g++
    cmd_base = [nvcc()] + NVCC_FLAGS + list(extra_flags) + ["-ccbin", "g++"]
    procs = []
    os.makedirs(bdir, exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(bdir, src + ".o")
        objs.append(obj)
        extra = ["-x", "cu"] if src.endswith(".cpp") else []
        cmd = cmd_base + (["-Xptxas", "-v"] if verbose else []) + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)))
    failed = False
    for src, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src}\n{out}\n")
        elif verbose:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("nvcc build failed")
    subprocess.check_call([nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-ccbin", "g++", "-Xcompiler", "-fPIC", "-cudart", "static"], env=env)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
