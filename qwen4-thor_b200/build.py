"""Builds libq4t_moe_b200.so (all CUDA kernels + the C ABI) and
libq4t_moe_b200_check.so (device-side checkers used only by the GPU tests) for
sm_100a with nvcc, in-tree, so that the shared objects travel with the source tree.

    python qwen4-thor_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libq4t_moe_b200.so")
CHECK_LIB = os.path.join(HERE, "libq4t_moe_b200_check.so")
SOURCES = ["api.cu", "quant_kernels.cu", "routing_kernels.cu", "tc_gemm.cu", "tc_gemm_pair.cu", "decode_small.cu", "bf16_small_m.cu", "noalloc.cu"]
CHECK_SOURCES = ["check/check_api.cu", "check/selftest.cu", "check/simt_check.cu"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _newest_source() -> float:
    paths = [os.path.join(d, f) for d in (CSRC, os.path.join(CSRC, "check")) for f in os.listdir(d)
             if f.endswith((".cu", ".cuh", ".h"))]
    paths += [os.path.join(HERE, "..", "include", h) for h in ("q4t_moe_b200.h", "q4t_moe_b200_check.h")]
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    newest = _newest_source()
    if not force and all(os.path.exists(l) and os.path.getmtime(l) >= newest for l in (LIB, CHECK_LIB)):
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    objs = []
    procs = []
    for src in SOURCES + CHECK_SOURCES:
        obj = os.path.join(CSRC, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {src}\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run([nvcc, "-shared", "-o", LIB, *objs[:len(SOURCES)]], check=True)
    subprocess.run([nvcc, "-shared", "-o", CHECK_LIB, *objs[len(SOURCES):]], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
