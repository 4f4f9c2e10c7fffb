"""Build libnckv.so (all CUDA sources of this directory) for sm_100a with nvcc.

Usage:  python -m nanochat_b200.csrc.build [--verbose] [--force]
The shared library is written next to the package (nanochat_b200/libnckv.so); it is a build
artefact and is not tracked.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT = os.path.join(PKG, "libnckv.so")
SOURCES = ["host.cu", "append.cu", "decode_attn.cu", "prefill_broadcast.cu", "lse_combine.cu",
           "prefill_attn.cu", "p2p_exchange.cu", "glue.cu", "flash_attn_bwd.cu", "host_step.cu"]
HEADERS = ["nckv_common.cuh", "tc05.cuh", os.path.join("..", "..", "include", "nckv.h")]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(verbose=False, force=False):
    if not force and up_to_date():
        return OUT
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
           "-o", OUT] + [os.path.join(HERE, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libnckv.so")
    return OUT


if __name__ == "__main__":
    build(verbose="--verbose" in sys.argv, force="--force" in sys.argv)
    print(OUT)
