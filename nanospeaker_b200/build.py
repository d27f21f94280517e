"""Build the CUDA library in-tree: nanospeaker_b200/libmoe_b200.so (sm_100a only).

Run as `python -m nanospeaker_b200.build`. nvcc cross-compiles without a GPU present.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmoe_b200.so")
SOURCES = ["api.cu", "routing.cu", "router_fused.cu", "movement.cu", "norm.cu", "gemm.cu", "ep.cu", "block.cu"]
HEADERS = ["ptx.cuh", "pdl.cuh", "gemm.cuh", "gemm_rows.cuh", "gemm_rows2.cuh", "gemm_wgrad2.cuh", "gemm_wgrad.cuh", "routing.cuh", "dispatch_scatter.cuh", os.path.join("..", "..", "include", "moe_b200.h")]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu for sm_100a into one shared library; returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [
        nvcc, "-shared", "-Xcompiler", "-fPIC", "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-t", "0",
        "-o", LIB,
    ] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
