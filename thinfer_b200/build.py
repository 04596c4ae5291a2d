"""Builds libthinfer_nvfp4.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libthinfer_nvfp4.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr", "-ccbin", "/usr/bin/g++", "-cudart", "static",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    deps.append(os.path.join(HERE, "..", "include", "thinfer_nvfp4.h"))
    return any(os.path.getmtime(d) > t for d in deps)


DIAG_OUT = os.path.join(HERE, "libthinfer_nvfp4_diag.so")


def build(force: bool = False, verbose: bool = False, diag: bool = False) -> str:
    """Builds the library. ``diag=True`` builds the diagnostic variant instead (clock64 traces, "skip
    this part" switches and kernel-selection overrides read from TNF_GEMM_* environment variables) as
    libthinfer_nvfp4_diag.so; point THINFER_B200_LIB at it to use it. The default library has none of that."""
    if diag:
        cmd = [NVCC, *FLAGS, "-DTNF_GEMM_DIAG", "-o", DIAG_OUT, *sources(), "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("nvcc failed building libthinfer_nvfp4_diag.so")
        return DIAG_OUT
    if not (force or stale()):
        return OUT
    cmd = [NVCC, *FLAGS, "-o", OUT, *sources(), "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libthinfer_nvfp4.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv, diag="--diag" in sys.argv))
