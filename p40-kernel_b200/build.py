"""Compile the CUDA library for sm_100a, in tree.

    python p40-kernel_b200/build.py [--force] [--verbose]

Output: p40-kernel_b200/libbonsai_p40.so (same library name as the reference's build target, so a
program linked with -lbonsai_p40 picks it up unchanged).  nvcc cross-compiles without a GPU.
No fast-math: the quantiser and the rotation must perform IEEE divisions and separate mul / add.
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libbonsai_p40.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr", "--extended-lambda",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh")) +
                  glob.glob(os.path.join(HERE, "..", "include", "*.h")))


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force=False, verbose=False, tuning=True):
    """tuning: compile the geometry knobs of bonsai_b200_set_option in (the parity tests force every tiling through
    them); a production build passes tuning=False (--no-tuning) and keeps only the documented options."""
    if not (force or stale()):
        return LIB
    cmd = [NVCC, *FLAGS, *(["-DBONSAI_B200_TUNING"] if tuning else []), "-o", LIB, os.path.join(CSRC, "bonsai_b200.cu")]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared-memory usage")
    ap.add_argument("--no-tuning", action="store_true", help="leave the test-only geometry knobs out of the library")
    a = ap.parse_args()
    print(build(a.force or a.no_tuning, a.verbose, not a.no_tuning))
    sys.exit(0)
