"""Build the CPU checkers (TEST INFRASTRUCTURE; nothing here is a product path).

  oracle/libbonsai_oracle.so      <- oracle/bonsai_oracle.c   (this repository's C restatement)
  oracle/_ref/libbonsai_ref.so    <- oracle/ref_shim.cpp + the reference's own headers, compiled
                                     where they lie (only when a reference checkout is present)

Both are built without fused multiply-add contraction, fast-math or host-specific vector flags so
that every fp32 operation is one IEEE operation, as in the reference's host build.

Usage: python oracle/build_oracle.py [--reference DIR]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libbonsai_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libbonsai_ref.so")
# where a checkout of the reference is looked for: $BONSAI_REFERENCE_DIR, else a directory named "reference"
# beside this repository; when neither holds the headers, a prebuilt oracle/_ref is used as it is
DEFAULT_REFERENCE = os.environ.get("BONSAI_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

FP_FLAGS = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared"]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force=False):
    src = os.path.join(HERE, "bonsai_oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        subprocess.check_call(["gcc", "-std=c99", *FP_FLAGS, "-o", ORACLE_SO, src, "-lm", "-lpthread"])
    return ORACLE_SO


def build_reference(reference=DEFAULT_REFERENCE, force=False):
    """Returns the path of the reference build, or None when no reference checkout exists."""
    inc = os.path.join(reference, "src")
    if not os.path.isfile(os.path.join(inc, "pq2_0.h")):
        return REF_SO if os.path.exists(REF_SO) else None
    src = os.path.join(HERE, "ref_shim.cpp")
    deps = [src] + [os.path.join(inc, h) for h in ("pq2_0.h", "fwht.h", "pq2_0_repack.h", "p40_common.h", "ops.h", "kv_cache.h")]
    if force or _stale(REF_SO, deps):
        os.makedirs(REF_DIR, exist_ok=True)
        subprocess.check_call(["g++", "-std=c++17", *FP_FLAGS, "-I", inc, "-I", os.path.join(reference, "include"), "-o", REF_SO, src,
                               "-lpthread"])
    return REF_SO


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    print(build_reference(a.reference, a.force) or "reference checkout absent: oracle/_ref not built")
    sys.exit(0)
