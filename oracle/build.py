"""Build the CPU oracle (test infrastructure) into oracle/_build/libvexel_oracle.so.

The reference is Go and no Go toolchain exists where this is built, so there is no
oracle/_ref/ build of the reference itself; the oracle is the C restatement only.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libvexel_oracle.so")
SRC = os.path.join(HERE, "vexel_oracle.c")
HDR = os.path.join(HERE, "vexel_oracle.h")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB):
        newest = max(os.path.getmtime(SRC), os.path.getmtime(HDR))
        if os.path.getmtime(LIB) >= newest:
            return LIB
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
           "-std=c11", "-Wall", "-Wno-maybe-uninitialized", "-o", LIB, SRC, "-lm"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
