"""Builds the oracle's C restatement (oracle/ref_order.c) into oracle/libaccy_oracle.so.

The reference itself is Zig and needs a Zig 0.17 toolchain that this environment does not have, so
there is no oracle/_ref build of the reference's own sources; the restatement is the oracle.
Flags keep the reference's arithmetic: no fast-math, no FMA contraction; OpenMP only spreads
independent rows over threads for the all-cores baseline (each row is still one serial fold).
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ref_order.c")
LIB = os.path.join(HERE, "libaccy_oracle.so")


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    cmd = ["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-Wall", "-Wextra",
           "-o", LIB, SRC, "-lm"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
