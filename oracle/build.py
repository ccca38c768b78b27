"""Compile the C restatement (oracle/ref_chain.c) into oracle/libref_chain.so with gcc + OpenMP.

The reference itself cannot be compiled here (no Rust/Futhark toolchain), so there is no oracle/_ref.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libref_chain.so")


def build(force: bool = False) -> str:
    srcs = [os.path.join(HERE, "ref_chain.c"), os.path.join(HERE, "ref_chain_body.inc")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    # x86-64-v3 (AVX2 + F16C) rather than -march=native: the library is built on one host and runs on another
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-fexcess-precision=standard", "-shared", "-fPIC",
           "-o", LIB, srcs[0], "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
