"""Compile the CPU oracle's C restatement into oracle/liborc.so (test infrastructure only)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "cmf_oracle.c")
OUT = os.path.join(HERE, "liborc.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    # -ffp-contract=off: no fused multiply-add, as in the reference's Rust build.
    # No -march=native: the library must also run on the GPU box's host CPU.
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-o", OUT, SRC, "-lm"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
