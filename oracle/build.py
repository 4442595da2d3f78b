"""Compile the CPU oracle (krea_oracle.c) into oracle/_build/libkrea_oracle.so.

Test infrastructure only.  The reference itself (Metal Shading Language + Objective-C++) cannot be
compiled with gcc/nvcc, so there is no oracle/_ref build: this restatement is the only CPU statement of
the path.  Flags stay at the x86-64-v3 level (AVX2 + FMA) so the library built on one machine also runs
on the GPU host.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "krea_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libkrea_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fno-math-errno", "-fno-trapping-math", "-std=gnu11",
           "-shared", "-fPIC", "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
