"""Build the C oracle (test infrastructure) into oracle/_build/liboracle.so with gcc.

Run as a script or call ``build()``.  The reference itself cannot be compiled into a CPU
oracle in this image: its host side is Rust (no cargo), its kernels are CUDA linked against
libtorch, and the flash-attention sources need a CUTLASS checkout that the reference tree
does not carry.  So there is no ``oracle/_ref`` target; the restatement in ``oracle.c`` is
pinned by the reference's stored known-answer test instead.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "liboracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
