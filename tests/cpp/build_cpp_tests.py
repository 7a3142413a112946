"""Builds tests/cpp/_build/test_tch_cuda: the C++ host-side tests (g++, no nvcc needed: the
program only calls the CUDA runtime and the two shared libraries).

    python tests/cpp/build_cpp_tests.py

Links libaici_b200.so (the product), oracle/_build/liboracle.so (the checker) and libcudart;
run-time library paths are relative to the binary, so the tree can be moved as a whole.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
SRC = os.path.join(HERE, "test_tch_cuda.cpp")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "test_tch_cuda")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build(force: bool = False) -> str:
    sys.path.insert(0, ROOT)
    from aici_b200 import build as lib_build
    from oracle import build_oracle
    lib = lib_build.build()
    oracle = build_oracle.build()
    deps = [SRC, lib, oracle, os.path.join(ROOT, "include", "aici_b200_tch.hpp"),
            os.path.join(ROOT, "include", "aici_b200.h")]
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(d) for d in deps):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-O1", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(CUDA, "include"), SRC, "-o", OUT,
           "-L", os.path.dirname(lib), "-laici_b200", "-L", os.path.dirname(oracle), "-loracle",
           "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN/../../../aici_b200", "-Wl,-rpath,$ORIGIN/../../../oracle/_build",
           "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed:\n%s\n%s" % (res.stdout, res.stderr))
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
