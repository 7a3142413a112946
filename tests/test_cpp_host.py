"""The C++ host side (include/aici_b200_tch.hpp) exercised by tests/cpp/test_tch_cuda.cpp, a
plain C++ program in the manner of the reference crate's own tests.  Without a GPU only the
build and the test list are checked; with one, the program runs and must report no failure."""
import importlib.util
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _binary():
    spec = importlib.util.spec_from_file_location("build_cpp_tests",
                                                  os.path.join(HERE, "cpp", "build_cpp_tests.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def test_cpp_host_tests_build_and_list():
    res = subprocess.run([_binary(), "--list"], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stderr
    names = res.stdout.split()
    assert len(names) >= 10 and "flash_attn_varlen_causal_ragged_gqa" in names


@pytest.mark.gpu
def test_cpp_host_tests_pass(cuda_device):
    res = subprocess.run([_binary()], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    assert "0 of" in res.stdout
