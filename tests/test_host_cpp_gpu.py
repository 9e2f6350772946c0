"""The C++ host layer (zdraw_b200/host/mattn.hpp) over the C ABI: a compiled test program in the
style of the reference's mattn_test.zig, run on the GPU."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_cpp_host_layer():
    subprocess.run(["make", "-C", os.path.join(HERE, "csrc")], check=True, capture_output=True)
    res = subprocess.run([os.path.join(HERE, "_build", "host_test")], capture_output=True, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode != 77, "no GPU visible to the C++ test: " + res.stdout
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PASS" in res.stdout


def test_cpp_multi_gpu_driver():
    """zdraw_b200/host/multi_gpu.hpp: one thread and one context per GPU (two ranks on one GPU when only one
    is visible), heads split over them, outputs gathered by the attention epilogue, byte for byte against a
    one-context run; a deadline that has passed is reported, nothing hangs."""
    subprocess.run(["make", "-C", os.path.join(HERE, "csrc")], check=True, capture_output=True)
    res = subprocess.run([os.path.join(HERE, "_build", "multi_gpu_test")], capture_output=True, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode != 77, "no GPU visible to the C++ test: " + res.stdout
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PASS" in res.stdout
