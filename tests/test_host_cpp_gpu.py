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
