"""The C++ partition logic (zdraw_b200/host/shard.hpp, the twin of zdraw_b200/shard.py) as a compiled CPU test."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))


def test_cpp_shard_logic():
    exe = os.path.join(HERE, "_build", "shard_test")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    subprocess.run(["g++", "-std=c++17", "-O2", "-o", exe, os.path.join(HERE, "csrc", "shard_test.cpp")],
                   check=True, capture_output=True)
    res = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0 and res.stdout.strip() == "ok", res.stdout + res.stderr
