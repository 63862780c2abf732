"""Runs the C++ host layer's own test binary (tokspur-public_b200/native/tests/test_moe.cpp): `encode_moe` on the CUDA graph
against the CPU oracle, written like the reference's native/tests/test_moe.cpp."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tokspur-public_b200", "native", "tests", "test_moe")


def test_encode_moe_cpp_suite():
    if not os.path.exists(BIN):
        subprocess.run(["make", "-s", "-C", os.path.dirname(os.path.dirname(BIN))], check=True)
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "MoE encode checks passed" in r.stdout
