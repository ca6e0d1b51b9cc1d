"""Runs the C++ host mirror's replay of the reference's tests (host/test_quantized.cpp): the same
assertions as tests/nn/quantization_tests.rs, written against nn_quantized.hpp over the C ABI."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_replay_of_reference_tests():
    exe = os.path.join(ROOT, "neural-network-engine_b200", "lib", "test_quantized")
    assert os.path.exists(exe), "build it with __graft_entry__.build()"
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    print(r.stdout, r.stderr)
    assert r.returncode == 0 and "all reference tests passed" in r.stdout
