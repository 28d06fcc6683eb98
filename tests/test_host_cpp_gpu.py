"""Runs the C++ host-layer tests (tests/cpp/host_tests.cpp: the nz:: mirror of NeuZephyr's API
driven the way the reference's GoogleTest cases drive it) on the GPU."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _binary(name):
    from neuzephyr_b200 import build as B
    B.build()
    return B.build_program(os.path.join(ROOT, "tests", "cpp", name + ".cpp"),
                           os.path.join(ROOT, "tests", "cpp", "bin", name), "../../../neuzephyr_b200")


def test_host_layer_cpp_suite():
    exe = _binary("host_tests")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-6000:])
    print(r.stderr[-2000:])
    assert r.returncode == 0, "C++ host tests failed:\n" + r.stdout[-4000:] + r.stderr[-2000:]
    assert " 0 failures" in r.stdout
