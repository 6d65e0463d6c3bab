"""The reference's C++ API as a C++ caller sees it: tests/cpp/dropin_sample.cpp is written against
hiptensor.hpp (mangled entry points, std::vector-bearing structs), linked with libhiptensor_b200.so and run."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_caller_runs_unchanged():
    sys.path.insert(0, os.path.join(ROOT, "tests", "cpp"))
    from hiptensor_b200 import build as libbuild

    libbuild.build()
    import build_sample

    exe = build_sample.build()
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "DROPIN OK" in out.stdout
