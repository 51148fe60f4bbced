"""The C++ host mirror (swiftrt_b200/host/srt_host.hpp) against the reference's known-answer tests:
runs the compiled program tests/cpp/test_host_kat, which calls the CUDA library through its C ABI."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_host_mirror_known_answers():
    binary = os.path.join(ROOT, "tests", "cpp", "test_host_kat")
    if not os.path.exists(binary):
        import importlib.util
        spec = importlib.util.spec_from_file_location("_srt_b200_build", os.path.join(ROOT, "swiftrt_b200", "build.py"))
        b = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(b)
        b.build_host_test()
    fixture = os.path.join(ROOT, "tests", "golden", "lstm_kat.json")
    res = subprocess.run([binary, fixture], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "all host-mirror checks passed" in res.stdout
