"""Builds and runs the C++ unit tests of the host internals (csrc/tests/unit_tests.cc)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_unit_tests(tmp_path):
    exe = tmp_path / "unit_tests"
    lib_dir = os.path.join(ROOT, "flagcx_b200", "lib")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-g", "-I" + os.path.join(ROOT, "csrc", "include"),
                           "-I" + os.path.join(ROOT, "csrc", "host"), "-I" + os.path.join(ROOT, "csrc", "kernels"),
                           "-I/usr/local/cuda/include", os.path.join(ROOT, "csrc", "tests", "unit_tests.cc"),
                           "-L" + lib_dir, "-lflagcx", "-Wl,-rpath," + lib_dir, "-lpthread", "-o", str(exe)])
    env = dict(os.environ, FLAGCX_DEBUG="WARN")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
