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


def test_cpp_unit_tests_under_asan_and_ubsan(tmp_path):
    """The same tests against a host runtime built with -fsanitize=address,undefined
    (`make -C csrc asan`): sockets, bootstrap threads, registry, tuner, reducers."""
    import shutil
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    probe = subprocess.run([cxx, "-fsanitize=address,undefined", "-x", "c++", "-", "-o", str(tmp_path / "probe")],
                           input="int main(){return 0;}", text=True, capture_output=True)
    if probe.returncode != 0:
        import pytest
        pytest.skip("this compiler has no sanitizer runtimes")
    subprocess.run(["make", "-C", os.path.join(ROOT, "csrc"), "-j", "16", "asan", "ASAN_CXX=" + cxx], check=True,
                   capture_output=True)
    lib_dir = os.path.join(ROOT, "csrc", "build", "asan")
    exe = tmp_path / "unit_tests_asan"
    subprocess.check_call([cxx, "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer",
                           "-I" + os.path.join(ROOT, "csrc", "include"), "-I" + os.path.join(ROOT, "csrc", "host"),
                           "-I" + os.path.join(ROOT, "csrc", "kernels"), "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "csrc", "tests", "unit_tests.cc"), "-L" + lib_dir, "-lflagcx",
                           "-Wl,-rpath," + lib_dir, "-lpthread", "-o", str(exe)])
    # the static CUDA runtime keeps process-lifetime allocations; leaks are not what this run is for
    env = dict(os.environ, FLAGCX_DEBUG="WARN", ASAN_OPTIONS="detect_leaks=0:abort_on_error=0",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "ERROR: AddressSanitizer" not in res.stderr and "runtime error" not in res.stderr, res.stderr[-3000:]
