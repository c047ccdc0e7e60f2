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


import pytest  # noqa: E402


@pytest.mark.parametrize("kind,flags", [("asan", "-fsanitize=address,undefined"), ("tsan", "-fsanitize=thread")])
def test_cpp_unit_tests_under_sanitizers(tmp_path, kind, flags):
    """The same tests against a host runtime built with AddressSanitizer + UBSan, and with
    ThreadSanitizer (`make -C csrc asan|tsan`): sockets, bootstrap threads, registry,
    tuner, reducers."""
    import shutil
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    probe = subprocess.run([cxx, flags, "-x", "c++", "-", "-o", str(tmp_path / "probe")],
                           input="int main(){return 0;}", text=True, capture_output=True)
    if probe.returncode != 0:
        pytest.skip("this compiler has no sanitizer runtimes")
    subprocess.run(["make", "-C", os.path.join(ROOT, "csrc"), "-j", "16", kind, "ASAN_CXX=" + cxx], check=True,
                   capture_output=True)
    lib_dir = os.path.join(ROOT, "csrc", "build", kind)
    exe = tmp_path / ("unit_tests_" + kind)
    subprocess.check_call([cxx, "-std=c++17", "-O1", "-g", flags, "-fno-omit-frame-pointer",
                           "-I" + os.path.join(ROOT, "csrc", "include"), "-I" + os.path.join(ROOT, "csrc", "host"),
                           "-I" + os.path.join(ROOT, "csrc", "kernels"), "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "csrc", "tests", "unit_tests.cc"), "-L" + lib_dir, "-lflagcx",
                           "-Wl,-rpath," + lib_dir, "-lpthread", "-o", str(exe)])
    # the static CUDA runtime keeps process-lifetime allocations; leaks are not what this run is for
    env = dict(os.environ, FLAGCX_DEBUG="WARN", ASAN_OPTIONS="detect_leaks=0:abort_on_error=0",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1", TSAN_OPTIONS="halt_on_error=0")
    for shm in ("1", "0"):  # host ranks over shared-memory rings, then over the socket adaptor
        res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=dict(env, FLAGCX_HOST_SHM=shm))
        assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
        for needle in ("ERROR: AddressSanitizer", "runtime error", "WARNING: ThreadSanitizer"):
            assert needle not in res.stderr, res.stderr[-3000:]
