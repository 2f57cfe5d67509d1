"""The host C++ library under AddressSanitizer + UndefinedBehaviorSanitizer: the library sources and a self-test
driver (csrc/host/selftest/selftest_main.cpp) are compiled with -fsanitize=address,undefined into one executable and
run; any report fails the test."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "mindspore_b200", "csrc", "host")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_library_under_asan_ubsan(tmp_path):
    srcs = [os.path.join(HOST, f) for f in sorted(os.listdir(HOST)) if f.endswith(".cpp")]
    srcs.append(os.path.join(HOST, "selftest", "selftest_main.cpp"))
    exe = str(tmp_path / "selftest")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-pthread", "-o", exe] + srcs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 and "cannot find" in r.stderr and "asan" in r.stderr:
        pytest.skip("the sanitizer runtime is not installed")
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "selftest ok" in r.stdout, (r.stdout + r.stderr)[-4000:]
