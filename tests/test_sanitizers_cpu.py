"""The C++ runtime under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer:
a stand-alone harness (csrc/tests/runtime_sanitize.cpp) drives the scheduler, block manager, prefix
cache and page pool from two threads; any report makes the binary exit non-zero."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "xllm_b200", "csrc")


@pytest.mark.parametrize("mode,flags", [("asan_ubsan", ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"]),
                                        ("tsan", ["-fsanitize=thread"])])
def test_runtime_under_sanitizers(mode, flags, tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / f"rt_{mode}")
    cmd = [cxx, "-std=c++17", "-O1", "-g", *flags, "-I", os.path.join(CSRC, "runtime"), "-I", "/usr/local/cuda/include",
           os.path.join(CSRC, "tests", "runtime_sanitize.cpp"), "-o", exe, "-pthread", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    if r.returncode != 0 and "sanitize" in r.stderr and "cannot find" in r.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert r.returncode == 0, r.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "RUNTIME_SANITIZE_OK" in r.stdout, (r.stdout[-1000:], r.stderr[-3000:])
