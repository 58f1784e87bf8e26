"""The host runtime library under AddressSanitizer and UndefinedBehaviorSanitizer (the reference ships no
sanitizer configuration; the GPU-side counterpart, compute-sanitizer, is not available where this runs)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "zml_b200", "csrc", "host")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_library_is_clean_under_asan_and_ubsan(tmp_path):
    exe = str(tmp_path / "host_sanitize")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", os.path.join(ROOT, "tests", "native", "host_sanitize_main.cpp"),
           os.path.join(HOST, "file_stream.cpp"), os.path.join(HOST, "tracer.cpp"), "-o", exe, "-lpthread", "-ldl"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=300, env=env)
    assert run.returncode == 0, (run.stdout[-2000:], run.stderr[-4000:])
    assert "HOST_SANITIZE_OK" in run.stdout
    assert "runtime error" not in run.stderr and "AddressSanitizer" not in run.stderr
