"""The host layer (block manager, requests, scheduler with removal / preemption / admission hold, batch
builder) under AddressSanitizer and UndefinedBehaviorSanitizer: dmlx_b200/csrc/host.cpp is compiled
with -fsanitize=address,undefined together with tests/sanitize/host_stress.cpp, which drives random
workloads against it (a small in-memory fake stands in for the device page pool) and checks the
block-accounting invariants after every operation.  Any sanitizer report or failed invariant fails
the test.  No GPU is involved: this is the stand-in for running the host code under a memory checker."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_layer_under_asan_ubsan(tmp_path):
    exe = str(tmp_path / "host_stress")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "dmlx_b200", "csrc"),
           os.path.join(ROOT, "dmlx_b200", "csrc", "host.cpp"), os.path.join(ROOT, "tests", "sanitize", "host_stress.cpp"),
           "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 and "sanitize" in r.stderr and "cannot find" in r.stderr:
        pytest.skip("sanitizer runtime not installed")
    assert r.returncode == 0, r.stderr
    for seed in ("1", "2", "3"):
        run = subprocess.run([exe, seed], capture_output=True, text=True, timeout=300,
                             env={**os.environ, "ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"})
        assert run.returncode == 0, run.stdout + run.stderr
        assert "host stress ok" in run.stdout
        assert "AddressSanitizer" not in run.stderr and "runtime error" not in run.stderr, run.stderr
