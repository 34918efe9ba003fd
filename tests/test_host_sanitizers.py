"""The C++ host runtime under AddressSanitizer + UndefinedBehaviorSanitizer: the randomised serving-loop driver in
csrc/host/tests/host_fuzz.cc (tiny block pools, shared prefixes, chunked prefill, drafts, forks, aborts, swap and
recompute pre-emption, non-prefix reuse, pipeline micro-batches) is built with both sanitizers and must finish
without a report and with every block back in the pool."""
import os
import shutil
import subprocess

import pytest

HOST = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ksanallm_b200", "csrc", "host")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_host_runtime_fuzz_under_asan_and_ubsan(tmp_path):
    exe = str(tmp_path / "host_fuzz")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined",
                            "-fno-sanitize-recover=all", "-I", HOST, os.path.join(HOST, "tests", "host_fuzz.cc"),
                            "-o", exe], capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip("sanitizer runtimes are not installed")
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe, "80", "7"], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0"))
    assert run.returncode == 0, run.stdout + run.stderr
    assert "80 rounds ok" in run.stdout and "flexible-hit tokens" in run.stdout
