"""The C++ scheduler under AddressSanitizer + UndefinedBehaviorSanitizer: a randomised stress driver with small page
pools (preemption, prefix-cache eviction, chunked prefill, aborts, cache resets) checks the scheduling invariants
after every step."""

import os
import shutil
import subprocess

import pytest

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "verl_b200", "csrc")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_scheduler_stress_under_asan_ubsan(tmp_path):
    exe = str(tmp_path / "sched_stress")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
                            "-o", exe, os.path.join(CSRC, "tests", "scheduler_stress.cpp"), os.path.join(CSRC, "scheduler.cpp")],
                           capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and "sanitize" in build.stderr.lower() and "cannot find" in build.stderr.lower():
        pytest.skip("sanitizer runtime libraries are not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    env.pop("LD_PRELOAD", None)
    for seed in (1, 2, 3):
        r = subprocess.run([exe, str(seed), "300"], capture_output=True, text=True, timeout=300, env=env)
        assert r.returncode == 0 and "SCHED_STRESS_OK" in r.stdout, (r.stdout[-500:], r.stderr[-3000:])
        fields = dict(kv.split("=") for kv in r.stdout.split()[2:])
        assert int(fields["finished"]) + int(fields["aborted"]) == 300
        assert int(fields["preempted"]) > 0 and int(fields["prefix_hits"]) > 0  # the hard paths were exercised
