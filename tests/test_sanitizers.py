"""Host code under AddressSanitizer + UndefinedBehaviorSanitizer and under ThreadSanitizer (CPU only).

Builds tests/native/core_stress.cpp twice and runs it: the page pool, the wire reader on mutated bytes and the
controller-in-simulator under ASan/UBSan, the flag, ticket, all-reduce rendezvous and two-source KV-push protocols (CPU-thread emulation of what the kernels do) under TSan.
"""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "native", "core_stress.cpp")
INC = os.path.join(os.path.dirname(HERE), "blitz_scale_b200", "csrc")


def _build(tmp_path, name, flags):
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++20", "-O1", "-g", *flags, f"-I{INC}", SRC, "-o", exe, "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if r.returncode != 0 and ("cannot find" in r.stderr or "unrecognized" in r.stderr):
        pytest.skip(f"sanitizer runtime not installed: {r.stderr[-200:]}")
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_core_under_asan_ubsan(tmp_path):
    exe = _build(tmp_path, "cs_asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"])
    for part in ("pool", "wire", "sim"):
        r = subprocess.run([exe, part], capture_output=True, text=True, timeout=600,
                           env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0"))
        assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_protocols_under_tsan(tmp_path):
    exe = _build(tmp_path, "cs_tsan", ["-fsanitize=thread"])
    for part in ("flags", "tickets", "allreduce", "kvpush"):
        r = subprocess.run([exe, part], capture_output=True, text=True, timeout=600,
                           env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1"))
        assert r.returncode == 0 and "OK" in r.stdout and "WARNING: ThreadSanitizer" not in r.stderr, \
            r.stdout[-2000:] + r.stderr[-4000:]
