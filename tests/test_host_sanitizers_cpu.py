"""Sanitizer builds of the host engine of the exchange protocol.

``tests/native/host_protocol_sanitize.cpp`` runs W ranks as threads over one copy of every rank's heap, all thirteen
codecs, three sizes, twelve steps with ranks de-synchronised on purpose and split phases on odd steps.  Built with
ThreadSanitizer the run must be free of data races (the flags are atomics, slots and error-feedback arrays are
plain memory: a slot rewritten while a peer reads it, or read before its flag, would be reported); built with
AddressSanitizer + UBSan it must be free of out-of-bounds accesses and undefined behaviour.  A negative control
(a ready flag raised before the slot is written) must be reported by the ThreadSanitizer build, which shows that
the detector sees these accesses."""
import os
import shutil
import subprocess
import sysconfig

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "grace_b200", "csrc")


def _cuda_include():
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "include", "cuda_runtime.h")):
            return os.path.join(cand, "include")
    return None


def _build(tmp_path, sanitize):
    gxx = shutil.which("g++")
    inc = _cuda_include()
    if gxx is None or inc is None:
        pytest.skip("needs g++ and the CUDA headers")
    probe = tmp_path / "probe.cpp"
    probe.write_text("int main() { return 0; }\n")
    res = subprocess.run([gxx, "-fsanitize=" + sanitize, str(probe), "-o", str(tmp_path / "probe")],
                         capture_output=True, text=True)
    if res.returncode != 0 or subprocess.run([str(tmp_path / "probe")]).returncode != 0:
        pytest.skip("the %s sanitizer runtime is not usable here" % sanitize)
    exe = tmp_path / ("driver_" + sanitize.replace(",", "_"))
    cmd = [gxx, "-std=c++17", "-O1", "-g", "-fsanitize=" + sanitize, "-fno-omit-frame-pointer", "-I", CSRC, "-I", inc,
           os.path.join(ROOT, "tests", "native", "host_protocol_sanitize.cpp"), os.path.join(CSRC, "host_exchange.cpp"),
           "-o", str(exe), "-lpthread", "-lrt"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    return str(exe)


def _env():
    return dict(os.environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66", ASAN_OPTIONS="detect_leaks=1",
                UBSAN_OPTIONS="print_stacktrace=1 halt_on_error=1")


def test_thread_sanitizer_finds_no_race_in_the_protocol_but_finds_a_planted_one(tmp_path):
    exe = _build(tmp_path, "thread")
    res = subprocess.run([exe, "4", "12"], capture_output=True, text=True, timeout=600, env=_env())
    assert res.returncode == 0 and "data race" not in res.stderr, res.stdout[-1000:] + res.stderr[-3000:]
    assert "13 codecs" in res.stdout
    bad = subprocess.run([exe, "broken"], capture_output=True, text=True, timeout=600, env=_env())
    assert bad.returncode != 0 and "data race" in bad.stderr, "the planted race went unreported"


def test_address_and_undefined_behaviour_sanitizers_are_clean(tmp_path):
    exe = _build(tmp_path, "address,undefined")
    res = subprocess.run([exe, "4", "12"], capture_output=True, text=True, timeout=600, env=_env())
    assert res.returncode == 0, res.stdout[-1000:] + res.stderr[-3000:]
    assert "runtime error" not in res.stderr and "AddressSanitizer" not in res.stderr
