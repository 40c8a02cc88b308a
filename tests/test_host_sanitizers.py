"""The native host structures under the address / undefined-behaviour sanitizers and under the thread
sanitizer: `csrc/host/tests/host_stress.cpp` drives the polled ring and the shared-memory channel from
several threads (payloads in plain memory, so a missing acquire / release shows up as a data race) and the
page store through a random operation mix with its invariants."""
import shutil
import subprocess
from pathlib import Path

import pytest

SRC = Path(__file__).resolve().parents[1] / "pie_b200" / "csrc" / "host" / "tests" / "host_stress.cpp"


def _has(lib: str) -> bool:
    out = subprocess.run(["gcc", f"-print-file-name={lib}"], capture_output=True, text=True).stdout.strip()
    return "/" in out


@pytest.mark.parametrize("flags,lib", [("address,undefined", "libasan.so"), ("thread", "libtsan.so")])
def test_host_structures_are_clean_under_sanitizers(tmp_path, flags, lib):
    if shutil.which("g++") is None or not _has(lib):
        pytest.skip(f"g++ or {lib} not available")
    exe = tmp_path / "host_stress"
    subprocess.run(["g++", "-std=c++20", "-O1", "-g", f"-fsanitize={flags}", "-fno-omit-frame-pointer", "-Wno-tsan",
                    "-pthread", str(SRC), "-o", str(exe), "-lrt"], check=True)
    env = {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "halt_on_error=1",
           "TSAN_OPTIONS": "halt_on_error=1", "PATH": "/usr/bin:/bin"}
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-4000:]
    assert "host stress: ok" in r.stdout and "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr
