"""The host runtime's concurrent pieces under ThreadSanitizer and AddressSanitizer/UBSan (CPU only)."""
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "crosspool_b200" / "csrc"
SOURCES = [CSRC / "tests" / "stress_runtime.cpp", CSRC / "runtime" / "capi.cpp", CSRC / "runtime" / "shmem.cpp",
           CSRC / "runtime" / "kv_vmm.cpp"]


@pytest.mark.parametrize("name,flags", [("tsan", ["-fsanitize=thread"]), ("asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=all"])])
def test_runtime_stress_is_clean_under_sanitizers(tmp_path, name, flags):
    exe = tmp_path / f"stress_{name}"
    cmd = ["g++", "-std=c++20", "-O1", "-g", "-pthread", *flags, f"-I{CSRC / 'include'}", *map(str, SOURCES), "-o", str(exe), "-lrt"]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66", ASAN_OPTIONS="detect_leaks=1")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "stress_runtime ok" in r.stdout, (r.stdout + r.stderr)[-4000:]
