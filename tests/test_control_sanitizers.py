"""The C++ control plane under ThreadSanitizer and AddressSanitizer: a multi-threaded stress
program (tests/cpp/control_stress.cpp) is built against the control-plane sources with the
sanitizer and must finish without a report.  The reference has no sanitizer coverage of its
Rust control plane; the data races this guards against live in the per-connection server
threads, the quorum rounds of the manager and the lighthouse's tick thread."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CONTROL = ROOT / "torchft_b200" / "csrc" / "control"
SOURCES = [p for p in sorted(CONTROL.glob("*.cpp")) if p.name != "bindings.cpp"]


@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_control_plane_under_sanitizer(sanitizer, tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = tmp_path / f"control_stress_{sanitizer}"
    cmd = [cxx, "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", f"-I{CONTROL}",
           str(ROOT / "tests" / "cpp" / "control_stress.cpp"), *map(str, SOURCES), "-o", str(exe), "-lpthread"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip(f"lib{sanitizer[0]}san is not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0 second_deadlock_stack=1", ASAN_OPTIONS="detect_leaks=1")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    report = run.stderr
    assert "ThreadSanitizer" not in report and "AddressSanitizer" not in report and "LeakSanitizer" not in report, report[-6000:]
    assert run.returncode == 0, (run.stdout[-2000:], report[-3000:])
    assert "control stress ok" in run.stdout
