"""Host runtime under ThreadSanitizer and AddressSanitizer: a native stress program against the
TCP parameter server (the reference serves reads outside its mutex; this store may not race)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "native", "ps_stress.cpp")
INC = os.path.join(ROOT, "paracel_b200", "csrc", "core")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
@pytest.mark.parametrize("san", ["thread", "address"])
def test_parameter_server_stress_is_clean_under_sanitizer(tmp_path, san):
    exe = tmp_path / f"ps_stress_{san}"
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={san}", "-fno-omit-frame-pointer", "-I", INC,
           SRC, "-o", str(exe), "-lpthread", "-ldl"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if build.returncode != 0 and "sanitize" in build.stderr and "cannot find" in build.stderr:
        pytest.skip(f"lib{san[0]}san is not installed")
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66", ASAN_OPTIONS="detect_leaks=1:exitcode=66")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0, (run.stdout[-2000:], run.stderr[-4000:])
    assert run.stdout.startswith("ok 3200")
