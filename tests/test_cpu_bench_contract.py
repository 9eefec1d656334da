"""bench.py contract pieces that need no GPU: the reference arm answers with one JSON line (a
measurement when a reference build is installed under baseline/_ref, else the reason it is not),
and the launcher's run log can be redirected."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    from benchmarks.reference_arm import find_reference_install
    if find_reference_install() is None:
        assert "unavailable" in d and "baseline/_ref" in d["unavailable"]
    else:
        assert d["metric"].startswith("rating updates/s") and d["value"] > 0


def test_run_log_path_comes_from_the_environment(tmp_path, monkeypatch):
    from paracel_b200.launch import prun
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("PARACEL_RUN_LOG", str(tmp_path / "elsewhere.log"))
    prun._log_cmd(["a", "b"])
    assert (tmp_path / "elsewhere.log").read_text() == "a b\n"
    monkeypatch.setenv("PARACEL_RUN_LOG", "")
    prun._log_cmd(["c"])
    assert not (tmp_path / "paracelrun_log").exists()
    monkeypatch.delenv("PARACEL_RUN_LOG")
    prun._log_cmd(["d"])
    assert (tmp_path / "paracelrun_log").read_text() == "d\n"
