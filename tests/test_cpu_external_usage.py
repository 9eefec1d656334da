"""The out-of-tree example: Python handler file and the native plug-in built from the template."""
import json
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EX = os.path.join(ROOT, "external_usage")


def _expected():
    hist = {}
    for line in open(os.path.join(EX, "demo_input.txt")):
        for w in line.split():
            hist[len(w)] = hist.get(len(w), 0) + 1
    return {f"len_{k}": v for k, v in hist.items()}


def _run(tmp_path, handler_file):
    cfg = json.load(open(os.path.join(EX, "demo_cfg.json")))
    cfg["input"] = os.path.join(EX, "demo_input.txt")
    cfg["output"] = str(tmp_path / "out") + "/"
    cfg["update_file"] = cfg["filter_file"] = handler_file
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(cfg))
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""),
               PARACEL_RUN_LOG=str(tmp_path / "paracelrun_log"))
    rc = subprocess.run([sys.executable, "-m", "paracel_b200.launch.prun", "-w", "2", "-p", "1", "-c",
                         str(cfg_path), "-m", "local", os.path.join(EX, "demo_app.py")],
                        env=env, cwd=ROOT, timeout=300).returncode
    assert rc == 0
    got = {}
    for line in open(tmp_path / "out" / "histogram_0"):
        k, v = line.rstrip("\n").split("\t")
        got[k] = int(v)
    return got


def test_demo_app_with_python_handlers(tmp_path):
    assert _run(tmp_path, os.path.join(EX, "demo_handlers.py")) == _expected()


@pytest.mark.skipif(shutil.which("g++") is None or shutil.which("make") is None, reason="needs g++ and make")
def test_demo_app_with_native_plugin(tmp_path):
    build = tmp_path / "build"
    shutil.copytree(EX, build)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    subprocess.run([sys.executable, "gen_makefile.py"], cwd=build, env=env, check=True, timeout=120)
    subprocess.run(["make"], cwd=build, check=True, timeout=300)
    assert _run(tmp_path, str(build / "libdemo_handlers.so")) == _expected()
