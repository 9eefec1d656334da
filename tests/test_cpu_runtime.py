"""Launcher, cluster scheduler (retry, gang semantics, watchdogs), checkpoint / resume,
metrics and phase timers -- all on CPU with host-side fault injection only."""
import json
import os
import subprocess
import sys
import time

import numpy as np

from paracel_b200.launch.cluster import (FAILED, FINISHED, GangScheduler, LocalAgent, SubmitScheduler,
                                         Task, TaskExecutor)
from paracel_b200.launch.local import LocalJob
from workers import cpu_workers as W
from paracel_b200.utils import checkpoint as C
from paracel_b200.utils.metrics import MetricsLogger, PhaseTimer, get_logger

PY = sys.executable
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_prun_local_mode_runs_lr(tmp_path):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((600, 5))
    y = (X @ rng.standard_normal(5) > 0).astype(float)
    inp = tmp_path / "train.csv"
    np.savetxt(str(inp), np.concatenate([X, y[:, None]], 1), delimiter=",", fmt="%.6f")
    cfg = tmp_path / "cfg.json"
    out = tmp_path / "out"
    cfg.write_text(json.dumps({"training_input": str(inp), "output": str(out), "method": "ipm",
                               "rounds": 5, "alpha": 0.01, "beta": 0.0, "update_file": "",
                               "update_func": "lr_theta_update"}))
    r = subprocess.run([PY, "-m", "paracel_b200.launch.prun", "-w", "2", "-p", "1", "-c", str(cfg), "-m",
                        "local", "lr"], cwd=str(tmp_path), env=dict(os.environ, PYTHONPATH=REPO),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "final loss" in r.stdout
    assert len(open(str(out / "lr_theta_0")).read().split("|")) == 6
    log = open(str(tmp_path / "paracelrun_log")).read()
    assert "paracel_b200.ps.server" in log and "--server_info" in log


def test_prun_stops_the_job_when_a_worker_dies(tmp_path):
    bad = tmp_path / "bad.py"
    bad.write_text("import os, sys, time\n"
                   "if os.environ['RANK'] == '1':\n    sys.exit(3)\n"
                   "time.sleep(60)\n")
    t0 = time.time()
    r = subprocess.run([PY, "-m", "paracel_b200.launch.prun", "-w", "2", "-p", "1", "-m", "local", str(bad)],
                       cwd=str(tmp_path), env=dict(os.environ, PYTHONPATH=REPO), capture_output=True,
                       text=True, timeout=120)
    assert r.returncode == 3 and time.time() - t0 < 60


def test_submit_scheduler_retries_and_gives_up(tmp_path):
    flag = tmp_path / "flag"
    flaky = [PY, "-c", f"import os,sys\np={str(flag)!r}\n"
                       "if not os.path.exists(p):\n open(p,'w').close(); sys.exit(1)\n"]
    lines = []
    s = SubmitScheduler([LocalAgent("a", 2)], max_retries=3, out=lines.append, err=lines.append)
    tasks = [Task(0, flaky), Task(1, [PY, "-c", "print('hello from task')"])]
    assert s.run(tasks) and tasks[0].tried == 2 and tasks[1].tried == 1
    assert "hello from task" in lines
    s2 = SubmitScheduler([LocalAgent("a", 1)], max_retries=2, out=lines.append, err=lines.append)
    t = [Task(0, [PY, "-c", "import sys; sys.exit(2)"])]
    assert not s2.run(t) and t[0].tried == 2 and "failed 2 times" in s2.error


def test_gang_scheduler_stops_everything_when_a_started_rank_fails():
    lines = []
    tasks = [Task(0, [PY, "-c", "import time; time.sleep(30)"]),
             Task(1, [PY, "-c", "import time,sys; time.sleep(0.5); sys.exit(1)"])]
    g = GangScheduler([LocalAgent("a", 1), LocalAgent("b", 1)], out=lines.append, err=lines.append)
    t0 = time.time()
    assert not g.run(tasks) and time.time() - t0 < 20
    assert tasks[1].state == FAILED and tasks[0].state != FINISHED and "after the gang started" in g.error
    g2 = GangScheduler([LocalAgent("a", 1)], out=lines.append, err=lines.append)
    assert not g2.run([Task(0, [PY, "-c", "pass"]), Task(1, [PY, "-c", "pass"])])
    assert "not enough slots" in g2.error
    g3 = GangScheduler([LocalAgent("a", 2)], job_timeout_s=1.0, out=lines.append, err=lines.append)
    assert not g3.run([Task(0, [PY, "-c", "import time; time.sleep(30)"])]) and g3.error == "job timeout"
    ok = GangScheduler([LocalAgent("a", 2)], out=lines.append, err=lines.append)
    assert ok.run([Task(0, [PY, "-c", "print(1)"]), Task(1, [PY, "-c", "print(2)"])])


def test_agent_loss_reoffers_tasks():
    a, b = LocalAgent("a", 1), LocalAgent("b", 1)
    s = SubmitScheduler([a, b], max_retries=3, out=lambda s_: None, err=lambda s_: None)
    t = Task(0, [PY, "-c", "import time; time.sleep(1.0)"])
    import threading

    def lose():
        time.sleep(0.3)
        s.agent_lost(t.agent)
    threading.Thread(target=lose, daemon=True).start()
    assert s.run([t]) and t.tried == 2 and t.agent.alive


def test_executor_memory_watchdog_kills_a_hog():
    hog = [PY, "-c", "import time\nx = bytearray(300 * 1024 * 1024)\ntime.sleep(30)"]
    errs = []
    ex = TaskExecutor(Task(0, hog, mem_limit_mb=50), err=errs.append, poll_s=0.1).start()
    t0 = time.time()
    while ex.poll() is None and time.time() - t0 < 25:
        time.sleep(0.1)
    assert ex.poll() is not None and ex.killed_for_memory and any("killed" in e for e in errs)


def test_checkpoint_resume_equals_uninterrupted_run(tmp_path):
    rng = np.random.default_rng(3)
    X = rng.standard_normal((500, 4))
    y = (rng.random(500) < 0.5).astype(float)
    inp = tmp_path / "t.csv"
    np.savetxt(str(inp), np.concatenate([X, y[:, None]], 1), delimiter=",", fmt="%.6f")
    ck = str(tmp_path / "ckpt")
    full = LocalJob(2, 2).run(W.checkpoint_resume, (str(inp), ck, "full"), timeout_s=300)
    LocalJob(2, 2).run(W.checkpoint_resume, (str(inp), ck, "first"), timeout_s=300)
    assert C.exists(ck) and C.load_rank_state(ck, 1)["rank"] == 1
    # resume in a fresh job with a different number of servers
    res = LocalJob(2, 1).run(W.checkpoint_resume, (str(inp), ck, "resume"), timeout_s=300)
    assert np.allclose(res[0], full[0], rtol=1e-12, atol=1e-12)


def test_metrics_and_timers(tmp_path):
    p = str(tmp_path / "m" / "metrics.jsonl")
    m = MetricsLogger(p, rank=0)
    m.log(round=1, loss=0.5, samples_per_s=1e6)
    m.log(round=2, loss=0.4, bytes_pulled=123)
    m.close()
    rows = MetricsLogger.read(p)
    assert [r["round"] for r in rows] == [1, 2] and rows[1]["bytes_pulled"] == 123 and "ts" in rows[0]
    MetricsLogger(str(tmp_path / "x.jsonl"), rank=1).log(a=1)
    assert not os.path.exists(str(tmp_path / "x.jsonl"))
    t = PhaseTimer(use_cuda=False)
    for _ in range(3):
        with t.phase("pull"):
            time.sleep(0.01)
    with t.phase("compute"):
        pass
    s = t.summary()
    assert s["pull"]["count"] == 3 and s["pull"]["ms"] >= 25 and "compute" in s
    t.dump(str(tmp_path / "trace" / "rank0.json"))
    assert json.load(open(str(tmp_path / "trace" / "rank0.json")))["phases"]["pull"]["count"] == 3
    get_logger("t", 0).info("hello")


def test_standalone_proxy_collects_two_server_daemons():
    """The rendezvous proxy as a program: two server daemons report to it, its output is the
    server_info string a worker is started with."""
    import socket
    import subprocess
    import sys
    import time
    from paracel_b200.ps.client import kvclt
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    proxy = subprocess.Popen([sys.executable, "-m", "paracel_b200.launch.proxy", "--nsrv", "2",
                              "--init_port", str(port), "--host", "127.0.0.1", "--timeout", "60"],
                             stdout=subprocess.PIPE, env=env, text=True)
    time.sleep(1.0)
    servers = [subprocess.Popen([sys.executable, "-m", "paracel_b200.ps.server", "--start_host", "127.0.0.1",
                                 "--init_port", str(port)], stdout=subprocess.DEVNULL, env=env)
               for _ in range(2)]
    try:
        out, _ = proxy.communicate(timeout=90)
        eps = [e for e in out.split("_PARACEL_") if e]
        assert len(eps) == 2 and len(set(eps)) == 2
        for n, ep in enumerate(eps):
            host, ports = ep.split(":")
            c = kvclt(host, int(ports.split(",")[0]), timeout_s=10.0)
            assert c.push(f"k{n}", n) and c.pull(f"k{n}") == n
            c.shutdown()
            c.close()
        for p in servers:
            assert p.wait(timeout=30) == 0
    finally:
        for p in servers + [proxy]:
            if p.poll() is None:
                p.kill()
