"""Cluster scheduling of a job's tasks (the role of the reference's Mesos layer,
mesos_scheduler.py:38-822 and mesos_executor.py:30-209, without Mesos).

``Agent`` abstracts "a place that can run a task" (``LocalAgent``: subprocess on this host;
``SshAgent``: a remote host through ssh).  Two schedulers mirror the reference's:

* ``SubmitScheduler``: independent tasks, each retried up to ``max_retries`` times when it
  fails or its agent is lost (mesos_scheduler.py:329-463);
* ``GangScheduler``: all-or-nothing launch of one job's ranks; a task that has not started
  within ``launch_timeout_s`` is re-assigned to another agent, but once the gang has started
  a failing rank stops the whole job ("MPI application can not retry", 575-577, 776-778).

Both enforce a job timeout.  ``TaskExecutor`` is the executor side: it runs the command,
forwards stdout / stderr line by line, and a watchdog kills the task when its resident set
exceeds 1.5 x its memory limit (mesos_executor.py:127-146)."""
from __future__ import annotations

import logging
import os
import shlex
import signal
import subprocess
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

logger = logging.getLogger("paracel.cluster")

PENDING, STARTING, RUNNING, FINISHED, FAILED, LOST, KILLED = (
    "PENDING", "STARTING", "RUNNING", "FINISHED", "FAILED", "LOST", "KILLED")


@dataclass
class Task:
    id: int
    command: List[str]
    env: Dict[str, str] = field(default_factory=dict)
    mem_limit_mb: int = 0
    state: str = PENDING
    tried: int = 0
    agent: Optional["Agent"] = None
    handle: object = None
    start_time: float = 0.0
    exit_code: Optional[int] = None


class TaskExecutor:
    """Runs one task; forwards its output; kills it when it uses too much memory."""

    def __init__(self, task: Task, out: Callable[[str], None] = lambda s: None,
                 err: Callable[[str], None] = lambda s: None, poll_s: float = 0.5):
        self.task, self.out, self.err, self.poll_s = task, out, err, poll_s
        self.proc: Optional[subprocess.Popen] = None
        self.killed_for_memory = False

    def _pump(self, stream, sink):
        for line in iter(stream.readline, ""):
            sink(line.rstrip("\n"))
        stream.close()

    def rss_mb(self) -> float:
        try:
            import psutil
            p = psutil.Process(self.proc.pid)
            rss = p.memory_info().rss
            for c in p.children(recursive=True):
                try:
                    rss += c.memory_info().rss
                except psutil.Error:
                    pass
            return rss / (1 << 20)
        except Exception:  # noqa: BLE001
            return 0.0

    def start(self):
        env = dict(os.environ)
        env.update(self.task.env)
        self.proc = subprocess.Popen(self.task.command, env=env, stdout=subprocess.PIPE,
                                     stderr=subprocess.PIPE, text=True, start_new_session=True)
        threading.Thread(target=self._pump, args=(self.proc.stdout, self.out), daemon=True).start()
        threading.Thread(target=self._pump, args=(self.proc.stderr, self.err), daemon=True).start()
        if self.task.mem_limit_mb > 0:
            threading.Thread(target=self._watch_memory, daemon=True).start()
        return self

    def _watch_memory(self):
        limit = 1.5 * self.task.mem_limit_mb
        while self.proc.poll() is None:
            if self.rss_mb() > limit:
                self.killed_for_memory = True
                self.err(f"task {self.task.id} used more than 1.5 x {self.task.mem_limit_mb} MB: killed")
                self.kill()
                return
            time.sleep(self.poll_s)

    def poll(self) -> Optional[int]:
        return self.proc.poll()

    def kill(self):
        if self.proc and self.proc.poll() is None:
            try:
                os.killpg(self.proc.pid, signal.SIGTERM)
            except (ProcessLookupError, PermissionError):
                self.proc.terminate()
            try:
                self.proc.wait(timeout=3)
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(self.proc.pid, signal.SIGKILL)
                except (ProcessLookupError, PermissionError):
                    self.proc.kill()


class Agent:
    """A slot provider.  ``slots`` tasks may run at once."""

    def __init__(self, name: str, slots: int = 1):
        self.name, self.slots = name, slots
        self.running: List[Task] = []
        self.alive = True

    def free_slots(self) -> int:
        return self.slots - len(self.running) if self.alive else 0

    def launch(self, task: Task, out, err) -> TaskExecutor:
        raise NotImplementedError


class LocalAgent(Agent):
    def launch(self, task: Task, out, err) -> TaskExecutor:
        return TaskExecutor(task, out, err).start()


class SshAgent(Agent):
    """Runs the task on ``host`` through the ssh client binary."""

    def __init__(self, host: str, slots: int = 1, ssh: Sequence[str] = ("ssh", "-o", "BatchMode=yes")):
        super().__init__(host, slots)
        self.ssh = list(ssh)

    def launch(self, task: Task, out, err) -> TaskExecutor:
        envs = " ".join(f"{k}={shlex.quote(v)}" for k, v in task.env.items())
        remote = f"cd {shlex.quote(os.getcwd())} && env {envs} " + " ".join(shlex.quote(c) for c in task.command)
        wrapped = Task(task.id, self.ssh + [self.name, remote], {}, task.mem_limit_mb)
        return TaskExecutor(wrapped, out, err).start()


class _Base:
    def __init__(self, agents: Sequence[Agent], job_timeout_s: float = 24 * 3600.0,
                 out: Callable[[str], None] = print, err: Callable[[str], None] = print,
                 poll_s: float = 0.1):
        self.agents = list(agents)
        self.job_timeout_s, self.out, self.err, self.poll_s = job_timeout_s, out, err, poll_s
        self.tasks: List[Task] = []
        self.error: Optional[str] = None

    def _launch(self, t: Task, a: Agent):
        t.agent, t.state, t.start_time = a, STARTING, time.time()
        t.tried += 1
        a.running.append(t)
        try:
            t.handle = a.launch(t, self.out, self.err)
            t.state = RUNNING
        except Exception as e:  # noqa: BLE001
            logger.error("launch of task %d on %s failed: %s", t.id, a.name, e)
            a.running.remove(t)
            t.state, t.agent = LOST, None

    def _reap(self, t: Task):
        if t.state != RUNNING:
            return
        rc = t.handle.poll()
        if rc is None:
            return
        t.exit_code = rc
        t.agent.running.remove(t)
        t.state = FINISHED if rc == 0 else FAILED

    def agent_lost(self, agent: Agent):
        """Mark an agent dead: its tasks are killed and reported LOST (executorLost / slaveLost)."""
        agent.alive = False
        for t in list(agent.running):
            if t.handle:
                t.handle.kill()
            agent.running.remove(t)
            t.state, t.agent = LOST, None

    def kill_all(self):
        for t in self.tasks:
            if t.state == RUNNING and t.handle:
                t.handle.kill()
                if t.agent and t in t.agent.running:
                    t.agent.running.remove(t)
                t.state = KILLED


class SubmitScheduler(_Base):
    def __init__(self, agents, max_retries: int = 3, **kw):
        super().__init__(agents, **kw)
        self.max_retries = max_retries

    def run(self, tasks: Sequence[Task]) -> bool:
        self.tasks = list(tasks)
        t0 = time.time()
        while True:
            for t in self.tasks:
                self._reap(t)
                if t.state in (FAILED, LOST):
                    if t.tried < self.max_retries:
                        logger.warning("task %d %s (try %d): retry", t.id, t.state, t.tried)
                        t.state = PENDING
                    else:
                        self.error = f"task {t.id} failed {t.tried} times"
                        self.kill_all()
                        return False
            for t in self.tasks:
                if t.state == PENDING:
                    a = next((a for a in self.agents if a.free_slots() > 0), None)
                    if a is not None:
                        self._launch(t, a)
            if all(t.state == FINISHED for t in self.tasks):
                return True
            if time.time() - t0 > self.job_timeout_s:
                self.error = "job timeout"
                self.kill_all()
                return False
            if not any(a.alive for a in self.agents):
                self.error = "no agent left"
                return False
            time.sleep(self.poll_s)


class GangScheduler(_Base):
    def __init__(self, agents, launch_timeout_s: float = 30.0, **kw):
        super().__init__(agents, **kw)
        self.launch_timeout_s = launch_timeout_s
        self.started = False

    def run(self, tasks: Sequence[Task]) -> bool:
        self.tasks = list(tasks)
        if sum(a.free_slots() for a in self.agents) < len(self.tasks):
            self.error = "not enough slots for a gang launch"
            return False
        t0 = time.time()
        while True:
            for t in self.tasks:
                self._reap(t)
            running = [t for t in self.tasks if t.state in (RUNNING, FINISHED)]
            if not self.started and len(running) == len(self.tasks):
                self.started = True
            bad = [t for t in self.tasks if t.state in (FAILED, LOST)]
            if bad:
                if self.started or any(t.state == FAILED for t in bad):
                    # once a rank of a started gang fails the whole job stops: ranks cannot be retried
                    self.error = f"task {bad[0].id} {bad[0].state} after the gang started"
                    self.kill_all()
                    return False
                for t in bad:  # lost before the gang was complete: re-offer
                    t.state = PENDING
            for t in self.tasks:
                if t.state == PENDING:
                    a = next((a for a in self.agents if a.free_slots() > 0), None)
                    if a is None:
                        if time.time() - t0 > self.launch_timeout_s:
                            self.error = "launch timeout: no free slot"
                            self.kill_all()
                            return False
                        continue
                    self._launch(t, a)
            if all(t.state == FINISHED for t in self.tasks):
                return True
            if time.time() - t0 > self.job_timeout_s:
                self.error = "job timeout"
                self.kill_all()
                return False
            time.sleep(self.poll_s)


def read_hostfile(path: Optional[str], ppn: int) -> List[Agent]:
    if not path:
        return [LocalAgent("localhost", slots=1 << 20)]
    agents: List[Agent] = []
    with open(path) as f:
        for line in f:
            h = line.strip()
            if h and not h.startswith("#"):
                agents.append(LocalAgent(h, ppn) if h in ("localhost", "127.0.0.1") else SshAgent(h, ppn))
    return agents


def run_cluster_job(args, command: List[str]) -> int:
    """``prun -m cluster``: servers through a SubmitScheduler (restartable), workers as a gang."""
    from .local import free_port
    from .prun import shutdown_servers, start_servers, worker_command
    servers, info = start_servers(args.snum, init_port=args.init_port)
    try:
        cmd = worker_command(command, info, args.cfg_file)
        port = free_port()
        master = os.environ.get("MASTER_ADDR", "127.0.0.1")
        tasks = [Task(r, cmd, {"RANK": str(r), "WORLD_SIZE": str(args.wnum), "LOCAL_RANK": str(r % max(args.ppn, 1)),
                               "MASTER_ADDR": master, "MASTER_PORT": str(port)}, args.mem_limit)
                 for r in range(args.wnum)]
        sch = GangScheduler(read_hostfile(args.hostfile, args.ppn), job_timeout_s=args.timeout)
        ok = sch.run(tasks)
        if not ok:
            logger.error("job failed: %s", sch.error)
        return 0 if ok else 1
    finally:
        shutdown_servers(info, servers)
