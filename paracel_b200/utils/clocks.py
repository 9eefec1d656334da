"""Sampling of SM clocks and throttle reasons with ``nvidia-smi`` while a timed
region runs (read-only: nothing here changes a GPU setting)."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import tempfile
from typing import Dict, List, Optional

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.tmp = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = subprocess.Popen(
            [exe, "-i", str(self.gpu_index), f"--query-gpu={_QUERY}",
             "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
            stdout=self.tmp, stderr=subprocess.DEVNULL)
        return self

    def stop(self) -> Dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        # one more blocking sample while the GPU is still under the load that was just timed
        try:
            extra = subprocess.run([shutil.which("nvidia-smi"), "-i", str(self.gpu_index),
                                    f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True, timeout=10).stdout
        except Exception:  # noqa: BLE001
            extra = ""
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        rows: List[List[str]] = [[c.strip() for c in ln.split(",")] for ln in list(self.tmp) + extra.splitlines()
                                 if ln.strip()]
        self.tmp.close()
        sm, mx, pw = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                pw.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w_max": max(pw), "samples": len(sm)}
