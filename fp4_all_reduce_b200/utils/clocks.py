"""Clock and throttle-reason sampling around a timed region (nvidia-smi in the background).

The reference project locks the HBM clock for its campaigns and aborts a cell when the lock is lost
(scripts/clk.sh:11-27, scripts/run_cell.sh:17-20).  On shared GPUs nothing may be locked, so every timed
region records what the clocks actually were instead.
"""
from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile
import time
from typing import Optional

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
           "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """with ClockSampler(device_index) as s: ...timed work... ; s.summary() -> dict for the result record."""

    def __init__(self, device_index: int = 0, period_ms: int = 100):
        self.device_index = device_index
        self.period_ms = period_ms
        self._proc: Optional[subprocess.Popen] = None
        self._path: Optional[str] = None
        self._rows: list[list[str]] = []

    def __enter__(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        fd, self._path = tempfile.mkstemp(prefix="fp4ar_clocks_", suffix=".csv")
        os.close(fd)
        out = open(self._path, "w")
        self._proc = subprocess.Popen(
            [exe, f"--id={self.device_index}", f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits",
             "-lms", str(self.period_ms)], stdout=out, stderr=subprocess.DEVNULL)
        out.close()
        time.sleep(0.25)   # let the first sample land before the timed region starts
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            time.sleep(0.05)
            self._proc.terminate()     # the exact child started above
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            with open(self._path) as f:
                self._rows = [[c.strip() for c in line.split(",")] for line in f if line.count(",") >= 8]
            os.unlink(self._path)
        return False

    def summary(self) -> dict:
        sm, mx, pw = [], [], []
        reasons = set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self._rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2])); pw.append(float(r[3]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # samples taken while the GPU was busy: the upper half of the observed power draw
        busy = [s for s, p in zip(sm, pw) if p >= 0.5 * max(pw)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "reasons": sorted(reasons), "samples": len(sm)}
