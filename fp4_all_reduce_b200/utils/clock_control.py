"""Memory-clock lock / reset with read-back verification, for dedicated machines only.  OFF by default.

The reference project pins the HBM clock for a measurement campaign and verifies the pin by reading the
clock back on every GPU; a state file per node records LOCKED / LOCK_FAILED / RESET_VERIFIED /
RESET_UNVERIFIED and a guard resets the clocks at a deadline (scripts/clk.sh:11-27, scripts/guard.sh:1-6).

This module keeps that behaviour behind two switches, because a lock outlives the process and the next user
of a shared GPU inherits it: `ClockControl(..., allow=True)` AND the environment variable
`FP4AR_ALLOW_CLOCK_CONTROL=1`.  Without both, `lock()` and `reset()` raise `ClockControlDisabled` before they
touch NVML; `read()` always works.  The NVML binding is injected (`nvml=`), so the logic is testable against a
fake on a machine without a GPU; nothing in this package calls `lock()` or `reset()` on its own.
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional, Sequence

LOCKED, LOCK_FAILED = "LOCKED", "LOCK_FAILED"
RESET_VERIFIED, RESET_UNVERIFIED = "RESET_VERIFIED", "RESET_UNVERIFIED"


class ClockControlDisabled(RuntimeError):
    pass


def _default_nvml():
    import pynvml

    pynvml.nvmlInit()
    return pynvml


class ClockControl:
    """Lock / reset / read the memory clock of a set of GPUs with read-back verification and a state file."""

    def __init__(self, gpus: Sequence[int], state_dir: str, *, allow: bool = False, nvml=None,
                 settle_s: float = 2.0, sleep=time.sleep):
        self.gpus = list(gpus)
        self.state_dir = state_dir
        self.allow = bool(allow)
        self._nvml = nvml
        self.settle_s = settle_s
        self._sleep = sleep
        os.makedirs(state_dir, exist_ok=True)

    # ---- plumbing -------------------------------------------------------------------------------------
    @property
    def nvml(self):
        if self._nvml is None:
            self._nvml = _default_nvml()
        return self._nvml

    def _enabled(self) -> bool:
        return self.allow and os.environ.get("FP4AR_ALLOW_CLOCK_CONTROL") == "1"

    def _require(self, what: str):
        if not self._enabled():
            raise ClockControlDisabled(
                f"{what}: clock control is off (needs allow=True and FP4AR_ALLOW_CLOCK_CONTROL=1); "
                "a clock lock outlives the process and is inherited by the GPU's next user")

    def _log(self, line: str):
        with open(os.path.join(self.state_dir, "CLOCK.log"), "a") as f:
            f.write(time.strftime("%Y-%m-%d %H:%M:%S ") + line + "\n")

    def _state_path(self) -> str:
        return os.path.join(self.state_dir, "clock_state.json")

    def state(self) -> Optional[dict]:
        try:
            with open(self._state_path()) as f:
                return json.load(f)
        except (OSError, json.JSONDecodeError):
            return None

    def _set_state(self, state: str, readback, why: str = ""):
        rec = {"state": state, "readback_mhz": readback, "why": why, "time": time.time()}
        with open(self._state_path(), "w") as f:
            json.dump(rec, f)
        self._log(f"STATE={state} readback={readback} {why}")
        return rec

    # ---- operations -----------------------------------------------------------------------------------
    def read(self) -> list[int]:
        """Current memory clock (MHz) of every GPU of the set."""
        n = self.nvml
        out = []
        for g in self.gpus:
            h = n.nvmlDeviceGetHandleByIndex(g)
            out.append(int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_MEM)))
        return out

    def lock(self, mhz: int) -> dict:
        """Pin the memory clock of every GPU to `mhz`, then verify by reading it back."""
        self._require("lock")
        n = self.nvml
        self._log(f"LOCK {mhz} before={self.read()}")
        for g in self.gpus:
            n.nvmlDeviceSetMemoryLockedClocks(n.nvmlDeviceGetHandleByIndex(g), mhz, mhz)
        self._sleep(self.settle_s)
        rb = self.read()
        ok = all(v == mhz for v in rb)
        return self._set_state(LOCKED if ok else LOCK_FAILED, rb, f"target={mhz}")

    def reset(self, default_mhz: int, why: str = "planned") -> dict:
        """Undo the pin; verified when every GPU reads `default_mhz` afterwards.  Idempotent."""
        self._require("reset")
        st = self.state()
        if st and st.get("state") == RESET_VERIFIED:
            return st
        n = self.nvml
        self._log(f"RESET ({why})")
        for g in self.gpus:
            n.nvmlDeviceResetMemoryLockedClocks(n.nvmlDeviceGetHandleByIndex(g))
        self._sleep(self.settle_s)
        rb = self.read()
        ok = all(v == default_mhz for v in rb)
        return self._set_state(RESET_VERIFIED if ok else RESET_UNVERIFIED, rb, why)

    def guard(self, at_epoch: float, default_mhz: int, now=time.time, poll_s: float = 10.0) -> Optional[dict]:
        """Back-stop: wait until `at_epoch`, then reset unless the state is already RESET_VERIFIED."""
        self._require("guard")
        while now() < at_epoch:
            self._sleep(poll_s)
        st = self.state()
        if st and st.get("state") == RESET_VERIFIED:
            return st
        self._log("guard fired")
        return self.reset(default_mhz, why="guard")

    def check(self, expected_mhz: int) -> list[int]:
        """GPUs whose memory clock differs from `expected_mhz` (a cell is aborted when this is non-empty)."""
        return [g for g, v in zip(self.gpus, self.read()) if v != expected_mhz]
