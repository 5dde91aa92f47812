"""Campaign driver and clock control, on the host only: cells are tiny python children, NVML is a fake."""
import json
import os

import pytest

from fp4_all_reduce_b200.harness import campaign as C
from fp4_all_reduce_b200.utils import clock_control as K


def _write_child(tmp_path, name, body):
    p = tmp_path / name
    p.write_text(body)
    return str(p)


def test_parse_cells_and_commands(tmp_path):
    cells = C.parse_cells("""
# comment
tp2_ar 2 600 NCCL_PROTO=Simple FOO=bar -- bench_cli --rows 1024 --nccl
ops    1 120 -- ops_bench --rows 4096
mine   1 60  -- some/script.py --x 1
dotted 4 60  -- pkg.mod --y
nt     2 60  -- nccl_tuned --nproc 2
""")
    assert [c.name for c in cells] == ["tp2_ar", "ops", "mine", "dotted", "nt"]
    assert cells[0].env == {"NCCL_PROTO": "Simple", "FOO": "bar"} and cells[0].gpus == 2 and cells[0].timeout_s == 600
    cmd = C.build_command(cells[0], str(tmp_path), 29711, python="py")
    assert cmd[:4] == ["py", "-m", "torch.distributed.run", "--nnodes=1"]
    assert "--nproc-per-node=2" in cmd and "127.0.0.1" in cmd and "29711" in cmd
    assert cmd[cmd.index("fp4_all_reduce_b200.harness.bench_cli") - 1] == "-m"
    assert cmd[-4:] == ["--out", os.path.join(str(tmp_path), "tp2_ar.jsonl"), "--tag", "tp2_ar"]
    assert C.build_command(cells[1], str(tmp_path), 1, python="py") == \
        ["py", "-m", "fp4_all_reduce_b200.harness.ops_bench", "--rows", "4096"]
    assert C.build_command(cells[2], str(tmp_path), 1, python="py") == ["py", "some/script.py", "--x", "1"]
    assert C.build_command(cells[3], str(tmp_path), 1, python="py")[-3:] == ["-m", "pkg.mod", "--y"]
    assert "torch.distributed.run" not in C.build_command(cells[4], str(tmp_path), 1, python="py")
    single = C.parse_cells("s 4 60 LAUNCH=single -- some/driver.py --tp 4")[0]
    assert C.build_command(single, str(tmp_path), 1, python="py") == ["py", "some/driver.py", "--tp", "4"]
    with pytest.raises(ValueError):
        C.parse_cells("a 1 10 bench_cli")            # no '--'
    with pytest.raises(ValueError):
        C.parse_cells("a 1 10 -- x\na 1 10 -- y")    # duplicate name
    with pytest.raises(ValueError):
        C.parse_cells("a 9 10 -- x")                 # too many GPUs


def test_campaign_runs_times_out_and_resumes(tmp_path):
    ok = _write_child(tmp_path, "ok.py", "import sys; print('hello'); sys.exit(0)\n")
    bad = _write_child(tmp_path, "bad.py", "import sys; sys.exit(7)\n")
    slow = _write_child(tmp_path, "slow.py", "import time; time.sleep(60)\n")
    cells = C.parse_cells(f"a 1 30 -- {ok}\nb 1 30 -- {bad}\nc 1 1 -- {slow}\n")
    out = str(tmp_path / "runs")
    msgs = []
    rc = C.run_campaign(cells, out, echo=msgs.append, lock_dir=str(tmp_path / "locks"))
    assert rc == 0
    st = C.load_state(os.path.join(out, "campaign_state.jsonl"))
    assert st["a"]["rc"] == 0 and st["b"]["rc"] == 7
    assert st["c"]["rc"] == 124 and st["c"]["timed_out"] is True and st["c"]["seconds"] < 20
    assert "hello" in open(os.path.join(out, "a.log")).read()
    assert not os.path.exists(os.path.join(out, "a.jsonl"))            # nothing that looks like a record was printed
    assert os.listdir(str(tmp_path / "locks")) == []          # every lock released
    # resume: only the failed cells run again
    msgs.clear()
    C.run_campaign(cells[:2], out, resume=True, echo=msgs.append)
    assert "SKIP a (done)" in msgs and any(m.startswith("START b") for m in msgs)


def test_campaign_deadline_clock_abort_and_rejection(tmp_path):
    out = str(tmp_path / "runs")
    os.makedirs(out)
    # a child that writes a record with a thermal slow-down on its first run only
    marker = tmp_path / "ran_once"
    child = _write_child(tmp_path, "therm.py", f"""
import json, os, sys
first = not os.path.exists({str(marker)!r})
open({str(marker)!r}, 'w').close()
with open(os.path.join({out!r}, 'hot.jsonl'), 'w') as f:
    f.write(json.dumps({{"kind": "timing", "med_us": 1.0, "reasons": ["sw_thermal_slowdown"] if first else ["sw_power_cap"]}}) + "\\n")
""")
    cells = C.parse_cells(f"hot 1 30 -- {child}\nlate 1 500 -- {child}\n")
    t = [1000.0]
    msgs = []
    rc = C.run_campaign(cells, out, deadline=1400.0, now=lambda: t[0], echo=msgs.append)
    assert rc == 0
    assert "SKIP late (deadline)" in msgs
    assert os.path.exists(os.path.join(out, "hot.jsonl.rejected"))
    assert C.slowdown_reasons(os.path.join(out, "hot.jsonl")) == []          # power cap alone is kept
    attempts = [json.loads(l) for l in open(os.path.join(out, "campaign_state.jsonl")) if '"hot"' in l]
    assert [a["attempt"] for a in attempts] == [1, 2] and attempts[0]["slowdown"] == ["sw_thermal_slowdown"]
    # clock guard: a read-back that differs stops the campaign with code 3 before anything runs
    msgs.clear()
    rc = C.run_campaign(cells[:1], str(tmp_path / "r2"), expect_mem_mhz=3996, clock_reader=lambda g: [3996 - 1],
                        echo=msgs.append)
    assert rc == 3 and msgs[0].startswith("CLOCK_ABORT")
    rc = C.run_campaign(cells[:1], str(tmp_path / "r3"), expect_mem_mhz=3996, clock_reader=lambda g: [3996], echo=msgs.append)
    assert rc == 0


def test_gpu_locks_exclusive_and_stale(tmp_path):
    d = str(tmp_path / "locks")
    a = C.GpuLocks(d, pid_alive=lambda pid: True)
    assert a.acquire(2, total=3) == [0, 1]
    b = C.GpuLocks(d, pid_alive=lambda pid: True)
    assert b.acquire(2, total=3) is None and b.held == []     # only one GPU left: nothing kept
    assert b.acquire(1, total=3) == [2]
    a.release(); b.release()
    assert os.listdir(d) == []
    a.acquire(1, total=1)
    c = C.GpuLocks(d, pid_alive=lambda pid: False)             # the owner died: the lock is taken over
    assert c.acquire(1, total=1) == [0]


def test_dry_run_and_deadline_parse(tmp_path, capsys):
    f = tmp_path / "cells.txt"
    f.write_text("x 2 60 -- gate_dist --rows 64\n")
    assert C.main([str(f), "--out", str(tmp_path / "o"), "--dry-run"]) == 0
    outp = capsys.readouterr().out
    assert "torch.distributed.run" in outp and "gate_dist" in outp
    assert C.parse_deadline(None, 0.0) == 0.0 and C.parse_deadline("12345", 0.0) == 12345.0 and C.parse_deadline("+90", 1000.0) == 1090.0
    assert C.parse_deadline("23:59", 1_700_000_000.0) > 0


# ------------------------------------------------------------------------------------------ clock control
class FakeNvml:
    NVML_CLOCK_MEM = 2

    def __init__(self, n, default=3996, obey=True):
        self.clk = [default] * n
        self.default, self.obey, self.calls = default, obey, []

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetClockInfo(self, h, kind):
        assert kind == self.NVML_CLOCK_MEM
        return self.clk[h]

    def nvmlDeviceSetMemoryLockedClocks(self, h, lo, hi):
        self.calls.append(("lock", h, lo, hi))
        if self.obey:
            self.clk[h] = lo

    def nvmlDeviceResetMemoryLockedClocks(self, h):
        self.calls.append(("reset", h))
        if self.obey:
            self.clk[h] = self.default


def test_clock_control_is_off_by_default(tmp_path, monkeypatch):
    nv = FakeNvml(2)
    monkeypatch.delenv("FP4AR_ALLOW_CLOCK_CONTROL", raising=False)
    cc = K.ClockControl([0, 1], str(tmp_path), nvml=nv, sleep=lambda s: None)
    assert cc.read() == [3996, 3996]
    with pytest.raises(K.ClockControlDisabled):
        cc.lock(3200)
    cc2 = K.ClockControl([0, 1], str(tmp_path), allow=True, nvml=nv, sleep=lambda s: None)
    with pytest.raises(K.ClockControlDisabled):      # the environment switch is missing
        cc2.reset(3996)
    monkeypatch.setenv("FP4AR_ALLOW_CLOCK_CONTROL", "1")
    with pytest.raises(K.ClockControlDisabled):      # the constructor switch is missing
        cc.lock(3200)
    assert nv.calls == []


def test_clock_control_lock_reset_guard_against_fake_nvml(tmp_path, monkeypatch):
    monkeypatch.setenv("FP4AR_ALLOW_CLOCK_CONTROL", "1")
    nv = FakeNvml(2)
    cc = K.ClockControl([0, 1], str(tmp_path), allow=True, nvml=nv, sleep=lambda s: None)
    assert cc.lock(3200)["state"] == K.LOCKED and cc.read() == [3200, 3200] and cc.check(3200) == []
    assert cc.check(3996) == [0, 1]
    assert cc.reset(3996)["state"] == K.RESET_VERIFIED and cc.read() == [3996, 3996]
    n = len(nv.calls)
    assert cc.reset(3996)["state"] == K.RESET_VERIFIED and len(nv.calls) == n      # idempotent
    # a driver that ignores the request: the read-back catches it
    nv2 = FakeNvml(2, obey=False)
    cc2 = K.ClockControl([0, 1], str(tmp_path / "b"), allow=True, nvml=nv2, sleep=lambda s: None)
    assert cc2.lock(3200)["state"] == K.LOCK_FAILED
    nv2.clk = [3200, 3200]
    assert cc2.reset(3996)["state"] == K.RESET_UNVERIFIED
    # guard: fires at the deadline and resets what is still locked
    nv3 = FakeNvml(1)
    cc3 = K.ClockControl([0], str(tmp_path / "c"), allow=True, nvml=nv3, sleep=lambda s: None)
    cc3.lock(3200)
    t = iter([0.0, 5.0, 11.0, 12.0])
    assert cc3.guard(10.0, 3996, now=lambda: next(t))["state"] == K.RESET_VERIFIED
    assert nv3.clk == [3996]
    assert "guard fired" in open(os.path.join(str(tmp_path / "c"), "CLOCK.log")).read()


def test_printed_records_are_harvested(tmp_path):
    child = _write_child(tmp_path, "p.py", "print('noise'); print('{\"op\": \"x\", \"us\": 1.5}'); print('{broken')\n")
    out = str(tmp_path / "runs")
    assert C.run_campaign(C.parse_cells(f"p 1 30 -- {child}\n"), out, echo=lambda m: None) == 0
    lines = open(os.path.join(out, "p.jsonl")).read().splitlines()
    assert [json.loads(l) for l in lines] == [{"op": "x", "us": 1.5}]


def test_shipped_cell_files_parse_and_name_real_programs():
    import importlib.util
    from pathlib import Path

    root = Path(C.__file__).resolve().parent
    files = sorted((root / "cells").glob("*.txt"))
    assert len(files) >= 4
    for f in files:
        cells = C.parse_cells(f.read_text())
        assert cells, f
        for c in cells:
            if c.program.endswith(".py"):
                assert (root.parent.parent / c.program).exists(), (f.name, c.program)
            else:
                assert c.program in C.HARNESS_MODULES, (f.name, c.program)
                assert importlib.util.find_spec(f"fp4_all_reduce_b200.harness.{c.program}") is not None
            assert c.gpus in (1, 2, 4, 8) and 30 <= c.timeout_s <= 900
