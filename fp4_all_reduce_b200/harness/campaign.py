"""Measurement campaign driver: runs a file of cells one after another, each as its own process tree with a
time limit, with per-GPU locks, a wall-clock deadline, resume, and a clock guard.

    python -m fp4_all_reduce_b200.harness.campaign cells.txt --out runs/ [--deadline HH:MM | +SECONDS] [--resume]
        [--expect-mem-mhz 3996] [--dry-run] [--lock-dir /tmp/fp4ar_locks] [--port 29700]

Cell file, one cell per line ('#' and blank lines ignored):

    <cell-name> <gpus> <timeout_s> [VAR=value ...] -- <program> [args ...]

<program> is a harness module name (bench_cli, gate_dist, gemm_ar_bench, micro, ops_bench, gemm_bench,
nccl_tuned, ...), a dotted module path, or a path to a .py file.  With <gpus> > 1 the cell is started through
`python -m torch.distributed.run` with one process per GPU on 127.0.0.1, unless the cell says `LAUNCH=single` among
its variables (a program that drives all of its GPUs from one process).  `--out <out>/<cell>.jsonl --tag <cell>`
is appended for harness modules that take them, so every record carries its cell name.

Behaviour, after the reference project's cluster scripts (scripts/driver.sh:8-17 cell loop with deadline,
scripts/run_cell.sh:9-26 one cell with time limit and clock abort, scripts/gpurun.sh:9-29 per-GPU mkdir locks):

  * a cell whose time limit would run past the deadline is skipped and recorded as such;
  * the cell's process tree is started in its own session and, when its limit passes, exactly that process
    group is terminated (then killed after a grace period) -- nothing is ever signalled by name;
  * `<lock-dir>/gpu<i>.lock` directories (atomic mkdir) keep two campaigns off the same GPU; a lock whose owner
    process is gone is taken over;
  * with --expect-mem-mhz the memory clock of the cell's GPUs is read before the cell and the whole campaign stops
    with exit code 3 ("CLOCK_ABORT") when it differs -- the guard only reads, it never sets a clock;
  * after a cell, its records are scanned for thermal / hardware slow-down reasons; such a cell is run once more
    and the first attempt is kept with the suffix `.rejected`;
  * JSON lines that a program only prints (no --out option) are copied from its log into `<out>/<cell>.jsonl`;
  * `<out>/campaign_state.jsonl` has one line per finished attempt; --resume skips cells that already ended
    with exit code 0.
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import signal
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, Optional

HARNESS_MODULES = ("bench_cli", "gate_dist", "gemm_ar_bench", "micro", "ops_bench", "gemm_bench", "nccl_tuned",
                   "profile_case", "block_bench", "compare_bench")
TAKES_OUT_TAG = ("bench_cli",)
TAKES_OUT = ("bench_cli", "gate_dist", "gemm_ar_bench", "micro", "nccl_tuned", "block_bench", "compare_bench")
SELF_LAUNCHING = ("nccl_tuned",)      # start their own ranks: never wrapped in torch.distributed.run
BAD_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


@dataclass
class Cell:
    name: str
    gpus: int
    timeout_s: int
    env: dict = field(default_factory=dict)
    program: str = ""
    args: list = field(default_factory=list)


def parse_cells(text: str) -> list[Cell]:
    cells = []
    for ln, raw in enumerate(text.splitlines(), 1):
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        tok = shlex.split(line)
        if "--" not in tok:
            raise ValueError(f"line {ln}: no '--' before the program")
        k = tok.index("--")
        head, cmd = tok[:k], tok[k + 1:]
        if len(head) < 3 or not cmd:
            raise ValueError(f"line {ln}: expected '<cell> <gpus> <timeout_s> [VAR=val ...] -- <program> [args]'")
        env = {}
        for kv in head[3:]:
            if "=" not in kv:
                raise ValueError(f"line {ln}: '{kv}' is not VAR=value")
            a, b = kv.split("=", 1)
            env[a] = b
        gpus, tmo = int(head[1]), int(head[2])
        if gpus < 1 or gpus > 8 or tmo < 1:
            raise ValueError(f"line {ln}: gpus must be 1..8 and the time limit positive")
        cells.append(Cell(head[0], gpus, tmo, env, cmd[0], cmd[1:]))
    names = [c.name for c in cells]
    if len(set(names)) != len(names):
        raise ValueError("cell names must be unique")
    return cells


def build_command(cell: Cell, out_dir: str, port: int, python: str = sys.executable) -> list[str]:
    prog = cell.program
    short = prog if prog in HARNESS_MODULES else None
    if short:
        target = ["-m", f"fp4_all_reduce_b200.harness.{prog}"]
    elif prog.endswith(".py"):
        target = [prog]
    else:
        target = ["-m", prog]
    extra = []
    if short in TAKES_OUT and "--out" not in cell.args:
        extra += ["--out", os.path.join(out_dir, cell.name + ".jsonl")]
    if short in TAKES_OUT_TAG and "--tag" not in cell.args:
        extra += ["--tag", cell.name]
    if cell.gpus > 1 and short not in SELF_LAUNCHING and cell.env.get("LAUNCH") != "single":
        head = [python, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={cell.gpus}",
                "--master-addr", "127.0.0.1", "--master-port", str(port)]
    else:
        head = [python]
    return head + target + cell.args + extra


# ---------------------------------------------------------------- per-GPU locks
class GpuLocks:
    def __init__(self, lock_dir: str, pid_alive: Callable[[int], bool] = None):
        self.dir = lock_dir
        self.held: list[str] = []
        self._alive = pid_alive or self._pid_alive
        os.makedirs(lock_dir, exist_ok=True)

    @staticmethod
    def _pid_alive(pid: int) -> bool:
        try:
            os.kill(pid, 0)
            return True
        except ProcessLookupError:
            return False
        except PermissionError:
            return True

    def _try(self, path: str) -> bool:
        try:
            os.mkdir(path)
        except FileExistsError:
            try:
                with open(os.path.join(path, "owner")) as f:
                    owner = int(f.read().strip() or "0")
            except (OSError, ValueError):
                owner = 0
            if owner and self._alive(owner):
                return False
            # stale: the owner is gone; take it over
            try:
                os.unlink(os.path.join(path, "owner"))
            except OSError:
                pass
        with open(os.path.join(path, "owner"), "w") as f:
            f.write(str(os.getpid()))
        return True

    def acquire(self, gpus: int, total: int = 8) -> Optional[list[int]]:
        got = []
        for i in range(total):
            p = os.path.join(self.dir, f"gpu{i}.lock")
            if self._try(p):
                got.append(i)
                self.held.append(p)
                if len(got) == gpus:
                    return got
        self.release()
        return None

    def release(self):
        for p in self.held:
            try:
                os.unlink(os.path.join(p, "owner"))
                os.rmdir(p)
            except OSError:
                pass
        self.held = []


# ---------------------------------------------------------------- one cell
def run_with_limit(cmd: list[str], env: dict, log_path: str, limit_s: float, grace_s: float = 10.0) -> tuple[int, float, bool]:
    """Run `cmd` in its own session; returns (exit code, seconds, timed_out).  On time-out the process GROUP
    started here gets SIGTERM, then SIGKILL after `grace_s`."""
    t0 = time.time()
    with open(log_path, "a") as log:
        log.write(f"# CMD {' '.join(shlex.quote(c) for c in cmd)}\n")
        log.flush()
        proc = subprocess.Popen(cmd, env=env, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
        timed_out = False
        try:
            rc = proc.wait(timeout=limit_s)
        except subprocess.TimeoutExpired:
            timed_out = True
            pgid = proc.pid                      # start_new_session: the child leads its own group
            try:
                os.killpg(pgid, signal.SIGTERM)
            except ProcessLookupError:
                pass
            try:
                rc = proc.wait(timeout=grace_s)
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(pgid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                rc = proc.wait()
            rc = 124
        log.write(f"# END rc={rc} seconds={time.time() - t0:.1f} timed_out={timed_out}\n")
    return rc, time.time() - t0, timed_out


def harvest_records(log_path: str, start: int, jsonl_path: str) -> int:
    """Programs without an --out option print their records: copy the JSON lines this attempt wrote to the log into
    <cell>.jsonl unless the program produced that file itself.  Returns the number of lines copied."""
    if os.path.exists(jsonl_path):
        return 0
    try:
        with open(log_path) as f:
            f.seek(start)
            lines = [l for l in f if l.startswith("{") and l.rstrip().endswith("}")]
    except OSError:
        return 0
    if lines:
        with open(jsonl_path, "w") as f:
            f.writelines(lines)
    return len(lines)


def slowdown_reasons(jsonl_path: str) -> list[str]:
    bad = set()
    try:
        with open(jsonl_path) as f:
            for line in f:
                if not line.startswith("{"):
                    continue
                try:
                    r = json.loads(line)
                except json.JSONDecodeError:
                    continue
                rs = r.get("reasons") or (r.get("clocks") or {}).get("reasons") or []
                bad.update(x for x in rs if x in BAD_REASONS)
    except OSError:
        pass
    return sorted(bad)


def read_mem_clocks(gpus: list[int]) -> Optional[list[int]]:
    """Memory clocks through nvidia-smi (read only); None when the tool is missing."""
    import shutil

    exe = shutil.which("nvidia-smi")
    if exe is None:
        return None
    out = subprocess.run([exe, "--id=" + ",".join(map(str, gpus)), "--query-gpu=clocks.mem",
                          "--format=csv,noheader,nounits"], capture_output=True, text=True)
    try:
        return [int(x) for x in out.stdout.split()]
    except ValueError:
        return None


def parse_deadline(s: Optional[str], now: float) -> float:
    if not s:
        return 0.0
    if s.startswith("+"):               # seconds from now
        return now + float(s[1:])
    if ":" in s:
        hh, mm = s.split(":")
        lt = time.localtime(now)
        t = time.mktime((lt.tm_year, lt.tm_mon, lt.tm_mday, int(hh), int(mm), 0, 0, 0, -1))
        return t
    return float(s)


def load_state(path: str) -> dict:
    done = {}
    try:
        with open(path) as f:
            for line in f:
                try:
                    r = json.loads(line)
                except json.JSONDecodeError:
                    continue
                done[r["cell"]] = r
    except OSError:
        pass
    return done


def run_campaign(cells: list[Cell], out_dir: str, *, deadline: float = 0.0, resume: bool = False, dry_run: bool = False,
                 expect_mem_mhz: int = 0, lock_dir: Optional[str] = None, port: int = 29700,
                 clock_reader: Callable[[list[int]], Optional[list[int]]] = read_mem_clocks,
                 now: Callable[[], float] = time.time, python: str = sys.executable, echo=print) -> int:
    os.makedirs(out_dir, exist_ok=True)
    state_path = os.path.join(out_dir, "campaign_state.jsonl")
    done = load_state(state_path) if resume else {}
    locks = GpuLocks(lock_dir) if lock_dir else None

    def record(rec):
        with open(state_path, "a") as f:
            f.write(json.dumps(rec) + "\n")

    for k, cell in enumerate(cells):
        if resume and done.get(cell.name, {}).get("rc") == 0:
            echo(f"SKIP {cell.name} (done)")
            continue
        if deadline and now() + cell.timeout_s > deadline:
            echo(f"SKIP {cell.name} (deadline)")
            record({"cell": cell.name, "rc": None, "skipped": "deadline", "time": now()})
            continue
        cmd = build_command(cell, out_dir, port + k % 200, python)
        if dry_run:
            echo(" ".join(shlex.quote(c) for c in cmd))
            continue
        gpus = list(range(cell.gpus))
        if locks:
            got = locks.acquire(cell.gpus)
            if got is None:
                echo(f"SKIP {cell.name} (GPUs locked by another campaign)")
                record({"cell": cell.name, "rc": None, "skipped": "locked", "time": now()})
                continue
            gpus = got
        try:
            if expect_mem_mhz:
                rb = clock_reader(gpus)
                if rb is not None and any(v != expect_mem_mhz for v in rb):
                    echo(f"CLOCK_ABORT {cell.name}: clocks.mem {rb} != {expect_mem_mhz}")
                    record({"cell": cell.name, "rc": 3, "clock_abort": rb, "time": now()})
                    return 3
            env = dict(os.environ)
            env.update(cell.env)
            env["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, gpus))
            log_path = os.path.join(out_dir, cell.name + ".log")
            jsonl = os.path.join(out_dir, cell.name + ".jsonl")
            for attempt in (1, 2):
                echo(f"START {cell.name} gpus={gpus} limit={cell.timeout_s}s attempt={attempt}")
                log_start = os.path.getsize(log_path) if os.path.exists(log_path) else 0
                rc, secs, tmo = run_with_limit(cmd, env, log_path, cell.timeout_s)
                harvest_records(log_path, log_start, jsonl)
                bad = slowdown_reasons(jsonl)
                rec = {"cell": cell.name, "rc": rc, "seconds": round(secs, 1), "timed_out": tmo, "attempt": attempt,
                       "slowdown": bad, "gpus": gpus, "time": now()}
                record(rec)
                echo(f"END {cell.name} rc={rc} {secs:.1f}s" + (f" slowdown={bad}" if bad else ""))
                if bad and attempt == 1 and rc == 0 and os.path.exists(jsonl):
                    os.replace(jsonl, jsonl + ".rejected")
                    continue
                break
        finally:
            if locks:
                locks.release()
    echo("CAMPAIGN DONE")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("cells")
    ap.add_argument("--out", required=True)
    ap.add_argument("--deadline", default=None, help="HH:MM (local, today), +SECONDS from now, or an epoch in seconds")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--expect-mem-mhz", type=int, default=0)
    ap.add_argument("--lock-dir", default=None)
    ap.add_argument("--port", type=int, default=29700)
    ns = ap.parse_args(argv)
    with open(ns.cells) as f:
        cells = parse_cells(f.read())
    return run_campaign(cells, ns.out, deadline=parse_deadline(ns.deadline, time.time()), resume=ns.resume,
                        dry_run=ns.dry_run, expect_mem_mhz=ns.expect_mem_mhz, lock_dir=ns.lock_dir, port=ns.port)


if __name__ == "__main__":
    sys.exit(main())
