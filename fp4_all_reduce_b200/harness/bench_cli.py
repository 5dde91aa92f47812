"""Timing harness: one JSON line of kind "timing" per cell, the way the reference's `fp4ar_bench` reports
(harness/fp4ar_bench.cu:154-187,423-428): K calls per CUDA graph, ranks aligned before every iteration,
CUDA events around the replay, per-iteration maximum over ranks, median / p10 / p90 per call.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m fp4_all_reduce_b200.harness.bench_cli --rows 1024,16384 --modes fused,xport,compute,empty \
        --inputs bf16,nvfp4 --epilogues 0,1 [--algos auto] [--team-warps 3,6] [--teams 0] [--graph 10] \
        [--iters 50] [--warmup 10] [--nccl] [--out timing.jsonl]

(also runs as a plain `python -m ...` on one GPU: a one-rank context.)

Modes: fused = the operator; xport = same bytes and waits, codec skipped; compute = same codec work with
every push looped back into the own window (no peer traffic); empty = the kernel launched with zero rows
(launch + prologue + call-state cost).  Corrected overlap = (X + C - F - E) / min(X - E, C - E).
`--nccl` adds BF16 NCCL AllReduce (and AllReduce + stand-alone add+RMSNorm) cells measured the same way.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from .. import _native as N
from ..models.m3_block import L2_BYTES
from ..ops import codec
from ..parallel.context import Fp4ArContext, make_args
from ..utils import data as D
from ..utils import timing
from ..utils.clocks import ClockSampler
from ..utils.runinfo import run_info

MODES = {"fused": N.MODE_FUSED, "xport": N.MODE_XPORT, "compute": N.MODE_COMPUTE}
INPUTS = {"bf16": N.IN_BF16, "nvfp4": N.IN_NVFP4}
ALGOS = {"auto": N.ALGO_AUTO, "oneshot": N.ALGO_ONESHOT, "twoshot": N.ALGO_TWOSHOT}


class Cell:
    """Buffers of one (rows, input, epilogue) cell: rotating partials larger than L2, residual, outputs."""

    def __init__(self, rows, kind, epi, rank, world, dev):
        row_bytes = N.HIDDEN * 2 if kind == N.IN_BF16 else N.QROW_BYTES
        self.nsets = min(24, max(2, -(-2 * L2_BYTES // (rows * row_bytes))))
        base = D.partial(rows, rank).to(dev)
        self.gs = None
        if kind == N.IN_NVFP4:
            am = base.float().abs().max()
            if world > 1:
                alls = [torch.zeros_like(am) for _ in range(world)]
                dist.all_gather(alls, am)
                self.gs = [float(a.item()) / 2688.0 for a in alls]
            else:
                self.gs = [float(am.item()) / 2688.0]
            base = codec.encode_static(base, self.gs[rank])
        self.xs = [base.clone() if i == 0 else torch.roll(base, i, 0) for i in range(self.nsets)]
        self.res = D.residual(rows).to(dev) if epi else None
        self.w = D.norm_weight().to(dev) if epi else None
        self.out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=dev) if epi <= 1 else None
        nb = N.QROW_BYTES if epi == 2 else N.MXROW_BYTES
        self.outq = torch.empty(rows, nb, dtype=torch.uint8, device=dev) if epi >= 2 else None
        self.rows, self.kind, self.epi = rows, kind, epi

    def args(self, i, mode, algo, teams, tw, rows=None, lags=0):
        return make_args(x=self.xs[i % self.nsets], out=self.out, rows=self.rows if rows is None else rows, mode=mode,
                         algo=algo, input=self.kind, epilogue=self.epi, gs=self.gs, res_in=self.res, res_out=self.res,
                         weight=self.w, outq=self.outq, qscale=168.0, teams=teams, team_warps=tw, lags=lags)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", default="1024,2048,4096,8192,16384")
    ap.add_argument("--modes", default="fused")
    ap.add_argument("--inputs", default="bf16")
    ap.add_argument("--epilogues", default="0")
    ap.add_argument("--algos", default="auto")
    ap.add_argument("--team-warps", default="0")
    ap.add_argument("--teams", default="0")
    ap.add_argument("--lags", default="0", help="two-shot depths, comma list of lag_owner+16*lag_finish (e.g. 33 = 1,2; 50 = 2,3; 66 = 2,4)")
    ap.add_argument("--graph", type=int, default=10)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--nccl", action="store_true")
    ap.add_argument("--nccl-only", action="store_true", help="skip the fused-kernel cells (NCCL sweeps)")
    ap.add_argument("--nccl-reg", action="store_true",
                    help="also time NCCL on buffers allocated with ncclMemAlloc and registered with the communicator")
    ap.add_argument("--timeout-ms", type=int, default=2000, help="device-side wait limit of the context")
    ap.add_argument("--tag", default="")
    ap.add_argument("--out", default=None)
    ns = ap.parse_args(argv)

    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    rows_list = [int(r) for r in ns.rows.split(",")]
    ctx = Fp4ArContext(max(rows_list), device=dev)
    ctx.set_timeout_ms(ns.timeout_ms)

    def rearm_if_failed():
        """A wait that gave up on ANY rank leaves slots un-armed everywhere: decide together, reset together."""
        code = torch.tensor([int(ctx.status().code != 0)], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(code)
        if int(code.item()) != 0:
            ctx.reset()

    common = {"kind": "timing", "tp": world, "hidden": N.HIDDEN, "graphK": ns.graph, "iters": ns.iters,
              "warmup": ns.warmup, "tag": ns.tag, **run_info(dev)}
    records = []

    def emit(rec):
        records.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    def timed(fn, before_each=None):
        g = timing.capture(fn, ns.graph, dev, warm_calls=2)
        if before_each is not None:
            before_each()
        with ClockSampler(local) as clk:
            t = timing.time_replays(g, ns.graph, ns.iters, ns.warmup, dev, before_each=before_each)
        c = clk.summary()
        del g
        return t, c

    for rows in rows_list:
        for inp in ns.inputs.split(","):
            for epi in (int(e) for e in ns.epilogues.split(",")):
                cell = Cell(rows, INPUTS[inp], epi, rank, world, dev)
                for algo in ([] if ns.nccl_only else ns.algos.split(",")):
                    for tw in (int(t) for t in ns.team_warps.split(",")):
                        for teams, lags in ((int(t), int(l)) for t in ns.teams.split(",") for l in ns.lags.split(",")):
                            res = {}
                            for mode in ns.modes.split(","):
                                if mode == "empty":
                                    fn = lambda i: ctx.launch(cell.args(i, N.MODE_FUSED, ALGOS[algo], teams, tw, rows=0, lags=lags))
                                else:
                                    fn = lambda i, m=MODES[mode]: ctx.launch(cell.args(i, m, ALGOS[algo], teams, tw, lags=lags))
                                t, c = timed(fn)
                                res[mode] = t["med_us"]
                                st = ctx.status()
                                emit({**common, "variant": "fp4ar", "mode": mode, "algo": algo, "rows": rows,
                                      "input": inp, "epilogue": epi, "team_warps": tw, "teams": teams, "lags": lags,
                                      "med_us": round(t["med_us"], 3), "p10_us": round(t["p10_us"], 3),
                                      "p90_us": round(t["p90_us"], 3), "rank_med_us": t.get("rank_med_us"),
                                      "sm_mhz": c.get("sm_mhz"), "reasons": c.get("reasons"), "status": st.describe(),
                                      "wire_gbs": round(rows * 3460 * (1 if world <= 2 else 2 * (world - 1) / world) /
                                                        t["med_us"] / 1e3, 1) if world > 1 else None})
                                rearm_if_failed()
                            if all(k in res for k in ("fused", "xport", "compute", "empty")):
                                F, X, Cc, E = res["fused"], res["xport"], res["compute"], res["empty"]
                                den = min(X - E, Cc - E)
                                emit({**common, "kind": "overlap", "rows": rows, "input": inp, "epilogue": epi, "algo": algo,
                                      "team_warps": tw, "teams": teams,
                                      "corrected_overlap": round((X + Cc - F - E) / den, 3) if den > 0 else None})
                if ns.nccl and inp == "bf16" and world > 1 and epi <= 1:
                    # NCCL reduces in place: one buffer per call of the graph, every buffer restored from the pristine
                    # partial before each replay (outside the events), so every all-reduce sums fresh, finite data.
                    pristine = D.partial(rows, rank).to(dev)
                    arms = [("", None)]
                    if ns.nccl_reg:
                        arms.append(("_reg", "registered"))
                    for suffix, reg in arms:
                        pool = None
                        try:
                            if reg:
                                # user-buffer registration: memory from ncclMemAlloc, registered with the communicator
                                # (the reference's registered arm: harness/fp4ar_bench.cu:453-457)
                                backend = dist.distributed_c10d._get_default_group()._get_backend(dev)
                                pool = torch.cuda.MemPool(backend.mem_allocator)
                                with torch.cuda.use_mem_pool(pool):
                                    buf = [torch.empty_like(pristine) for _ in range(ns.graph)]
                                backend.register_mem_pool(pool)
                            else:
                                buf = [torch.empty_like(pristine) for _ in range(ns.graph)]
                        except Exception as e:
                            emit({**common, "variant": "nccl_bf16" + suffix, "rows": rows, "epilogue": epi,
                                  "skipped": f"{type(e).__name__}: {str(e)[:160]}"})
                            continue

                        def restore(buf=buf):
                            for b in buf:
                                b.copy_(pristine)

                        def nccl_fn(i, buf=buf):
                            dist.all_reduce(buf[i % len(buf)])
                            if epi:
                                codec.add_rmsnorm(buf[i % len(buf)], cell.res, cell.w, inplace_residual=True, out=cell.out,
                                                  epilogue=N.EPI_NORM_BF16)
                        t, c = timed(nccl_fn, before_each=restore)
                        emit({**common, "variant": "nccl_bf16" + suffix + ("+norm" if epi else ""), "mode": "fused", "rows": rows,
                              "input": "bf16", "epilogue": epi, "med_us": round(t["med_us"], 3),
                              "p10_us": round(t["p10_us"], 3), "p90_us": round(t["p90_us"], 3),
                              "sm_mhz": c.get("sm_mhz"), "reasons": c.get("reasons"), "registered": bool(reg),
                              "proto": os.environ.get("NCCL_PROTO", "default"), "nccl_algo": os.environ.get("NCCL_ALGO", "default"),
                              "nchannels": os.environ.get("NCCL_MIN_NCHANNELS", "default")})
                        del buf
                        if pool is not None:
                            try:
                                backend.deregister_mem_pool(pool)
                            except Exception:
                                pass
                            del pool
                    del pristine
                del cell
                torch.cuda.empty_cache()
    if rank == 0 and ns.out:
        with open(ns.out, "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
    ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
