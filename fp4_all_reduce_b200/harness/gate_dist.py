"""The five-phase bitwise gate on real GPUs, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m fp4_all_reduce_b200.harness.gate_dist --rows 1024,4096 --inputs bf16,nvfp4 --epilogues 0,1 \
        [--algos auto] [--reps 50] [--graph-calls 10] [--graph-reps 20] [--skew-reps 20] [--negctl stale|flip] \
        [--out gate.jsonl]

Every rank generates every rank's inputs (they are pure functions of rank and set number), evaluates the
host model, runs the calls on its own GPU and compares its own outputs; rank 0 gathers the per-rank
verdicts and prints one JSON record of kind "check" per cell.  Exit code 3 when any cell fails (so that a
negative control can be recognised by its exit code), as in the reference harness
(harness/fp4ar_bench.cu:331-346,546).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import time

import torch
import torch.distributed as dist

from .. import _native as N
from .. import oracle as O
from ..parallel.context import Fp4ArContext
from ..utils.runinfo import sources_digest
from .gate import CellConfig, InputSet, Outputs, args_for, make_inputs, mismatches, rel_l2

IN_NAMES = {"bf16": N.IN_BF16, "nvfp4": N.IN_NVFP4}
ALGO_NAMES = {"auto": N.ALGO_AUTO, "oneshot": N.ALGO_ONESHOT, "twoshot": N.ALGO_TWOSHOT}


def make_inputs_shared(cfg: CellConfig, dev, rank: int, world: int) -> list:
    """The three input sets of a cell, each built (inputs + host model) by ONE rank and handed to the others over the
    process group: the host model is the expensive part of a gate cell, and P ranks evaluating the same model on the
    same cores would multiply its cost by P while the GPUs idle."""
    builder = [s % world for s in range(3)]
    mine = {s: make_inputs(cfg, s, dev) for s in range(3) if builder[s] == rank}
    keys = (["out"] if cfg.epilogue <= 1 else ["outq"]) + (["res_out"] if cfg.epilogue >= 1 else [])
    width = {"out": N.HIDDEN, "res_out": N.HIDDEN, "outq": N.QROW_BYTES if cfg.epilogue == 2 else N.MXROW_BYTES}
    sets = []
    for s in range(3):
        src = builder[s]
        inp = mine.get(s)
        box = [inp.gs if inp is not None else None]
        dist.broadcast_object_list(box, src=src)
        gs = box[0]
        if inp is None:
            in_dtype, in_cols = (torch.bfloat16, N.HIDDEN) if cfg.input == N.IN_BF16 else (torch.uint8, N.QROW_BYTES)
            xs = [torch.empty(cfg.rows, in_cols, dtype=in_dtype, device=dev) for _ in range(world)]
            res = torch.empty(cfg.rows, N.HIDDEN, dtype=torch.bfloat16, device=dev) if cfg.epilogue else None
            weight = torch.empty(N.HIDDEN, dtype=torch.bfloat16, device=dev) if cfg.epilogue else None
            exp_dev = {k: torch.empty(cfg.rows, width[k], dtype=torch.int16 if k != "outq" else torch.uint8, device=dev)
                       for k in keys}
            inp = InputSet(xs, gs, res, weight, {}, None, exp_dev)
        # as bytes: the expectations are 16-bit integer patterns, a type NCCL does not move
        for t in inp.xs:
            dist.broadcast(t.view(torch.uint8), src=src)
        if cfg.epilogue:
            dist.broadcast(inp.res.view(torch.uint8), src=src)
            dist.broadcast(inp.weight.view(torch.uint8), src=src)
        for k in keys:
            dist.broadcast(inp.exp_dev[k].view(torch.uint8), src=src)
        sets.append(inp)
    torch.cuda.synchronize()
    return sets


def gate_cell(ctx: Fp4ArContext, cfg: CellConfig, *, reps: int, graph_calls: int, graph_reps: int, skew_reps: int,
              skew_us: float, negctl: str | None, percall: int = 0) -> dict:
    dev = ctx.device
    rank, world = ctx.rank, ctx.nranks
    sets = make_inputs_shared(cfg, dev, rank, world)
    outs = Outputs(cfg, dev, 1)

    launch_cfg = dataclasses.replace(cfg, weight_bias=cfg.weight_bias + 2.0 ** -7) if negctl == "bias" else cfg

    def call(s: int):
        src = sets[(s + 1) % 3] if negctl == "stale" else sets[s % 3]
        ctx.launch(args_for(launch_cfg, src, outs, 0, rank))

    def compare(s: int) -> int:
        torch.cuda.synchronize()
        if negctl == "flip" and rank == world - 1:
            t = outs.out[0] if outs.out[0] is not None else outs.outq[0]
            t.view(torch.uint8).view(-1)[0] ^= 1
        return mismatches(cfg, sets[s % 3], outs, 0)

    def total(v: int) -> int:
        t = torch.tensor([v], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        return int(t.item())

    rec = {"kind": "check", "tp": world, "rows": cfg.rows, "hidden": N.HIDDEN, "algo": cfg.resolved_algo(),
           "input": cfg.input, "epilogue": cfg.epilogue, "dist": cfg.dist, "negctl": negctl}
    # Building the inputs runs the host model, whose duration differs between the rank processes (they share the
    # CPU cores); the device-side waits are bounded, so the ranks are lined up before the first launch.
    torch.cuda.synchronize()
    dist.barrier()
    # 1: first call
    call(0)
    rec["mism_first"] = total(compare(0))
    st = ctx.status()
    if total(st.code) != 0:
        rec["status"] = st.describe()
        rec["ranks_with_error"] = total(int(st.code != 0))
        rec["pass"] = False
        return rec
    if cfg.epilogue == N.EPI_NONE and rank == 0:      # rank 0 built set 0 and holds its exact FP32 sum
        rec["rel_l2_vs_fp32"] = rel_l2(sets[0], O.bf16_bits(outs.out[0]))
    first = outs.out[0] if outs.out[0] is not None else outs.outq[0]
    digest = torch.tensor([int(first.view(torch.uint8).to(torch.int64).sum().item())], dtype=torch.int64, device=dev)
    lo, hi = digest.clone(), digest.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    rec["ranks_identical"] = bool(lo.item() == hi.item()) or negctl == "flip"
    # 2: back-to-back calls cycling the three sets, one compare at the end
    for s in range(1, reps + 1):
        call(s)
    rec["b2b_calls"] = reps
    rec["mism_b2b_final"] = total(compare(reps))
    # 3: compare after every call
    bad = mm = 0
    per = percall if percall > 0 else max(3, reps // 5)
    for s in range(per):
        outs.clear()
        call(s)
        m = compare(s)
        mm += m
        bad += m > 0
    rec["percall_calls"] = per
    rec["mism_percall"] = total(mm)
    rec["bad_calls_percall"] = total(bad)
    # 4: graph replay
    bad = 0
    if graph_calls > 0:
        stream = torch.cuda.Stream(device=dev)
        stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(stream):
            call(0)
            stream.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for s in range(graph_calls):
                    call(s)
        torch.cuda.synchronize()
        for _ in range(graph_reps):
            outs.clear()
            graph.replay()
            bad += compare(graph_calls - 1) > 0
        del graph
    rec["graph_calls"] = graph_calls * graph_reps
    rec["bad_calls_graph"] = total(bad)
    # 5: one rank late, rotating
    bad = 0
    cycles = int(skew_us * 1.9e3)
    for s in range(skew_reps):
        outs.clear()
        torch.cuda.synchronize()
        dist.barrier()
        if s % world == rank:
            torch.cuda._sleep(cycles)
        call(s)
        bad += compare(s) > 0
    rec["skew_calls"] = skew_reps
    rec["skew_us"] = skew_us
    rec["bad_calls_skew"] = total(bad)
    st = ctx.status()
    rec["status"] = st.describe()
    code = total(st.code)
    rec["pass"] = (rec["mism_first"] == 0 and rec["ranks_identical"] and rec["mism_b2b_final"] == 0 and
                   rec["bad_calls_percall"] == 0 and rec["bad_calls_graph"] == 0 and rec["bad_calls_skew"] == 0 and
                   code == 0)
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", default="1024")
    ap.add_argument("--inputs", default="bf16")
    ap.add_argument("--epilogues", default="0")
    ap.add_argument("--algos", default="auto")
    ap.add_argument("--dist", default="partial")
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--graph-calls", type=int, default=10)
    ap.add_argument("--graph-reps", type=int, default=10)
    ap.add_argument("--skew-reps", type=int, default=8)
    ap.add_argument("--skew-us", type=float, default=50.0)
    ap.add_argument("--negctl", default=None, choices=[None, "stale", "flip", "bias"])
    ap.add_argument("--timeout-ms", type=int, default=1000)
    ap.add_argument("--team-warps", default="0", help="comma list of warps per row team (0 = the library's default)")
    ap.add_argument("--lags", default="0", help="comma list of two-shot depths, lag_owner + 16 * lag_finish (0 = default)")
    ap.add_argument("--percall", type=int, default=0, help="calls with a compare after each (0 = reps / 5, at least 3)")
    ap.add_argument("--out", default=None)
    ns = ap.parse_args(argv)

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    rows_list = [int(r) for r in ns.rows.split(",")]
    ctx = Fp4ArContext(max(rows_list), device=dev)
    ctx.set_timeout_ms(ns.timeout_ms)
    fails = 0
    records = []
    for rows in rows_list:
        for inp in ns.inputs.split(","):
            for epi in (int(e) for e in ns.epilogues.split(",")):
                for algo, tw, lags in ((a, int(t), int(l)) for a in ns.algos.split(",") for t in ns.team_warps.split(",")
                                       for l in ns.lags.split(",")):
                    cfg = CellConfig(nranks=world, rows=rows, algo=ALGO_NAMES[algo], input=IN_NAMES[inp], epilogue=epi,
                                     dist=ns.dist, team_warps=tw, lags=lags)
                    t0 = time.time()
                    rec = gate_cell(ctx, cfg, reps=ns.reps, graph_calls=ns.graph_calls, graph_reps=ns.graph_reps,
                                    skew_reps=ns.skew_reps, skew_us=ns.skew_us, negctl=ns.negctl, percall=ns.percall)
                    rec["team_warps"], rec["lags"] = tw, lags
                    rec["seconds"] = round(time.time() - t0, 2)
                    rec["sources"] = sources_digest()
                    fails += not rec["pass"]
                    records.append(rec)
                    if rank == 0:
                        print(json.dumps(rec), flush=True)
                    # a wait that gave up on ANY rank leaves slots un-armed: re-arm everywhere (collective decision)
                    code = torch.tensor([int(ctx.status().code != 0)], dtype=torch.int64, device=dev)
                    dist.all_reduce(code)
                    if int(code.item()) != 0:
                        ctx.reset()
    if rank == 0 and ns.out:
        with open(ns.out, "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    return 3 if fails else 0


if __name__ == "__main__":
    sys.exit(main())
