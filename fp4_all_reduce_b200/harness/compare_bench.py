"""Timing of the comparison variants (flag push, pull, pull with NVFP4 input, two-shot pull, pull reduce-scatter +
pushed all-gather) against the main operator's one-shot and two-shot paths, one process per GPU, measured like every
other cell (K calls per CUDA graph, ranks aligned, CUDA events, max over ranks):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port X \
        -m fp4_all_reduce_b200.harness.compare_bench [--rows 1024,4096,16384] [--check] [--out compare.jsonl]

--check first compares every variant's output of the first row count with the host model (bitwise).
The reference project compares its push kernels with its pull family and its flag-based control the same way
(docs/RESULTS.md pull and control rows; kernels/pull/variants.txt, kernels/control/variants.txt).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

from .. import _native as N
from .. import oracle as O
from ..models.m3_block import L2_BYTES
from ..ops import codec
from ..parallel.compare import CompareContext
from ..parallel.context import Fp4ArContext, make_args
from ..utils import data as D
from ..utils import timing
from ..utils.clocks import ClockSampler


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", default="1024,4096,16384")
    ap.add_argument("--graph", type=int, default=10)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--only", default="", help="comma list of variant names (default: all)")
    ap.add_argument("--timeout-ms", type=int, default=1000, help="device-side wait limit of both contexts")
    ap.add_argument("--out", default=None)
    ns = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank()
    rows_list = [int(r) for r in ns.rows.split(",")]
    main_ctx = Fp4ArContext(max(rows_list), device=dev)
    cmp_ctx = CompareContext(max(rows_list), device=dev)
    cmp_ctx.timeout_ms = ns.timeout_ms
    main_ctx.set_timeout_ms(ns.timeout_ms)
    records = []

    def emit(r):
        records.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    for k, rows in enumerate(rows_list):
        nsets = min(24, max(2, -(-2 * L2_BYTES // (rows * N.HIDDEN * 2))))
        base = D.partial(rows, rank).to(dev)
        xs = [base.clone() if i == 0 else torch.roll(base, i, 0) for i in range(nsets)]
        out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=dev)

        # NVFP4 rows with the static scale amax / 2688 of every rank's partial
        am = base.float().abs().max()
        alls = [torch.zeros_like(am) for _ in range(world)]
        dist.all_gather(alls, am)
        gs = [float(a.item()) / 2688.0 for a in alls]
        xq0 = codec.encode_static(base, gs[rank])
        xqs = [xq0.clone() if i == 0 else torch.roll(xq0, i, 0) for i in range(nsets)]

        # name -> (call, host-model algorithm, host-model input kind)
        variants = {
            "fp4ar_oneshot": (lambda i: main_ctx.launch(make_args(x=xs[i % nsets], out=out, rows=rows, algo=N.ALGO_ONESHOT)), 0, 0),
            "fp4ar_twoshot": (lambda i: main_ctx.launch(make_args(x=xs[i % nsets], out=out, rows=rows, algo=N.ALGO_TWOSHOT)), 1, 0),
            "fp4ar_oneshot_nvfp4": (lambda i: main_ctx.launch(make_args(x=xqs[i % nsets], out=out, rows=rows, algo=N.ALGO_ONESHOT,
                                                                        input=N.IN_NVFP4, gs=gs)), 0, 1),
            "flag_push": (lambda i: cmp_ctx.all_reduce("flag_push", xs[i % nsets], out), 0, 0),
            "pull": (lambda i: cmp_ctx.all_reduce("pull", xs[i % nsets], out), 0, 0),
            "pull_nvfp4": (lambda i: cmp_ctx.all_reduce("pull_nvfp4", xqs[i % nsets], out, gs=gs), 0, 1),
            "pull_twoshot": (lambda i: cmp_ctx.all_reduce("pull_twoshot", xs[i % nsets], out), 1, 0),
            "pull_rs_push_ag": (lambda i: cmp_ctx.all_reduce("pull_rs_push_ag", xs[i % nsets], out), 1, 0),
        }
        if ns.only:
            variants = {k2: v for k2, v in variants.items() if k2 in ns.only.split(",")}
        if ns.check and k == 0:
            allx = [torch.empty_like(base) for _ in range(world)]
            dist.all_gather(allx, base)
            allq = [torch.empty_like(xq0) for _ in range(world)]
            dist.all_gather(allq, xq0)
            exps = {}
            for name, (fn, algo, kind) in variants.items():
                if (algo, kind) not in exps:
                    ins = [t.cpu().numpy() for t in allq] if kind else [O.bf16_bits(t) for t in allx]
                    exps[(algo, kind)] = O.allreduce(ins, algo=algo, input_kind=kind, gs=gs if kind else None)["out"]
                exp = exps[(algo, kind)]
                out.zero_()
                fn(0)
                torch.cuda.synchronize()
                m = torch.tensor([int(np.count_nonzero(O.bf16_bits(out) != exp))], device=dev)
                dist.all_reduce(m)
                st = main_ctx.status() if name.startswith("fp4ar") else cmp_ctx.status()
                emit({"kind": "check", "variant": name, "tp": world, "rows": rows, "mismatches_vs_host_model": int(m.item()),
                      "status": st.describe(), "pass": int(m.item()) == 0 and st.ok})
        for name, (fn, algo, kind) in variants.items():
            g = timing.capture(fn, ns.graph, dev, warm_calls=2)
            with ClockSampler(local) as clk:
                t = timing.time_replays(g, ns.graph, ns.iters, ns.warmup, dev)
            del g
            c = clk.summary()
            st = main_ctx.status() if name.startswith("fp4ar") else cmp_ctx.status()
            emit({"kind": "timing", "variant": name, "mode": "fused", "algo": "twoshot" if algo else "oneshot", "tp": world,
                  "rows": rows, "input": "nvfp4" if kind else "bf16", "epilogue": 0, "med_us": round(t["med_us"], 3), "p10_us": round(t["p10_us"], 3),
                  "p90_us": round(t["p90_us"], 3), "sm_mhz": c.get("sm_mhz"), "reasons": c.get("reasons"),
                  "status": st.describe()})
        del xs, xqs, out
        torch.cuda.empty_cache()
    if rank == 0 and ns.out:
        with open(ns.out, "a") as f:
            for r in records:
                f.write(json.dumps(r) + "\n")
    main_ctx.close()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
