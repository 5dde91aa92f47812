"""Row-parallel linear + AllReduce + residual + Gemma RMSNorm, fused versus unfused, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port X \
        -m fp4_all_reduce_b200.harness.gemm_ar_bench [--ms 1024,4096,16384] [--graph 4] [--iters 20] [--check]

Per rank: X [M, 16384/P] ~ N(0,1), Wt [6144, 16384/P] ~ N(0, 1/sqrt(16384)) (BF16).  The static scale of every
rank is calibrated on a seed-1 batch (gs = amax of that rank's partial / 2688) and all-gathered.  Variants:

  fused      tcgen05 GEMM whose epilogue quantises and pushes into the peers' windows, then the AllReduce
             kernel in pushed-input mode with the residual + RMSNorm epilogue           (2 kernels)
  fp4_bf16   cuBLAS BF16 GEMM, then the fused NVFP4 AllReduce + residual + RMSNorm        (2 kernels)
  nccl       cuBLAS BF16 GEMM, NCCL BF16 AllReduce, stand-alone add + RMSNorm             (3 kernels)

--check compares the fused result of the first M with the host model fed with every rank's NVFP4 partial.
One JSON line per (M, variant): median microseconds per call (graph, max over ranks), roofline terms.
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
from ..ops import codec
from ..ops import gemm as G
from ..parallel.context import Fp4ArContext
from ..utils import data as D
from ..utils import timing
from ..utils.clocks import ClockSampler


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ms", dest="m", default="1024,4096,16384")
    ap.add_argument("--graph", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
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
    Ms = [int(m) for m in ns.m.split(",")]
    K = 16384 // world
    ctx = Fp4ArContext(max(Ms), device=dev)
    g = torch.Generator().manual_seed(100 + rank)
    wt = (torch.randn(N.HIDDEN, K, generator=g) / 16384 ** 0.5).to(torch.bfloat16).to(dev)
    # calibration batch (seed 1)
    gc = torch.Generator().manual_seed(1000 + rank)
    xc = torch.randn(512, K, generator=gc).to(torch.bfloat16).to(dev)
    my_gs = torch.tensor([G.calibrate_gs(xc, wt)], device=dev)
    if world > 1:
        alls = [torch.zeros_like(my_gs) for _ in range(world)]
        dist.all_gather(alls, my_gs)
        gs = [float(a.item()) for a in alls]
    else:
        gs = [float(my_gs.item())]
    weight = D.norm_weight().to(dev)
    records = []

    def emit(r):
        records.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    for M in Ms:
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
        res0 = D.residual(M).to(dev)
        res = res0.clone()
        out = torch.empty(M, N.HIDDEN, dtype=torch.bfloat16, device=dev)
        part = torch.empty(M, N.HIDDEN, dtype=torch.bfloat16, device=dev)

        if ns.check and M == Ms[0]:
            lq = torch.empty(M, N.QROW_BYTES, dtype=torch.uint8, device=dev)
            G.gemm_push(ctx, x, wt, gs[rank], local_q=lq)
            from ..parallel.context import make_args
            ctx.launch(make_args(x=None, out=out, rows=M, input=N.IN_PUSHED, gs=gs, epilogue=N.EPI_NORM_BF16, res_in=res,
                                 res_out=res, weight=weight, algo=N.ALGO_TWOSHOT if world > 2 else N.ALGO_ONESHOT))
            torch.cuda.synchronize()
            if world > 1:
                allq = [torch.empty_like(lq) for _ in range(world)]
                dist.all_gather(allq, lq)
            else:
                allq = [lq]
            exp = O.allreduce([q.cpu().numpy() for q in allq], algo=1 if world > 2 else 0, input_kind=1, gs=gs, epi=1,
                              res_in=O.bf16_bits(res0), weight=O.bf16_bits(weight))
            mism = int(np.count_nonzero(O.bf16_bits(out) != exp["out"])) + int(np.count_nonzero(O.bf16_bits(res) != exp["res_out"]))
            t = torch.tensor([mism], device=dev)
            if world > 1:
                dist.all_reduce(t)
            # accuracy of the whole fused path against an FP32 evaluation of sum(x @ wt.T) + residual
            emit({"kind": "check", "tp": world, "M": M, "mismatches_vs_host_model": int(t.item()),
                  "status": ctx.status().describe(), "gemm_status": G.gemm_status().code})
            res.copy_(res0)

        def fused(i):
            G.gemm_all_reduce_add_rms_norm(ctx, x, wt, gs, res, weight, out=out)

        def fp4_bf16(i):
            torch.matmul(x, wt.t(), out=part)
            ctx.all_reduce_add_rms_norm(part, res, weight, out=out)

        def nccl(i):
            torch.matmul(x, wt.t(), out=part)
            if world > 1:
                dist.all_reduce(part)
            codec.add_rmsnorm(part, res, weight, inplace_residual=True, out=out)

        def gemm_only(i):
            torch.matmul(x, wt.t(), out=part)

        flops = 2.0 * M * K * N.HIDDEN
        wire = M * 3456 * (1 if world <= 2 else 2 * (world - 1) / world) if world > 1 else 0
        for name, fn in (("fused", fused), ("fp4_bf16", fp4_bf16), ("nccl", nccl), ("cublas_gemm_only", gemm_only)):
            gph = timing.capture(fn, ns.graph, dev, warm_calls=1)
            with ClockSampler(local) as clk:
                t = timing.time_replays(gph, ns.graph, ns.iters, ns.warmup, dev)
            del gph
            c = clk.summary()
            emit({"kind": "timing", "variant": name, "tp": world, "M": M, "K": K, "N": N.HIDDEN,
                  "med_us": round(t["med_us"], 2), "p10_us": round(t["p10_us"], 2), "p90_us": round(t["p90_us"], 2),
                  "tflops": round(flops / t["med_us"] / 1e6, 1), "gemm_floor_us_at_1391T": round(flops / 1391e6, 1),
                  "link_floor_us_at_770GBs": round(wire / 770e3, 1), "sm_mhz": c.get("sm_mhz"), "reasons": c.get("reasons"),
                  "status": ctx.status().describe()})
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
