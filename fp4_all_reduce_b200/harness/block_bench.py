"""The transformer block's "AllReduce -> residual add -> Gemma RMSNorm" against external baselines, one process per
GPU, measured like every other cell (K calls per CUDA graph, ranks aligned, CUDA events, max over ranks):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port X \
        -m fp4_all_reduce_b200.harness.block_bench [--rows 1024,4096,16384] [--out block.jsonl]

Variants (each is skipped with a record saying why when its library cannot be imported or fails on first use):

  fp4ar_block        this package's fused NVFP4 AllReduce + residual + RMSNorm kernel
  nccl+fp4ar_norm    NCCL BF16 all-reduce, then this package's stand-alone add + RMSNorm kernel
  nccl+vllm_norm     NCCL BF16 all-reduce, then vLLM's `fused_add_rms_norm` (weight passed as 1 + w: vLLM's kernel is
                     the plain RMSNorm form)
  nccl+flashinfer    NCCL BF16 all-reduce, then FlashInfer's `gemma_fused_add_rmsnorm`
  *_norm_only        the three norm kernels alone (no communication), for scale
  fp4ar_block_nvfp4out / nccl+vllm_norm+fp4quant
                     the block with NVFP4 rows out for a quantised next GEMM: this package's fused kernel
                     (`EPI_NORM_NVFP4`) against NCCL + vLLM's norm + vLLM's `scaled_fp4_quant`

Only library kernels that work on LOCAL tensors are used: fused all-reduce kernels of other libraries take peer
memory as an operand and are not run here.  The reference project's counterpart is bench/block/block_bench.py:22-43,
75-132 (vLLM and FlashInfer norm / quant kernels, FlashInfer's fused all-reduce, NCCL all-reduce (+ norm)).
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
from ..parallel.context import Fp4ArContext
from ..utils import data as D
from ..utils import timing
from ..utils.clocks import ClockSampler


def _external_norms(eps: float):
    """name -> (callable(x, residual, weight_plus_one, weight) or None, reason)."""
    out = {}
    try:
        from vllm import _custom_ops as vops

        out["vllm_norm"] = (lambda x, res, w1, w: vops.fused_add_rms_norm(x, res, w1, eps), "")
    except Exception as e:  # library missing or its extension cannot load
        out["vllm_norm"] = (None, f"{type(e).__name__}: {str(e)[:120]}")
    try:
        import flashinfer

        out["flashinfer"] = (lambda x, res, w1, w: flashinfer.norm.gemma_fused_add_rmsnorm(x, res, w, eps), "")
    except Exception as e:
        out["flashinfer"] = (None, f"{type(e).__name__}: {str(e)[:120]}")
    return out


def _external_fp4_quant():
    """(callable(x_bf16, global_scale_tensor) or None, reason): vLLM's NVFP4 quantiser of a local BF16 tensor."""
    try:
        from vllm import _custom_ops as vops

        return (lambda x, gsc: vops.scaled_fp4_quant(x, gsc)), ""
    except Exception as e:
        return None, f"{type(e).__name__}: {str(e)[:120]}"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", default="1024,4096,16384")
    ap.add_argument("--graph", type=int, default=10)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
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
    eps = 1e-6
    ext = _external_norms(eps)
    fp4q, fp4q_why = _external_fp4_quant()
    records = []

    def emit(r):
        records.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    for rows in rows_list:
        nsets = min(24, max(2, -(-2 * L2_BYTES // (rows * N.HIDDEN * 2))))
        base = D.partial(rows, rank).to(dev)
        xs = [base.clone() if i == 0 else torch.roll(base, i, 0) for i in range(nsets)]
        res = D.residual(rows).to(dev)
        w = D.norm_weight().to(dev)
        w1 = (w.float() + 1.0).to(torch.bfloat16)
        out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=dev)
        scratch = torch.empty_like(base)

        def ar(i):
            scratch.copy_(xs[i % nsets])          # library norms work in place: keep the rotating inputs intact
            if world > 1:
                dist.all_reduce(scratch)
            return scratch

        variants = {
            "fp4ar_block": lambda i: ctx.all_reduce_add_rms_norm(xs[i % nsets], res, w, out=out),
            "nccl+fp4ar_norm": lambda i: codec.add_rmsnorm(ar(i), res, w, inplace_residual=True, out=out),
            "fp4ar_norm_only": lambda i: codec.add_rmsnorm(xs[i % nsets], res, w, inplace_residual=True, out=out),
        }
        outq = torch.empty(rows, N.QROW_BYTES, dtype=torch.uint8, device=dev)
        qscale = 168.0                            # 448 * 6 / 16: activations of the order of 16 use the full range
        variants["fp4ar_block_nvfp4out"] = lambda i: ctx.all_reduce_add_rms_norm(
            xs[i % nsets], res, w, epilogue=N.EPI_NORM_NVFP4, qscale=qscale, out=outq)
        vnorm = ext.get("vllm_norm", (None, "vLLM norm unavailable"))[0]
        if fp4q is not None and vnorm is not None:
            gsc = torch.full((1,), qscale, dtype=torch.float32, device=dev)

            def vllm_chain(i, vnorm=vnorm):
                t = ar(i)
                vnorm(t, res, w1, w)               # in place: t = norm(t + res), res = t + res
                return fp4q(t, gsc)
            variants["nccl+vllm_norm+fp4quant"] = vllm_chain
        else:
            emit({"kind": "timing", "variant": "nccl+vllm_norm+fp4quant", "tp": world, "rows": rows,
                  "skipped": fp4q_why or "vLLM norm unavailable"})
        for name, (fn, why) in ext.items():
            if fn is None:
                emit({"kind": "timing", "variant": "nccl+" + name, "tp": world, "rows": rows, "skipped": why})
                continue
            variants["nccl+" + name] = lambda i, fn=fn: fn(ar(i), res, w1, w)
            variants[name + "_norm_only"] = lambda i, fn=fn: fn(scratch, res, w1, w)
        for name, fn in variants.items():
            try:
                res.copy_(D.residual(rows).to(dev))
                fn(0)                              # first use outside the capture: JIT builds, lazy initialisation
                torch.cuda.synchronize()
                g = timing.capture(fn, ns.graph, dev, warm_calls=1)
                with ClockSampler(local) as clk:
                    t = timing.time_replays(g, ns.graph, ns.iters, ns.warmup, dev)
                del g
            except Exception as e:
                emit({"kind": "timing", "variant": name, "tp": world, "rows": rows,
                      "skipped": f"{type(e).__name__}: {str(e)[:160]}"})
                continue
            c = clk.summary()
            emit({"kind": "timing", "variant": name, "mode": "fused", "algo": "auto", "tp": world, "rows": rows, "input": "bf16",
                  "epilogue": 2 if name in ("fp4ar_block_nvfp4out", "nccl+vllm_norm+fp4quant") else 1, "med_us": round(t["med_us"], 3), "p10_us": round(t["p10_us"], 3),
                  "p90_us": round(t["p90_us"], 3), "sm_mhz": c.get("sm_mhz"), "reasons": c.get("reasons")})
        del xs, out, scratch
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
