"""Timing of the tcgen05 GEMM with NVFP4 epilogue against a plain BF16 matmul (cuBLAS through torch).

    python -m fp4_all_reduce_b200.harness.gemm_bench [--ms 1024,4096,16384] [--tp 2,4,8] [--iters 10]

Per (M, tensor-parallel degree): K = 16384 / tp, N = 6144.  Reports microseconds, TFLOP/s and the fraction of
the measured cuBLAS BF16 rate (`bf16_tflops_sustained` of MEASURED_PEAKS.json when present, else 1400 "of
fallback").  The GEMM here writes NVFP4 rows (3456 B per row) instead of a BF16 tensor (12288 B per row).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from ..ops import gemm as G


def _peak():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1400.0, "fallback"


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        torch.cuda._sleep(400_000)   # the GPU idles ~0.2 ms while the host enqueues: launch overhead stays outside the events
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record(); b.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    return statistics.median(ts)


def _plan(M: int, Nn: int, K: int) -> dict:
    """The shape the library takes for this size by itself (environment overrides of a run are not reflected)."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    pl = G.gemm_plan(M, Nn, K, sms)
    return {"pair": pl["pair"], "tile_n": pl["tile_n"], "stream_k": pl["stream_k"], "units": pl["units"], "tiles": pl["tiles"]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ms", dest="m", default="1024,4096,16384")
    ap.add_argument("--tp", default="2,4,8")
    ap.add_argument("--iters", type=int, default=10)
    ns = ap.parse_args(argv)
    torch.cuda.set_device(0)
    peak, kind = _peak()
    Nn = 6144
    for tp in (int(t) for t in ns.tp.split(",")):
        K = 16384 // tp
        g = torch.Generator().manual_seed(tp)
        wt = (torch.randn(Nn, K, generator=g) / 16384 ** 0.5).to(torch.bfloat16).cuda()
        for M in (int(m) for m in ns.m.split(",")):
            x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
            gs = G.calibrate_gs(x[:256], wt)
            out = torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda")
            us_ours = _time(lambda: G.gemm_nvfp4(x, wt, gs), ns.iters)
            us_ref = _time(lambda: torch.matmul(x, wt.t(), out=out), ns.iters)
            fl = 2.0 * M * K * Nn
            print(json.dumps({"op": "gemm_nvfp4", "M": M, "K": K, "N": Nn, "tp": tp, "us": round(us_ours, 1),
                              "tflops": round(fl / us_ours / 1e6, 1), "frac_of_cublas_bf16": round(fl / us_ours / 1e6 / peak, 3),
                              "cublas_bf16_us": round(us_ref, 1), "cublas_tflops": round(fl / us_ref / 1e6, 1),
                              "peak_kind": kind, "plan": _plan(M, Nn, K), "status": G.gemm_status().code}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
