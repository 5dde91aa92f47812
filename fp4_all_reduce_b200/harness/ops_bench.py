"""Timing of the stand-alone codec / norm kernels on one GPU, as a fraction of the measured HBM copy rate.

    python -m fp4_all_reduce_b200.harness.ops_bench [--rows 16384] [--iters 20] [--ops encode,decode2,...]

Each op is timed with CUDA events on its stream after 3 warm-up launches; a 512 MiB buffer is overwritten
between timed launches so that no input is found in L2, and a short device-side sleep before the first event lets
the host enqueue the launch ahead of time, so the events bracket device time only.  Bytes counted are the algorithmic ones (inputs read
once, outputs written once).  The denominator is `hbm_gbs` of MEASURED_PEAKS.json next to the repository
root when present (a plain device copy measured on the same machine pool), else 6650 GB/s ("of fallback").
The reference project's equivalent is bench/codec/codec_bench.cu:730-928 (copy roof + per-kernel times).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from .. import _native as N
from ..ops import codec
from ..utils import data as D


def _peak():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ops", default="encode,encode_static,decode1,decode2,decode4,decode8,reencode4,norm_bf16,norm_nvfp4,norm_mxfp8,fill,copy")
    ns = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    rows = ns.rows
    peak, kind = _peak()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    x = D.partial(rows, 0).to(dev)
    res = D.residual(rows).to(dev)
    w = D.norm_weight().to(dev)
    enc = [codec.encode(torch.roll(x, i, 0)) for i in range(8)]
    qs, rss = [e[0] for e in enc], [e[1] for e in enc]
    gs = float(x.float().abs().max().item()) / 2688.0
    out_bf16 = torch.empty_like(x)
    win = torch.empty(2 * rows * N.REC_STRIDE, dtype=torch.uint8, device=dev)
    R, Q, B = rows * 3460, rows * N.QROW_BYTES, rows * N.HIDDEN * 2
    cases = {
        "encode": (lambda: codec.encode(x), B + R),
        "encode_static": (lambda: codec.encode_static(x, gs), B + Q),
        "decode1": (lambda: codec.decode_sum(qs[:1], rss[:1]), R + B),
        "decode2": (lambda: codec.decode_sum(qs[:2], rss[:2]), 2 * R + B),
        "decode4": (lambda: codec.decode_sum(qs[:4], rss[:4]), 4 * R + B),
        "decode8": (lambda: codec.decode_sum(qs[:8], rss[:8]), 8 * R + B),
        "reencode4": (lambda: codec.reduce_reencode(qs[:4], rss[:4]), 4 * R + B + R),
        "norm_bf16": (lambda: codec.add_rmsnorm(x, res, w, epilogue=1, inplace_residual=True, out=out_bf16), 4 * B),
        "norm_nvfp4": (lambda: codec.add_rmsnorm(x, res, w, epilogue=2, qscale=168.0, inplace_residual=True), 3 * B + Q),
        "norm_mxfp8": (lambda: codec.add_rmsnorm(x, res, w, epilogue=3, inplace_residual=True), 3 * B + rows * N.MXROW_BYTES),
        "fill": (lambda: codec.fill_sentinel(win, rows * N.REC_STRIDE, 2), 2 * rows * N.REC_STRIDE),
        "copy": (lambda: out_bf16.copy_(x), 2 * B),
    }
    for name in ns.ops.split(","):
        fn, nbytes = cases[name]
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(ns.iters):
            flush.fill_(1)
            torch.cuda._sleep(400_000)   # the GPU idles ~0.2 ms while the host enqueues: launch overhead stays outside the events
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); b.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        us = statistics.median(ts)
        gbs = nbytes / us / 1e3
        print(json.dumps({"op": name, "rows": rows, "med_us": round(us, 2), "bytes": nbytes, "gbs": round(gbs, 1),
                          "frac_of_hbm_copy": round(gbs / peak, 3), "peak_kind": kind, "peak_gbs": peak}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
