"""Tuned BF16 NCCL AllReduce baseline: best of several NCCL configurations, measured like the fused kernels.

    python -m fp4_all_reduce_b200.harness.nccl_tuned --nproc 2 [--rows 1024,...,16384] [--norm] [--out nccl.jsonl]

NCCL reads NCCL_PROTO / NCCL_ALGO / NCCL_MIN_NCHANNELS when a communicator is created, so every configuration
runs in its own torchrun job (this program launches them one after another and keeps, per row count, the best
median).  Configurations: library defaults; Ring with LL128 / Simple and 64 channels; NVLS forced and off; each on
plain tensors and on buffers from ncclMemAlloc registered with the communicator (`--configs` picks a subset by
index).  Every all-reduce sums fresh data: one buffer per call of the graph, restored between replays.
The reference tunes the same knobs (harness/fp4ar_bench.cu:441-476, docs/RESULTS.md:89-97).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

CONFIGS = [
    {},
    {"NCCL_ALGO": "Ring", "NCCL_PROTO": "LL128", "NCCL_MIN_NCHANNELS": "64"},
    {"NCCL_ALGO": "Ring", "NCCL_PROTO": "Simple", "NCCL_MIN_NCHANNELS": "64"},
    {"NCCL_ALGO": "NVLS"},
    {"NCCL_NVLS_ENABLE": "0"},
]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nproc", type=int, default=2)
    ap.add_argument("--rows", default="1024,2048,4096,8192,16384")
    ap.add_argument("--norm", action="store_true")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--port", type=int, default=29700)
    ap.add_argument("--out", default=None)
    ap.add_argument("--configs", default="", help="comma list of indices into CONFIGS (default: all)")
    ap.add_argument("--no-reg", action="store_true", help="skip the registered-buffer arm")
    ns = ap.parse_args(argv)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    best = {}
    allrecs = []
    pick = [int(i) for i in ns.configs.split(",")] if ns.configs else list(range(len(CONFIGS)))
    for ci, cfg in enumerate(CONFIGS):
        if ci not in pick:
            continue
        env = dict(os.environ, **cfg, MASTER_ADDR="127.0.0.1")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ns.nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(ns.port + ci), "-m",
               "fp4_all_reduce_b200.harness.bench_cli", "--rows", ns.rows, "--nccl-only", "--nccl", *([] if ns.no_reg else ["--nccl-reg"]),
               "--iters", str(ns.iters),
               "--warmup", "5", "--epilogues", "0,1" if ns.norm else "0", "--tag", json.dumps(cfg, sort_keys=True)]
        try:
            p = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=600)
        except subprocess.TimeoutExpired:
            continue
        if p.returncode != 0:
            print(json.dumps({"kind": "nccl_config_failed", "nccl_env": cfg, "rc": p.returncode, "tail": p.stderr[-300:]}), flush=True)
        for line in p.stdout.splitlines():
            if not line.startswith("{"):
                continue
            r = json.loads(line)
            if not str(r.get("variant", "")).startswith("nccl") or "med_us" not in r:
                continue
            r["nccl_env"] = cfg
            allrecs.append(r)
            key = (r["rows"], r["epilogue"])
            if key not in best or r["med_us"] < best[key]["med_us"]:
                best[key] = r
    for key in sorted(best):
        r = dict(best[key]); r["kind"] = "timing"; r["best_of"] = r["variant"]; r["variant"] = "nccl_bf16_tuned" + ("+norm" if key[1] else "")
        print(json.dumps(r), flush=True)
        allrecs.append(r)
    if ns.out:
        with open(ns.out, "a") as f:
            for r in allrecs:
                f.write(json.dumps(r) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
