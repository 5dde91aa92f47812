"""Run the reference project's own kernels (built by baseline/build_ref.py) on this machine.

    python baseline/reference_arm.py check  [--tp 2] [--rows 512] [--input bf16|nvfp4]
                                  bit-compare the reference's L2 / L4 output with this repository's host model
    python baseline/reference_arm.py sweep  [--tp 2] [--out ref.jsonl] [--input bf16|nvfp4]
                                  latency of L2 / L4 / lnorm at 1K..16K rows

The binary runs all ranks as threads of one process on GPUs 0..tp-1.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SHIM = HERE / "_ref" / "ref_shim"
sys.path.insert(0, str(HERE.parent))


def run_shim(args, timeout=300):
    if not SHIM.exists():
        return {"impl": "reference", "unavailable": "baseline/_ref/ref_shim has not been built (python baseline/build_ref.py)"}
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([str(SHIM)] + [str(a) for a in args], capture_output=True, text=True, timeout=timeout, env=env)
    for line in p.stdout.splitlines():
        if line.startswith("{"):
            return json.loads(line)
    return {"impl": "reference", "unavailable": f"driver exited with code {p.returncode}: {(p.stderr or p.stdout)[-300:]}"}


def check(tp: int, rows: int, input_kind: str = "bf16") -> int:
    from fp4_all_reduce_b200 import oracle as O
    from fp4_all_reduce_b200.utils import data as D

    ok = True
    with tempfile.TemporaryDirectory() as td:
        pre = os.path.join(td, "case")
        xs = [O.bf16_bits(D.gaussian_mags(rows, r, 7)) for r in range(tp)]
        for r, x in enumerate(xs):
            x.tofile(f"{pre}.x{r}.bin")
        for variant, algo in (("L2", 0), ("L2", 1), ("L4", 0), ("L4", 1)):
            if variant == "L4" and tp != 4:
                continue
            if input_kind == "nvfp4" and variant == "L2" and algo == 1:
                continue        # the reference's L2 takes NVFP4 input for its one-shot path only (kernels/push/tp2_l2.cu:1031)
            rec = run_shim(["--tp", tp, "--variant", variant, "--rows", rows, "--algo", algo, "--graph", 2, "--iters", 3,
                            "--warmup", 1, "--in", pre, "--dump", pre, "--input", input_kind])
            if "unavailable" in rec:
                print(json.dumps(rec)); return 1
            got = np.fromfile(f"{pre}.out.bin", dtype=np.uint16).reshape(rows, 6144)
            if input_kind == "nvfp4":
                # the driver's static scales (amax / 2688 per rank) and this repository's static-scale quantiser
                gs = [float(v) for v in np.fromfile(f"{pre}.gs.bin", dtype=np.float32)[:tp]]
                want = O.allreduce([O.encode_static(x, g) for x, g in zip(xs, gs)], algo=algo, input_kind=1, gs=gs)["out"]
            else:
                want = O.allreduce(xs, algo=algo)["out"]
            mism = int(np.count_nonzero(got != want))
            ok &= mism == 0
            print(json.dumps({"kind": "reference_vs_host_model", "variant": variant, "input": input_kind, "algo": algo, "tp": tp,
                              "rows": rows, "mismatches": mism}))
    return 0 if ok else 3


def sweep(tp: int, out: str | None, input_kind: str = "bf16") -> int:
    recs = []
    for rows in (1024, 2048, 4096, 8192, 16384):
        cases = [("L2", 0, 0)] if tp == 2 else [("L4", 1, 0), ("L4", 0, 0)]
        if input_kind == "bf16" or tp == 2:      # the reference's fused norm takes NVFP4 input at 2 ranks only
            cases += [("lnorm", 0, 1)]
        for variant, algo, epi in cases:
            rec = run_shim(["--tp", tp, "--variant", variant, "--rows", rows, "--algo", algo, "--epi", epi, "--graph", 10,
                            "--iters", 30, "--warmup", 5, "--input", input_kind])
            rec["algo"] = algo
            recs.append(rec)
            print(json.dumps(rec), flush=True)
    if out:
        with open(out, "a") as f:
            for r in recs:
                f.write(json.dumps(r) + "\n")
    return 0


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["check", "sweep"])
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--rows", type=int, default=512)
    ap.add_argument("--out", default=None)
    ap.add_argument("--input", default="bf16", choices=["bf16", "nvfp4"])
    ns = ap.parse_args()
    sys.exit(check(ns.tp, ns.rows, ns.input) if ns.cmd == "check" else sweep(ns.tp, ns.out, ns.input))
