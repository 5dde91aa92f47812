"""Run a handful of launches of ONE fused-kernel shape on one GPU, for `ncu` and for quick timing.

    python -m fp4_all_reduce_b200.harness.profile_case --ranks 1 --rows 16384 --epilogue 1 --calls 3
    python -m fp4_all_reduce_b200.harness.profile_case --ranks 2 --rows 8192 --calls 3        # emulated ranks

With --ranks > 1 the ranks are emulated on the one GPU (one cooperative launch, SMs/ranks CTAs per rank), so a
profiler sees the real fused path, Lamport waits included, without a second process.  Prints one JSON line
with the CUDA-event time per call (after one warm-up call).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .. import _native as N
from ..parallel.context import EmulatedGroup, Fp4ArContext, SoloRankContext, make_args
from ..utils import data as D
from ..ops import codec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=1)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--epilogue", type=int, default=0)
    ap.add_argument("--input", type=int, default=0)
    ap.add_argument("--algo", type=int, default=-1)
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--calls", type=int, default=3)
    ap.add_argument("--teams", type=int, default=0)
    ap.add_argument("--team-warps", type=int, default=0)
    ap.add_argument("--lags", type=int, default=0, help="two-shot pipeline depths, lag_owner + 16 * lag_finish (0 = default)")
    ap.add_argument("--solo", action="store_true",
                    help="create rank 0 of a --ranks group on this GPU and launch it alone (needs --mode 2: every push is looped back)")
    ns = ap.parse_args(argv)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    P, rows = ns.ranks, ns.rows
    base = [D.partial(rows, r).to(dev) for r in range(P)]
    gs = None
    if ns.input == N.IN_NVFP4:
        gs = [float(b.float().abs().max().item()) / 2688.0 for b in base]
        xs = [codec.encode_static(b, g) for b, g in zip(base, gs)]
    else:
        xs = base
    res = [D.residual(rows).to(dev) for _ in range(P)]
    w = D.norm_weight().to(dev)
    outs = [torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(P)]
    nb = N.QROW_BYTES if ns.epilogue == 2 else N.MXROW_BYTES
    outq = [torch.empty(rows, nb, dtype=torch.uint8, device=dev) if ns.epilogue >= 2 else None for _ in range(P)]

    def args(r):
        return make_args(x=xs[r], out=outs[r] if ns.epilogue <= 1 else None, rows=rows, mode=ns.mode, algo=ns.algo,
                         input=ns.input, epilogue=ns.epilogue, gs=gs, res_in=res[r] if ns.epilogue else None,
                         res_out=res[r] if ns.epilogue else None, weight=w if ns.epilogue else None, outq=outq[r],
                         qscale=168.0, teams=ns.teams, team_warps=ns.team_warps, lags=ns.lags)

    if ns.solo:
        if ns.mode != N.MODE_COMPUTE:
            raise SystemExit("--solo needs --mode 2 (a rank launched alone would wait for peers that never run)")
        ctx = SoloRankContext(P, rows, dev)
        a0 = args(0)
        launch = lambda: ctx.launch(a0)
    elif P == 1:
        ctx = Fp4ArContext(rows, device=dev)
        a0 = args(0)
        launch = lambda: ctx.launch(a0)
    else:
        ctx = EmulatedGroup(P, rows)
        a_all = [args(r) for r in range(P)]     # built once: host work between the events would be timed
        launch = lambda: ctx.launch(a_all)
    launch()
    torch.cuda.synchronize()
    times = []
    for _ in range(ns.calls):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); launch(); b.record(); b.synchronize()
        times.append(a.elapsed_time(b) * 1000.0)
    st = ctx.status()
    print(json.dumps({"ranks": P, "rows": rows, "epilogue": ns.epilogue, "input": ns.input, "mode": ns.mode,
                      "team_warps": ns.team_warps, "lags": ns.lags, "solo": bool(ns.solo),
                      "us_per_call": [round(t, 2) for t in times], "status": st.describe(),
                      "ctas_per_rank": ctx.ctas_per_rank()}))
    ctx.close()
    return 0 if st.ok else 4


if __name__ == "__main__":
    sys.exit(main())
