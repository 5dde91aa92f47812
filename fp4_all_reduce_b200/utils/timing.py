"""Device-side timing of graph-captured call sequences, max over ranks.

Protocol (that of the reference project's harness, harness/fp4ar_bench.cu:154-187, for one process per
GPU): capture `calls_per_graph` calls in a CUDA graph; before every iteration align the ranks (host
barrier through a 1-element all-reduce); bracket the replay with CUDA events on the launching stream;
after the loop take, per iteration, the maximum over ranks; report median / p10 / p90 per call.
"""
from __future__ import annotations

import statistics
from typing import Callable, Optional

import torch


def _dist():
    import torch.distributed as dist

    return dist if dist.is_available() and dist.is_initialized() else None


def align_ranks(device) -> None:
    d = _dist()
    if d is not None and d.get_world_size() > 1:
        t = torch.zeros(1, device=device)
        d.all_reduce(t)
    torch.cuda.synchronize(device)


def capture(fn: Callable[[int], None], calls: int, device, warm_calls: int = 2) -> torch.cuda.CUDAGraph:
    """Graph of fn(0), fn(1), ..., fn(calls-1) on a side stream."""
    st = torch.cuda.Stream(device=device)
    st.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(st):
        align_ranks(device)          # ranks may arrive seconds apart (host-side set-up); the device waits are bounded
        for i in range(warm_calls):
            fn(i)
        st.synchronize()
        align_ranks(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(calls):
                fn(i)
    torch.cuda.current_stream(device).wait_stream(st)
    torch.cuda.synchronize(device)
    return g


def time_replays(graph: torch.cuda.CUDAGraph, calls: int, iters: int, warmup: int, device,
                 before_each: Optional[Callable[[], None]] = None) -> dict:
    """Per-call microseconds of `iters` replays after `warmup` untimed ones; max over ranks per iteration."""
    for _ in range(warmup):
        align_ranks(device)
        graph.replay()
    torch.cuda.synchronize(device)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        if before_each is not None:
            before_each()
        align_ranks(device)
        a.record()
        graph.replay()
        b.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([a.elapsed_time(b) for a, b in ev], dtype=torch.float64, device=device)
    d = _dist()
    rank_med = [float(ms.median().item()) * 1000.0 / calls]           # this rank's own median, before the max over ranks
    if d is not None and d.get_world_size() > 1:
        try:
            mine = torch.tensor(rank_med, dtype=torch.float64, device=device)
            every = [torch.zeros_like(mine) for _ in range(d.get_world_size())]
            d.all_gather(every, mine)
            rank_med = [float(t.item()) for t in every]
        except Exception:        # the per-rank view is informational: never lose a measurement over it
            pass
        d.all_reduce(ms, op=d.ReduceOp.MAX)
    us = sorted((ms * 1000.0 / calls).tolist())
    n = len(us)
    return {"med_us": statistics.median(us), "p10_us": us[max(0, int(0.1 * n))], "p90_us": us[min(n - 1, int(0.9 * n))],
            "min_us": us[0], "iters": iters, "warmup": warmup, "calls_per_graph": calls,
            "total_ms": float(ms.sum().item()), "rank_med_us": [round(v, 3) for v in rank_med]}
