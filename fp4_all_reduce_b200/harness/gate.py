"""The bitwise correctness gate.

`expected(...)` evaluates the host bit-exact model for one call; `run_call` / `check_call` launch the fused
kernel on an `EmulatedGroup` or an `Fp4ArContext` and count mismatching 16-bit words; `gate_cell` runs
the multi-phase protocol on one (ranks, algorithm, input, epilogue, rows) cell:

  1. first call: mismatches against the host model, every rank bitwise identical, rel-L2 against the
     exact FP32 sum;
  2. `reps` back-to-back calls cycling three input sets (stale window contents cannot pass), compared
     after the last call;
  3. `reps` calls with a compare after every call and a count of bad calls;
  4. a CUDA graph of `graph_calls` calls replayed `graph_reps` times;
  5. calls with one rank delayed by a spin kernel, the delayed rank rotating.

Negative controls: `negctl="stale"` feeds the kernel the next input set while the expectation uses the
current one, `negctl="flip"` flips one bit of one rank's output before the compare, `negctl="bias"` (norm
epilogues) runs the kernel with the weight bias shifted by 2^-7 against the unshifted expectation; all must turn
every phase red.  This is the protocol of the reference project's harness (harness/fp4ar_bench.cu:248-347
and tests/negative_control.sh:11-18) re-stated for one-process-per-GPU groups and for the emulated group.
"""
from __future__ import annotations

import dataclasses

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .. import _native as N
from .. import oracle as O
from ..parallel.context import EmulatedGroup, make_args
from ..utils import data as D


@dataclass
class CellConfig:
    nranks: int
    rows: int
    algo: int = N.ALGO_AUTO
    input: int = N.IN_BF16
    epilogue: int = N.EPI_NONE
    dist: str = "partial"          # partial | mags | special
    eps: float = 1e-6
    weight_bias: float = 1.0
    qscale: float = 168.0
    teams: int = 0
    lags: int = 0                  # two-shot pipeline depths, lag_owner | lag_finish << 4 (0 = default)
    team_warps: int = 0            # warps per row team (0 = default)

    def resolved_algo(self) -> int:
        if self.nranks == 1:
            return 0
        if self.algo == N.ALGO_AUTO:
            return 0 if self.nranks <= 2 else 1
        return self.algo


@dataclass
class InputSet:
    xs: list                       # per rank: BF16 [rows,6144] (cuda) or NVFP4 rows [rows,3456] uint8 (cuda)
    gs: Optional[list]
    res: Optional[torch.Tensor]
    weight: Optional[torch.Tensor]
    exp: dict = field(default_factory=dict)      # host model outputs (numpy)
    exact: Optional[np.ndarray] = None           # exact FP32 sum of the BF16 partials
    exp_dev: dict = field(default_factory=dict)  # the same outputs on the device (bit patterns), for the compares


_GEN_CACHE: dict = {}


def _gen(cfg: CellConfig, rank: int, set_id: int) -> torch.Tensor:
    """One rank's BF16 partial of one input set.  Cells of a gate run that differ only in input kind or epilogue use
    the same partials, so the generated tensors are kept (for one row count and distribution at a time)."""
    key = (cfg.dist, cfg.rows, rank, set_id)
    if key in _GEN_CACHE:
        return _GEN_CACHE[key]
    if _GEN_CACHE and next(iter(_GEN_CACHE))[:2] != key[:2]:
        _GEN_CACHE.clear()
    if cfg.dist == "partial":
        x = D.partial(cfg.rows, rank, seed_offset=set_id)
    elif cfg.dist == "mags":
        x = D.gaussian_mags(cfg.rows, rank, set_id)
    elif cfg.dist == "special":
        x = D.special_rows(cfg.rows, rank + 3 * set_id)
    else:
        raise ValueError(cfg.dist)
    _GEN_CACHE[key] = x
    return x


def make_inputs(cfg: CellConfig, set_id: int, device) -> InputSet:
    """Inputs of one set and the host model's outputs for them."""
    bf = [_gen(cfg, r, set_id) for r in range(cfg.nranks)]
    bits = [O.bf16_bits(b) for b in bf]
    exact = np.zeros((cfg.rows, N.HIDDEN), np.float32)
    for b in bits:
        exact = exact + O.bf16_bits_to_f32(b)
    gs = None
    if cfg.input == N.IN_BF16:
        xs_dev = [b.to(device) for b in bf]
        model_in, kind = bits, 0
    else:
        # static calibration the way the reference harness emulates it: gs = tensor amax / 2688
        gs = []
        for b in bits:
            f = O.bf16_bits_to_f32(b)
            am = float(np.max(np.abs(f[np.isfinite(f)]))) if f.size else 1.0
            gs.append(float(np.float32(max(am, 1e-30) / 2688.0)))
        q = [O.encode_static(b, g) for b, g in zip(bits, gs)]
        xs_dev = [torch.from_numpy(a).to(device) for a in q]
        model_in, kind = q, 1
    res = weight = None
    res_bits = w_bits = None
    if cfg.epilogue != N.EPI_NONE:
        res = D.residual(cfg.rows, seed=4242 + set_id).to(device)
        weight = D.norm_weight().to(device)
        res_bits, w_bits = O.bf16_bits(res), O.bf16_bits(weight)
    exp = O.allreduce(model_in, algo=cfg.resolved_algo(), input_kind=kind, gs=gs, epi=cfg.epilogue, res_in=res_bits,
                      weight=w_bits, eps=cfg.eps, wbias=cfg.weight_bias, qscale=cfg.qscale)
    # The expectation is uploaded once: the per-call compares then run on the device (a 16K-row output is 200 MB;
    # bringing it to the host after every call would dominate the gate's run time on a multi-GPU machine).
    exp_dev = {}
    for k in ("out", "outq", "res_out"):
        v = exp.get(k)
        if v is not None:
            a = np.ascontiguousarray(v)
            exp_dev[k] = torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(device)
    return InputSet(xs_dev, gs, res, weight, exp, exact, exp_dev)


class Outputs:
    """Per-rank output buffers of one cell."""

    def __init__(self, cfg: CellConfig, device, nlocal: int):
        r, e = cfg.rows, cfg.epilogue
        self.out = [torch.zeros(r, N.HIDDEN, dtype=torch.bfloat16, device=device) if e <= 1 else None for _ in range(nlocal)]
        nb = N.QROW_BYTES if e == 2 else N.MXROW_BYTES
        self.outq = [torch.zeros(r, nb, dtype=torch.uint8, device=device) if e >= 2 else None for _ in range(nlocal)]
        self.res_out = [torch.zeros(r, N.HIDDEN, dtype=torch.bfloat16, device=device) if e >= 1 else None for _ in range(nlocal)]

    def clear(self):
        for lst in (self.out, self.outq, self.res_out):
            for t in lst:
                if t is not None:
                    t.zero_()


def args_for(cfg: CellConfig, inp: InputSet, outs: Outputs, local: int, rank: int, mode=N.MODE_FUSED) -> N.Args:
    return make_args(x=inp.xs[rank], out=outs.out[local], rows=cfg.rows, mode=mode, algo=cfg.algo, input=cfg.input,
                     epilogue=cfg.epilogue, gs=inp.gs, res_in=inp.res, res_out=outs.res_out[local], weight=inp.weight,
                     eps=cfg.eps, weight_bias=cfg.weight_bias, outq=outs.outq[local], qscale=cfg.qscale, teams=cfg.teams, lags=cfg.lags,
                     team_warps=cfg.team_warps)


def _mism(t: Optional[torch.Tensor], want: Optional[np.ndarray]) -> int:
    if t is None:
        return 0
    if t.dtype == torch.bfloat16:
        got = O.bf16_bits(t)
        w = want
        # a NaN is a NaN: the model canonicalises payloads, the comparison ignores them
        gn = (got & 0x7FFF) > 0x7F80
        wn = (w & 0x7FFF) > 0x7F80
        return int(np.count_nonzero((got != w) & ~(gn & wn)))
    return int(np.count_nonzero(t.cpu().numpy() != want))


def _mism_dev(t: Optional[torch.Tensor], want: Optional[torch.Tensor]) -> int:
    """The same count on the device: `want` holds the model's bit patterns (int16 for BF16 outputs, uint8 otherwise)."""
    if t is None:
        return 0
    if t.dtype == torch.bfloat16:
        got = t.view(torch.int16)
        gn = (got & 0x7FFF) > 0x7F80
        wn = (want & 0x7FFF) > 0x7F80
        return int(((got != want) & ~(gn & wn)).sum().item())
    return int((t != want).sum().item())


def mismatches(cfg: CellConfig, inp: InputSet, outs: Outputs, local: int) -> int:
    """Number of differing output elements of one local rank against the host model."""
    pairs = ((outs.out[local], "out"), (outs.outq[local], "outq"), (outs.res_out[local], "res_out"))
    if all(t is None or k in inp.exp_dev for t, k in pairs):
        return sum(_mism_dev(t, inp.exp_dev.get(k)) for t, k in pairs)
    return sum(_mism(t, inp.exp[k]) for t, k in pairs)


def rel_l2(inp: InputSet, out_bits: np.ndarray) -> float:
    got = O.bf16_bits_to_f32(out_bits).astype(np.float64)
    ex = inp.exact.astype(np.float64)
    ok = np.isfinite(got) & np.isfinite(ex)
    den = float(np.sqrt(np.sum(ex[ok] ** 2)))
    return float(np.sqrt(np.sum((got[ok] - ex[ok]) ** 2)) / den) if den > 0 else 0.0


def gate_cell_emulated(cfg: CellConfig, *, reps: int = 30, graph_calls: int = 5, graph_reps: int = 6,
                       negctl: Optional[str] = None, device=0, group: Optional[EmulatedGroup] = None) -> dict:
    """Phases 1-4 on an emulated group (phase 5 needs ranks that can be delayed independently)."""
    dev = torch.device("cuda", device)
    own = group is None
    g = group if group is not None else EmulatedGroup(cfg.nranks, max(cfg.rows, 1), device)
    g.set_timeout_ms(300)
    try:
        sets = [make_inputs(cfg, s, dev) for s in range(3)]
        outs = Outputs(cfg, dev, cfg.nranks)

        launch_cfg = dataclasses.replace(cfg, weight_bias=cfg.weight_bias + 2.0 ** -7) if negctl == "bias" else cfg

        def call(s: int):
            src = sets[(s + 1) % 3] if negctl == "stale" else sets[s % 3]
            g.launch([args_for(launch_cfg, src, outs, r, r) for r in range(cfg.nranks)])

        def compare(s: int) -> int:
            torch.cuda.synchronize()
            if negctl == "flip":
                t = outs.out[-1] if outs.out[-1] is not None else outs.outq[-1]
                flat = t.view(torch.uint8).view(-1)
                flat[0] ^= 1
            return sum(mismatches(cfg, sets[s % 3], outs, r) for r in range(cfg.nranks))

        rec = {"nranks": cfg.nranks, "rows": cfg.rows, "algo": cfg.resolved_algo(), "input": cfg.input,
               "epilogue": cfg.epilogue, "dist": cfg.dist, "negctl": negctl}
        # phase 1
        call(0)
        rec["mism_first"] = compare(0)
        if not g.status(0).ok:      # a wait gave up: the window is no longer consistent, stop here
            rec["status"] = g.status(0).describe()
            rec["pass"] = False
            return rec
        first = [t for t in (outs.out if cfg.epilogue <= 1 else outs.outq)]
        as_bits = lambda t: t.view(torch.int16) if t.dtype == torch.bfloat16 else t   # NaN == NaN bitwise
        rec["ranks_identical"] = all(torch.equal(as_bits(first[0]), as_bits(t)) for t in first[1:])
        if cfg.epilogue == N.EPI_NONE:
            rec["rel_l2_vs_fp32"] = rel_l2(sets[0], O.bf16_bits(outs.out[0]))
        # phase 2
        for s in range(1, reps + 1):
            call(s)
        rec["b2b_calls"] = reps
        rec["mism_b2b_final"] = compare(reps)
        # phase 3
        bad = 0
        total = 0
        for s in range(reps // 3 + 1):
            outs.clear()
            call(s)
            m = compare(s)
            total += m
            bad += m > 0
        rec["percall_calls"] = reps // 3 + 1
        rec["mism_percall"] = total
        rec["bad_calls_percall"] = bad
        # phase 4: graph of graph_calls calls over the rotating sets
        bad = 0
        if graph_calls > 0:
            st = torch.cuda.Stream(device=dev)
            st.wait_stream(torch.cuda.current_stream(dev))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(st):
                call(0)
                st.synchronize()
                with torch.cuda.graph(graph, stream=st):
                    for s in range(graph_calls):
                        call(s)
            for _ in range(graph_reps):
                outs.clear()
                graph.replay()
                bad += compare(graph_calls - 1) > 0
        rec["graph_calls"] = graph_calls * graph_reps
        rec["bad_graph_replays"] = bad
        stt = g.status(0)
        rec["status"] = stt.code
        rec["pass"] = (rec["mism_first"] == 0 and rec["ranks_identical"] and rec["mism_b2b_final"] == 0 and
                       rec["bad_calls_percall"] == 0 and rec["bad_graph_replays"] == 0 and stt.code == 0)
        return rec
    finally:
        if own:
            g.close()
