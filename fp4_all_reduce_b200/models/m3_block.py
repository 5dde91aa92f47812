"""The communication skeleton of one MiniMax-M3 prefill step under tensor parallelism.

A prefill step runs 121 "blocks"; each block ends a row-parallel GEMM (o_proj, MLP / shared-expert down
projection) with  AllReduce -> residual add -> Gemma RMSNorm  over [tokens, 6144] activations
(reference project: README.md:3-5, docs/RESULTS.md:209-215 "per prefill step = block x 121").
`M3PrefillChain` is that chain with the GEMMs replaced by pre-computed partials, which is exactly what the
reference times; `M3PrefillChain.step()` launches the 121 fused kernels, `capture()` records them in one
CUDA graph.  `impl="nccl"` runs the same chain as BF16 NCCL AllReduce + the stand-alone add+RMSNorm
kernel: the baseline the fused kernels are measured against.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native as N
from ..ops import codec
from ..parallel.context import Fp4ArContext, input_sets_for
from ..utils import data as D

BLOCKS_PER_STEP = 121
L2_BYTES = 126 * 1024 * 1024


class M3PrefillChain:
    def __init__(self, ctx: Optional[Fp4ArContext], rows: int, *, blocks: int = BLOCKS_PER_STEP, impl: str = "fp4",
                 input_kind: int = N.IN_BF16, epilogue: int = N.EPI_NORM_BF16, algo: int = N.ALGO_AUTO,
                 norm: bool = True, device: Optional[torch.device] = None, rank: int = 0, nranks: int = 1, group=None,
                 teams: int = 0, qscale: float = 168.0, mode: int = N.MODE_FUSED, nsets: Optional[int] = None):
        self.ctx, self.rows, self.blocks, self.impl = ctx, rows, blocks, impl
        self.input_kind, self.epilogue, self.algo, self.norm = input_kind, epilogue, algo, norm
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.rank, self.nranks, self.group, self.teams, self.qscale, self.mode = rank, nranks, group, teams, qscale, mode
        row_bytes = N.HIDDEN * 2 if input_kind == N.IN_BF16 else N.QROW_BYTES
        # enough distinct partials that consecutive blocks never find their input in L2
        self.nsets = nsets if nsets else input_sets_for(rows, row_bytes, L2_BYTES)
        base = D.partial(rows, rank).to(self.device)
        self.gs = None
        if input_kind == N.IN_BF16:
            self.partials = [base.clone() if i == 0 else torch.roll(base, shifts=i, dims=0) for i in range(self.nsets)]
            # the NCCL arm reduces in place: pristine copies let `restore_partials()` undo that between replays
            self.pristine = [p.clone() for p in self.partials] if impl == "nccl" else None
        else:
            amax = base.float().abs().max()
            import torch.distributed as dist
            if nranks > 1 and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) == nranks:
                allmax = [torch.zeros_like(amax) for _ in range(nranks)]
                dist.all_gather(allmax, amax, group=group)
                self.gs = [float(a.item()) / 2688.0 for a in allmax]
            else:      # one rank, or a rank of a larger group running alone: every rank's scale is this rank's
                self.gs = [float(amax.item()) / 2688.0] * nranks
            q = codec.encode_static(base, self.gs[rank])
            self.partials = [q.clone() if i == 0 else torch.roll(q, shifts=i, dims=0) for i in range(self.nsets)]
        self.residual = D.residual(rows).to(self.device)
        self.residual0 = self.residual.clone()
        self.weight = D.norm_weight().to(self.device)
        self.out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=self.device)
        self.outq = None
        if epilogue == N.EPI_NORM_NVFP4:
            self.outq = torch.empty(rows, N.QROW_BYTES, dtype=torch.uint8, device=self.device)
        elif epilogue == N.EPI_NORM_MXFP8:
            self.outq = torch.empty(rows, N.MXROW_BYTES, dtype=torch.uint8, device=self.device)
        self.launches = 0

    def load_inputs(self, x_host: torch.Tensor, res_host: torch.Tensor) -> None:
        """Host -> device copy of one step's first partial and of the residual stream (pinned sources)."""
        self.partials[0].copy_(x_host, non_blocking=True)
        self.residual.copy_(res_host, non_blocking=True)

    def block(self, i: int) -> None:
        x = self.partials[i % self.nsets]
        if self.impl == "fp4":
            if self.norm:
                self.ctx.all_reduce_add_rms_norm(x, self.residual, self.weight, epilogue=self.epilogue, gs=self.gs,
                                                 algo=self.algo, out=self.out if self.outq is None else self.outq,
                                                 teams=self.teams, qscale=self.qscale, mode=self.mode)
            else:
                self.ctx.all_reduce(x, self.out, gs=self.gs, algo=self.algo, teams=self.teams, mode=self.mode)
            self.launches += 1
        else:
            import torch.distributed as dist

            # NCCL reduces the partial in place.  With one buffer per block of the graph (nsets >= blocks) and
            # `restore_partials()` between replays every all-reduce sees fresh, finite data; a longer chain that
            # reuses buffers averages instead of summing (same kernel, same bytes) so that values stay bounded.
            if self.nranks > 1:
                op = dist.ReduceOp.SUM if self.nsets >= self.blocks else dist.ReduceOp.AVG
                dist.all_reduce(x, op=op, group=self.group)
            if self.norm:
                codec.add_rmsnorm(x, self.residual, self.weight, inplace_residual=True, out=self.out)
                self.launches += 1

    def step(self) -> None:
        for i in range(self.blocks):
            self.block(i)

    def restore_partials(self) -> None:
        """NCCL arm: put the original partials back (call between replays, outside the timed region)."""
        if getattr(self, "pristine", None):
            for p, q in zip(self.partials, self.pristine):
                p.copy_(q)

    def reset_residual(self) -> None:
        self.residual.copy_(self.residual0)
