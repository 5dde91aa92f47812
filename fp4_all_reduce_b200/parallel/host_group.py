"""The NVFP4 AllReduce on the host, over any `torch.distributed` backend that moves CPU tensors (gloo).

Same wire records, same arithmetic and the same roles as the GPU operator -- every rank encodes its own rows, one-shot
ranks gather everybody's records and decode them in rank order, two-shot row owners (row % P) reduce, re-encode and
broadcast -- but executed by the host model (`csrc/oracle/oracle.cpp`) and moved by the process group's collectives.
Results are bit-identical to the GPU kernels and to `oracle.allreduce` fed with all ranks' inputs.

What it is for: running the distributed structure (who sends what to whom, rank order, ownership, uneven row counts)
on machines without GPUs, debugging a mismatch between ranks, and the multi-process tests of this package.  It is
not a fast path.  A peer that never shows up surfaces as the process group's timeout error, which `all_reduce`
turns into `PeerTimeout` -- the host-side counterpart of the kernels' bounded waits.

The reference project has no CPU rank path; its host model runs all "ranks" inside one process
(bench/codec/codec_bench.cu:594-674).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import _native as N
from .. import oracle as O


class PeerTimeout(RuntimeError):
    """A collective of the host path did not complete: some rank never joined or left."""


class HostAllReduce:
    def __init__(self, group=None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.nranks = dist.get_world_size(self.group)
        if self.nranks > N.MAX_RANKS:
            raise ValueError(f"at most {N.MAX_RANKS} ranks")

    # ------------------------------------------------------------------ transport helpers
    def _gather_records(self, rec: np.ndarray) -> list[np.ndarray]:
        """All ranks' record arrays (same shape everywhere), in rank order."""
        mine = torch.from_numpy(np.ascontiguousarray(rec))
        every = [torch.empty_like(mine) for _ in range(self.nranks)]
        try:
            dist.all_gather(every, mine, group=self.group)
        except RuntimeError as e:          # gloo reports a missing peer as a timeout / connection error
            raise PeerTimeout(str(e)) from e
        return [t.numpy() for t in every]

    @staticmethod
    def _pack(v: np.ndarray, s: np.ndarray, rs: np.ndarray) -> np.ndarray:
        """values | scales | row scale (4 bytes) per row: the payload of one window record."""
        rows = v.shape[0]
        rec = np.empty((rows, N.VALUE_BYTES + N.SCALE_BYTES + 4), np.uint8)
        rec[:, :N.VALUE_BYTES] = v
        rec[:, N.VALUE_BYTES:N.VALUE_BYTES + N.SCALE_BYTES] = s
        rec[:, N.VALUE_BYTES + N.SCALE_BYTES:] = np.ascontiguousarray(rs, np.float32).view(np.uint8).reshape(rows, 4)
        return rec

    @staticmethod
    def _unpack(rec: np.ndarray):
        v = np.ascontiguousarray(rec[:, :N.VALUE_BYTES])
        s = np.ascontiguousarray(rec[:, N.VALUE_BYTES:N.VALUE_BYTES + N.SCALE_BYTES])
        rs = np.ascontiguousarray(rec[:, N.VALUE_BYTES + N.SCALE_BYTES:]).view(np.float32).reshape(-1)
        return v, s, rs

    # ------------------------------------------------------------------ the operator
    def all_reduce(self, x: torch.Tensor, *, algo: int = N.ALGO_AUTO, gs: Optional[list] = None) -> torch.Tensor:
        """x: this rank's partial, BF16 [rows, 6144] (or NVFP4 rows [rows, 3456] uint8 with every rank's static scale
        in `gs`).  Returns the reduced BF16 [rows, 6144]; every rank gets the same bits."""
        P, me = self.nranks, self.rank
        if algo == N.ALGO_AUTO:
            algo = N.ALGO_ONESHOT if P <= 2 else N.ALGO_TWOSHOT
        if P == 1:
            algo = N.ALGO_ONESHOT
        if x.dtype == torch.bfloat16:
            v, s, rs = O.encode(O.bf16_bits(x), canon=True)
        else:
            if gs is None or len(gs) != P:
                raise ValueError("NVFP4 input needs the static scale of every rank")
            q = x.detach().cpu().numpy().reshape(-1, N.QROW_BYTES)
            v = np.ascontiguousarray(q[:, :N.VALUE_BYTES])
            s = np.ascontiguousarray(q[:, N.VALUE_BYTES:])
            rs = np.full(q.shape[0], np.float32(gs[me]), np.float32)
        rows = v.shape[0]
        recs = self._gather_records(self._pack(v, s, rs))          # one-shot: everyone's rows; two-shot: the
        acc = np.zeros((rows, N.HIDDEN), np.float32)               # reduce-scatter step delivers the same bytes
        if algo == N.ALGO_ONESHOT:
            for r in range(P):
                rv, rsc, rrs = self._unpack(recs[r])
                O.decode_acc(acc, rv, rsc, rrs)
            return O.from_bf16_bits(O.f32_to_bf16_bits(acc))
        # two-shot: the owner of a row reduces it in rank order, re-encodes the FP32 sum and broadcasts that
        own = np.arange(rows) % P == me
        n_own = int(own.sum())
        again = np.zeros((rows, N.VALUE_BYTES + N.SCALE_BYTES + 4), np.uint8)
        if n_own:
            part = np.zeros((n_own, N.HIDDEN), np.float32)
            for r in range(P):
                rv, rsc, rrs = self._unpack(recs[r][own])
                O.decode_acc(part, rv, rsc, rrs)
            ov, osc, ors = O.encode_f32(part, canon=True)
            again[own] = self._pack(ov, osc, ors)
        every = self._gather_records(again)                        # all-gather step: row i is valid in every[i % P]
        final = np.zeros_like(again)
        for r in range(P):
            sel = np.arange(rows) % P == r
            final[sel] = every[r][sel]
        fv, fs, frs = self._unpack(final)
        O.decode_acc(acc, fv, fs, frs)
        return O.from_bf16_bits(O.f32_to_bf16_bits(acc))
