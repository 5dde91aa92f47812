"""Comparison variants of the one-shot AllReduce (flag push and pull), see csrc/kernels/compare_variants.cu.

`CompareEmulated(P, max_rows)` runs P ranks on one GPU (one cooperative launch; for tests and profiling);
`CompareContext(max_rows)` is the one-process-per-GPU form over torch symmetric memory.  Both give
`all_reduce(variant, x, out)` with variant "flag_push" or "pull"; results are bit-identical to the main
operator's one-shot path.  The reference project's counterparts are its `r1` control and `P` pull variants
(kernels/control/r1.cu, kernels/pull/tp2_p.cu).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native as N
from .context import Status

VARIANTS = {"flag_push": 0, "pull": 1}


def _lib():
    lib = N.cuda()
    lib.fp4ar_compare_window_bytes.restype = C.c_size_t
    lib.fp4ar_compare_window_bytes.argtypes = [C.c_int, C.c_int]
    lib.fp4ar_compare_allreduce.restype = C.c_int
    lib.fp4ar_compare_allreduce.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p,
                                            C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    return lib


def _check_io(x: torch.Tensor, out: torch.Tensor, max_rows: int):
    if x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or x.shape != out.shape or x.dim() != 2 or \
            x.shape[1] != N.HIDDEN or not x.is_contiguous() or not out.is_contiguous() or x.shape[0] > max_rows:
        raise ValueError("x and out must be contiguous bfloat16 [rows <= max_rows, 6144] tensors of the same shape")


class _CompareBase:
    timeout_ms = 2000

    def _status(self, t: torch.Tensor) -> Status:
        w = t.cpu().tolist()
        return Status(*[int(v) & 0xFFFFFFFF for v in w[:7]])


class CompareEmulated(_CompareBase):
    def __init__(self, nranks: int, max_rows: int, device: int | torch.device = 0):
        self.lib = _lib()
        self.nranks, self.max_rows = nranks, max_rows
        self.device = torch.device("cuda", device) if isinstance(device, int) else device
        self.window_bytes = int(self.lib.fp4ar_compare_window_bytes(max_rows, nranks))
        if self.window_bytes == 0:
            raise ValueError("unsupported shape")
        self.windows = [torch.zeros(self.window_bytes, dtype=torch.uint8, device=self.device) for _ in range(nranks)]
        self.status_words = [torch.zeros(8, dtype=torch.int32, device=self.device) for _ in range(nranks)]
        torch.cuda.synchronize(self.device)

    def all_reduce(self, variant: str, xs: Sequence[torch.Tensor], outs: Sequence[torch.Tensor],
                   stream: Optional[torch.cuda.Stream] = None) -> None:
        P = self.nranks
        if len(xs) != P or len(outs) != P:
            raise ValueError("one input and one output per rank")
        for x, o in zip(xs, outs):
            _check_io(x, o, self.max_rows)
        wins = (C.c_void_p * P)(*[w.data_ptr() for w in self.windows])
        xp = (C.c_void_p * P)(*[x.data_ptr() for x in xs])
        op = (C.c_void_p * P)(*[o.data_ptr() for o in outs])
        sp = (C.c_void_p * P)(*[s.data_ptr() for s in self.status_words])
        st = stream or torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            N.check(self.lib.fp4ar_compare_allreduce(VARIANTS[variant], 0, P, P, wins, self.window_bytes, self.max_rows, xp, op,
                                                     xs[0].shape[0], sp, self.timeout_ms, C.c_void_p(st.cuda_stream)),
                    "fp4ar_compare_allreduce")

    def status(self, rank: int = 0) -> Status:
        return self._status(self.status_words[rank])


class CompareContext(_CompareBase):
    """One process per GPU; the window is torch symmetric memory, zeroed, with a barrier before first use."""

    def __init__(self, max_rows: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist

        from .symmetric import allocate_symmetric

        self.lib = _lib()
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.nranks = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_rows = max_rows
        self.window_bytes = int(self.lib.fp4ar_compare_window_bytes(max_rows, self.nranks))
        if self.window_bytes == 0:
            raise ValueError("unsupported shape")
        self.window, self.ptrs, self._handle = allocate_symmetric(self.window_bytes, self.device, self.group)
        self.window.zero_()
        self.status_word = torch.zeros(8, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def all_reduce(self, variant: str, x: torch.Tensor, out: torch.Tensor, stream: Optional[torch.cuda.Stream] = None) -> None:
        _check_io(x, out, self.max_rows)
        P = self.nranks
        wins = (C.c_void_p * P)(*self.ptrs)
        xp = (C.c_void_p * 1)(x.data_ptr())
        op = (C.c_void_p * 1)(out.data_ptr())
        sp = (C.c_void_p * 1)(self.status_word.data_ptr())
        st = stream or torch.cuda.current_stream(self.device)
        N.check(self.lib.fp4ar_compare_allreduce(VARIANTS[variant], self.rank, P, 1, wins, self.window_bytes, self.max_rows, xp, op,
                                                 x.shape[0], sp, self.timeout_ms, C.c_void_p(st.cuda_stream)),
                "fp4ar_compare_allreduce")

    def status(self) -> Status:
        return self._status(self.status_word)
