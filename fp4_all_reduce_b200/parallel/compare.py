"""Comparison variants of the AllReduce, see csrc/kernels/compare_variants.cu.

`CompareEmulated(P, max_rows)` runs P ranks on one GPU (one cooperative launch; for tests and profiling);
`CompareContext(max_rows)` is the one-process-per-GPU form over torch symmetric memory.  Both give
`all_reduce(variant, x, out, gs=None)` with variant

    "flag_push"        one-shot, direct stores + a release flag per tile (the control)
    "pull"             one-shot, records pulled from the producers' windows
    "pull_nvfp4"       the same with NVFP4 input rows ([rows, 3456] uint8) and static scales `gs`
    "pull_twoshot"     the row owner pulls, reduces and re-encodes; the others pull the re-encoding
    "pull_rs_push_ag"  the owner pulls and reduces, then stores the re-encoding into every peer

Results are bit-identical to the main operator's one-shot / two-shot host model.  The reference project's
counterparts are its `r1` control and its pull family `P`, `Pq`, `P4`, `P4t` (kernels/control/r1.cu,
kernels/pull/tp2_p.cu, tp2_pq.cu, tp4_p4.cu).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native as N
from .context import Status

VARIANTS = {"flag_push": 0, "pull": 1, "pull_nvfp4": 2, "pull_twoshot": 3, "pull_rs_push_ag": 4}
TWO_SHOT = ("pull_twoshot", "pull_rs_push_ag")


def _lib():
    lib = N.cuda()
    lib.fp4ar_compare_window_bytes.restype = C.c_size_t
    lib.fp4ar_compare_window_bytes.argtypes = [C.c_int, C.c_int]
    lib.fp4ar_compare_allreduce.restype = C.c_int
    lib.fp4ar_compare_allreduce.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p,
                                            C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    return lib


def _check_io(variant: str, x: torch.Tensor, out: torch.Tensor, max_rows: int, gs, nranks: int):
    if variant not in VARIANTS:
        raise KeyError(variant)
    if out.dtype != torch.bfloat16 or out.dim() != 2 or out.shape[1] != N.HIDDEN or not out.is_contiguous() or \
            x.dim() != 2 or x.shape[0] != out.shape[0] or not x.is_contiguous() or x.shape[0] > max_rows:
        raise ValueError("out must be a contiguous bfloat16 [rows <= max_rows, 6144] tensor and x must have as many rows")
    if variant == "pull_nvfp4":
        if x.dtype != torch.uint8 or x.shape[1] != N.QROW_BYTES:
            raise ValueError("pull_nvfp4 takes NVFP4 rows: uint8 [rows, 3456]")
        if gs is None or len(gs) != nranks or not all(float(g) > 0 for g in gs):
            raise ValueError("pull_nvfp4 needs one positive static scale per rank")
    elif x.dtype != torch.bfloat16 or x.shape[1] != N.HIDDEN:
        raise ValueError("x must be a contiguous bfloat16 [rows, 6144] tensor")


def _gs_array(gs):
    if gs is None:
        return None
    arr = (C.c_float * N.MAX_RANKS)()
    for i, g in enumerate(gs):
        arr[i] = float(g)
    return arr


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
                   stream: Optional[torch.cuda.Stream] = None, gs=None) -> None:
        P = self.nranks
        if len(xs) != P or len(outs) != P:
            raise ValueError("one input and one output per rank")
        for x, o in zip(xs, outs):
            _check_io(variant, x, o, self.max_rows, gs, P)
        wins = (C.c_void_p * P)(*[w.data_ptr() for w in self.windows])
        xp = (C.c_void_p * P)(*[x.data_ptr() for x in xs])
        op = (C.c_void_p * P)(*[o.data_ptr() for o in outs])
        sp = (C.c_void_p * P)(*[s.data_ptr() for s in self.status_words])
        st = stream or torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            N.check(self.lib.fp4ar_compare_allreduce(VARIANTS[variant], 0, P, P, wins, self.window_bytes, self.max_rows, xp, op,
                                                     xs[0].shape[0], _gs_array(gs), sp, self.timeout_ms,
                                                     C.c_void_p(st.cuda_stream)),
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

    def all_reduce(self, variant: str, x: torch.Tensor, out: torch.Tensor, stream: Optional[torch.cuda.Stream] = None,
                   gs=None) -> None:
        P = self.nranks
        _check_io(variant, x, out, self.max_rows, gs, P)
        wins = (C.c_void_p * P)(*self.ptrs)
        xp = (C.c_void_p * 1)(x.data_ptr())
        op = (C.c_void_p * 1)(out.data_ptr())
        sp = (C.c_void_p * 1)(self.status_word.data_ptr())
        st = stream or torch.cuda.current_stream(self.device)
        N.check(self.lib.fp4ar_compare_allreduce(VARIANTS[variant], self.rank, P, 1, wins, self.window_bytes, self.max_rows, xp, op,
                                                 x.shape[0], _gs_array(gs), sp, self.timeout_ms, C.c_void_p(st.cuda_stream)),
                "fp4ar_compare_allreduce")

    def status(self) -> Status:
        return self._status(self.status_word)
