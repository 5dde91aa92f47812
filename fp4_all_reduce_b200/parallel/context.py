"""AllReduce contexts: the Python owner of a receive window and of the native `fp4ar_ctx`.

* `Fp4ArContext`      one rank of a `torch.distributed` process group (one process per GPU).  The window is
                      CUDA symmetric memory: every rank allocates the same size, the handles are exchanged
                      once at construction, and each rank ends up with a device pointer to every peer's
                      window over NVLink.  NCCL is used only for the rendezvous and the arm barrier.
* `EmulatedGroup`     all ranks of a group on ONE GPU, run as CTA groups of a single cooperative launch.
                      Exists for tests and for profiling the fused kernel where a profiler cannot follow
                      peers that wait on one another.

What the reference project does instead: one host thread per GPU inside one process, `ncclMemAlloc` +
`ncclCommWindowRegister` + `ncclGetLsaDevicePointer` (harness/fp4ar_bench.cu:384-394).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import _native as N


@dataclass
class Status:
    code: int
    row: int
    source: int
    detail: int
    cta: int
    call: int
    count: int

    @property
    def ok(self) -> bool:
        return self.code == 0

    def describe(self) -> str:
        names = {0: "ok", 1: "peer data did not arrive in time", 2: "local load did not complete in time",
                 3: "inconsistent launch parameters"}
        phases = {1: "one-shot gather", 2: "owner reduce", 3: "broadcast gather", 4: "local load"}
        if self.ok:
            return "ok"
        return (f"{names.get(self.code, self.code)} (call {self.call}, row {self.row}, source rank {self.source}, "
                f"{phases.get(self.detail, self.detail)}, CTA {self.cta}, {self.count} waits gave up)")


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> C.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def make_args(*, x=None, out=None, rows: int, mode=N.MODE_FUSED, algo=N.ALGO_AUTO, input=N.IN_BF16,
              epilogue=N.EPI_NONE, gs: Optional[Sequence[float]] = None, res_in=None, res_out=None, weight=None,
              eps: float = 1e-6, weight_bias: float = 1.0, outq=None, qscale: float = 1.0,
              teams: int = 0, no_pdl: bool = False, team_warps: int = 0, lags: int = 0) -> N.Args:
    a = N.Args()
    a.x = _ptr(x); a.out = _ptr(out)
    a.rows = rows; a.hidden = N.HIDDEN
    a.mode = mode; a.algo = algo; a.input = input; a.epilogue = epilogue
    for i in range(N.MAX_RANKS):
        a.gs[i] = float(gs[i]) if gs is not None and i < len(gs) else 1.0
    a.res_in = _ptr(res_in); a.res_out = _ptr(res_out); a.weight = _ptr(weight)
    a.eps = eps; a.weight_bias = weight_bias
    a.outq = _ptr(outq); a.qscale = qscale
    a.tune[0] = teams; a.tune[1] = 1 if no_pdl else 0; a.tune[2] = team_warps; a.tune[3] = lags
    return a


class _Base:
    """Shared by both context kinds: status, timeout, teardown."""

    _ctx: C.c_void_p
    nranks: int
    max_rows: int

    def status(self, local_rank: int = 0) -> Status:
        w = N.StatusWords()
        N.check(N.cuda().fp4ar_status(self._ctx, local_rank, C.byref(w)), "fp4ar_status")
        return Status(w.code, w.row, w.source, w.detail, w.cta, w.call, w.count)

    def set_timeout_ms(self, ms: int) -> None:
        N.check(N.cuda().fp4ar_set_timeout_ms(self._ctx, int(ms)), "fp4ar_set_timeout_ms")

    def ctas_per_rank(self) -> int:
        return int(N.cuda().fp4ar_ctas_per_rank(self._ctx))

    def push_view(self, local_rank: int = 0) -> N.PushView:
        v = N.PushView()
        N.check(N.cuda().fp4ar_get_push_view(self._ctx, local_rank, C.byref(v)), "fp4ar_get_push_view")
        return v

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            torch.cuda.synchronize()
            N.cuda().fp4ar_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class EmulatedGroup(_Base):
    """`nranks` ranks on one device.  `launch(args_per_rank)` runs one call of every rank."""

    def __init__(self, nranks: int, max_rows: int, device: int | torch.device = 0):
        self.device = torch.device("cuda", device) if isinstance(device, int) else device
        self.nranks, self.max_rows = nranks, max_rows
        lib = N.cuda()
        self.window_bytes = int(lib.fp4ar_window_bytes(max_rows, N.HIDDEN, nranks))
        if self.window_bytes == 0:
            raise ValueError("unsupported shape")
        self.windows = [torch.empty(self.window_bytes, dtype=torch.uint8, device=self.device) for _ in range(nranks)]
        ptrs = (C.c_void_p * nranks)(*[w.data_ptr() for w in self.windows])
        ctx = C.c_void_p()
        N.check(lib.fp4ar_create_emulated(C.byref(ctx), nranks, self.device.index or 0, max_rows, N.HIDDEN, ptrs,
                                          self.window_bytes), "fp4ar_create_emulated")
        self._ctx = ctx

    def launch(self, args: Sequence[N.Args], stream: Optional[torch.cuda.Stream] = None) -> None:
        if len(args) != self.nranks:
            raise ValueError("one argument block per rank")
        arr = (N.Args * self.nranks)(*args)
        N.check(N.cuda().fp4ar_launch(self._ctx, arr, _stream_ptr(stream)), "fp4ar_launch")

    def reset(self) -> None:
        N.check(N.cuda().fp4ar_reset(self._ctx), "fp4ar_reset")


def input_sets_for(rows: int, row_bytes: int, l2_bytes: int = 126 * 1024 * 1024, most: int = 24) -> int:
    """How many rotating copies of a [rows, row_bytes] input a timed chain needs so that consecutive calls never find
    their input in the L2 cache (together they exceed twice its size)."""
    return min(most, max(2, -(-2 * l2_bytes // (rows * row_bytes))))


class Fp4ArContext(_Base):
    """One rank of a tensor-parallel group; `group` is a torch.distributed process group (NCCL)."""

    def __init__(self, max_rows: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.rank = dist.get_rank(self.group)
            self.nranks = dist.get_world_size(self.group)
        else:                      # no process group: a one-rank context (encode, decode of the own encoding, epilogue)
            self.group, self.rank, self.nranks = None, 0, 1
        self.max_rows = max_rows
        if device is None or device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        lib = N.cuda()
        self.window_bytes = int(lib.fp4ar_window_bytes(max_rows, N.HIDDEN, self.nranks))
        if self.window_bytes == 0:
            raise ValueError(f"unsupported group size {self.nranks} or max_rows {max_rows}")
        if self.nranks == 1:
            self.window = torch.empty(self.window_bytes, dtype=torch.uint8, device=self.device)
            ptr_list = [self.window.data_ptr()]
            self._handle = None
        else:
            from .symmetric import allocate_symmetric

            self.window, ptr_list, self._handle = allocate_symmetric(self.window_bytes, self.device, self.group)
        ptrs = (C.c_void_p * self.nranks)(*ptr_list)
        ctx = C.c_void_p()
        N.check(lib.fp4ar_create(C.byref(ctx), self.rank, self.nranks, self.device.index or 0, max_rows, N.HIDDEN,
                                 ptrs, self.window_bytes), "fp4ar_create")
        self._ctx = ctx
        self._barrier()   # nobody pushes before every window is armed

    def _barrier(self) -> None:
        import torch.distributed as dist

        torch.cuda.synchronize()
        if self.nranks > 1:
            dist.barrier(group=self.group, device_ids=[self.device.index or 0])
            torch.cuda.synchronize()

    def launch(self, args: N.Args, stream: Optional[torch.cuda.Stream] = None) -> None:
        arr = (N.Args * 1)(args)
        N.check(N.cuda().fp4ar_launch(self._ctx, arr, _stream_ptr(stream)), "fp4ar_launch")

    def reset(self) -> None:
        """Collective: every rank must call it."""
        self._barrier()
        N.check(N.cuda().fp4ar_reset(self._ctx), "fp4ar_reset")
        self._barrier()

    # ---- argument checks of the convenience wrappers (the kernel trusts its pointers) ----
    def _check_input(self, x: torch.Tensor, gs) -> int:
        """Returns the input kind after checking dtype, shape, contiguity, scales, row count and device."""
        from ..ops.codec import _req_layout

        if x.dtype == torch.bfloat16:
            _req_layout(x, torch.bfloat16, N.HIDDEN, "x")
            kind = N.IN_BF16
        elif x.dtype == torch.uint8:
            _req_layout(x, torch.uint8, N.QROW_BYTES, "x (NVFP4 rows)")
            kind = N.IN_NVFP4
            if gs is None or len(gs) != self.nranks or not all(float(g) > 0.0 for g in gs):
                raise ValueError(f"NVFP4 input needs `gs`: one positive static scale per rank ({self.nranks})")
        else:
            raise ValueError(f"x must be bfloat16 [rows, {N.HIDDEN}] or uint8 NVFP4 rows [rows, {N.QROW_BYTES}], got {x.dtype}")
        if x.shape[0] > self.max_rows:
            raise ValueError(f"{x.shape[0]} rows exceed the context's max_rows {self.max_rows}")
        if x.device != self.device:
            raise ValueError(f"x is on {x.device}, the context on {self.device}")
        return kind

    def _check_like(self, t: torch.Tensor, dtype, rows: int, cols: int, name: str) -> None:
        from ..ops.codec import _req_layout

        _req_layout(t, dtype, cols, name)
        if t.shape[0] != rows:
            raise ValueError(f"{name} must have {rows} rows, got {t.shape[0]}")
        if t.device != self.device:
            raise ValueError(f"{name} is on {t.device}, the context on {self.device}")

    # ---- convenience wrappers: allocate outputs, launch on the current stream ----
    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, *, gs=None, algo=N.ALGO_AUTO,
                   mode=N.MODE_FUSED, teams: int = 0) -> torch.Tensor:
        """x: BF16 [rows,6144] partial, or NVFP4 rows [rows,3456] uint8 with the static scales `gs`."""
        kind = self._check_input(x, gs)
        rows = x.shape[0]
        if out is None:
            out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=x.device)
        else:
            self._check_like(out, torch.bfloat16, rows, N.HIDDEN, "out")
        self.launch(make_args(x=x, out=out, rows=rows, input=kind, gs=gs, algo=algo, mode=mode, teams=teams))
        return out

    def all_reduce_add_rms_norm(self, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, *,
                                eps: float = 1e-6, weight_bias: float = 1.0, epilogue=N.EPI_NORM_BF16,
                                qscale: float = 1.0, gs=None, algo=N.ALGO_AUTO, out: Optional[torch.Tensor] = None,
                                residual_out: Optional[torch.Tensor] = None, mode=N.MODE_FUSED, teams: int = 0):
        """Returns (normed output, updated residual).  `residual_out=None` updates `residual` in place."""
        kind = self._check_input(x, gs)
        rows = x.shape[0]
        if epilogue not in (N.EPI_NORM_BF16, N.EPI_NORM_NVFP4, N.EPI_NORM_MXFP8):
            raise ValueError("epilogue must be 1 (BF16), 2 (NVFP4) or 3 (MXFP8)")
        self._check_like(residual, torch.bfloat16, rows, N.HIDDEN, "residual")
        if residual_out is not None:
            self._check_like(residual_out, torch.bfloat16, rows, N.HIDDEN, "residual_out")
        if (weight.device != self.device or weight.dtype != torch.bfloat16 or weight.numel() != N.HIDDEN
                or not weight.is_contiguous()):
            raise ValueError(f"weight must be a contiguous bfloat16 tensor of {N.HIDDEN} elements on {self.device}")
        res_out = residual if residual_out is None else residual_out
        o = q = None
        if epilogue == N.EPI_NORM_BF16:
            if out is not None:
                self._check_like(out, torch.bfloat16, rows, N.HIDDEN, "out")
            o = out if out is not None else torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=x.device)
        else:
            nb = N.QROW_BYTES if epilogue == N.EPI_NORM_NVFP4 else N.MXROW_BYTES
            if out is not None:
                self._check_like(out, torch.uint8, rows, nb, "out")
            q = out if out is not None else torch.empty(rows, nb, dtype=torch.uint8, device=x.device)
        self.launch(make_args(x=x, out=o, rows=rows, input=kind, gs=gs, algo=algo, epilogue=epilogue, res_in=residual,
                              res_out=res_out, weight=weight, eps=eps, weight_bias=weight_bias, outq=q, qscale=qscale,
                              mode=mode, teams=teams))
        return (o if o is not None else q), res_out


class SoloRankContext(Fp4ArContext):
    """Rank 0 of an `nranks` group created ALONE on one GPU: every "peer" window is this GPU's own window.

    Only the compute mode (`mode=MODE_COMPUTE`: the full codec, owner and epilogue work of one rank, every push
    looped back into the own window, no wait on a peer) may be launched on it; a fused or transport-only launch
    would wait for peers that never run and end with a PeerTimeout status.  It is the one-GPU stand-in for a rank
    of a real group: what a profiler captures, and what `bench.py --gpus 1` times.  The reference project has the
    same mode (include/fp4ar_api.h:12-16, FP4AR_COMPUTE)."""

    def __init__(self, nranks: int, max_rows: int, device: Optional[torch.device] = None):
        if device is None or device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.group, self.rank, self.nranks, self.max_rows, self.device = None, 0, nranks, max_rows, device
        lib = N.cuda()
        self.window_bytes = int(lib.fp4ar_window_bytes(max_rows, N.HIDDEN, nranks))
        if self.window_bytes == 0:
            raise ValueError(f"unsupported group size {nranks} or max_rows {max_rows}")
        self.window = torch.empty(self.window_bytes, dtype=torch.uint8, device=device)
        self._handle = None
        ptrs = (C.c_void_p * nranks)(*([self.window.data_ptr()] * nranks))
        ctx = C.c_void_p()
        N.check(lib.fp4ar_create(C.byref(ctx), 0, nranks, device.index or 0, max_rows, N.HIDDEN, ptrs,
                                 self.window_bytes), "fp4ar_create")
        self._ctx = ctx

    def launch(self, args: N.Args, stream: Optional[torch.cuda.Stream] = None) -> None:
        if args.mode != N.MODE_COMPUTE:
            raise ValueError("a rank created alone can only run compute-mode calls (mode=MODE_COMPUTE)")
        super().launch(args, stream)
