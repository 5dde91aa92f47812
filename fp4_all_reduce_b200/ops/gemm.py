"""Row-parallel linear layer with the NVFP4 epilogue (tcgen05 / TMEM kernel, csrc/kernels/gemm_fp4.cu).

    q = gemm_nvfp4(x, wt, gs)                        # [M, N/2 + N/16] NVFP4 rows of x @ wt.T, static scale gs
    gemm_push(ctx, x, wt, gs_self)                   # same, stored straight into the AllReduce receive windows
    y, res = gemm_all_reduce_add_rms_norm(ctx, x, wt, gs, residual, weight)   # GEMM -> push -> fused AR + norm

`wt` is the weight in nn.Linear layout [N, K] (K contiguous).  `calibrate_gs` derives the static per-rank
scale from a calibration batch: gs = amax(|x @ wt.T|) / 2688, the convention of the reference harness
(harness/fp4ar_bench.cu:206-214) applied to a real GEMM output.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native as N


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(x: torch.Tensor, wt: torch.Tensor):
    if not (x.is_cuda and wt.is_cuda and x.dtype == torch.bfloat16 and wt.dtype == torch.bfloat16):
        raise ValueError("x and wt must be CUDA BF16 tensors")
    if x.dim() != 2 or wt.dim() != 2 or x.shape[1] != wt.shape[1] or not x.is_contiguous() or not wt.is_contiguous():
        raise ValueError("x [M, K] and wt [N, K] must be contiguous with equal K")
    M, K = x.shape
    Nn = wt.shape[0]
    if K % 64 or Nn % 256:
        raise ValueError("K must be a multiple of 64 and N a multiple of 256")
    return M, Nn, K


def calibrate_gs(x: torch.Tensor, wt: torch.Tensor) -> float:
    """Static scale of this rank's partial from a calibration batch (runs a plain BF16 matmul)."""
    y = torch.matmul(x, wt.t()).float()
    return max(float(y.abs().max().item()), 1e-30) / 2688.0


def gemm_nvfp4(x: torch.Tensor, wt: torch.Tensor, gs: float, *, want_acc: bool = False, out: Optional[torch.Tensor] = None):
    """Local NVFP4 rows of x @ wt.T (into `out` when given); with want_acc also the kernel's FP32 accumulators [M, N]."""
    M, Nn, K = _check(x, wt)
    if out is None:
        q = torch.empty(M, Nn // 2 + Nn // 16, dtype=torch.uint8, device=x.device)
    else:
        q = out
        if q.dtype != torch.uint8 or tuple(q.shape) != (M, Nn // 2 + Nn // 16) or not q.is_contiguous() or q.device != x.device:
            raise ValueError("out must be a contiguous uint8 [M, N/2 + N/16] tensor on the device of x")
    acc = torch.empty(M, Nn, dtype=torch.float32, device=x.device) if want_acc else None
    with torch.cuda.device(x.device):
        N.check(N.cuda().fp4ar_gemm_nvfp4(None, 0, x.data_ptr(), wt.data_ptr(), M, Nn, K, C.c_float(gs), q.data_ptr(),
                                          acc.data_ptr() if acc is not None else None, _stream()), "fp4ar_gemm_nvfp4")
    return (q, acc) if want_acc else q


def gemm_push(ctx, x: torch.Tensor, wt: torch.Tensor, gs_self: float, *, two_shot: Optional[bool] = None,
              local_rank: int = 0, local_q: Optional[torch.Tensor] = None) -> None:
    """GEMM whose epilogue stores this rank's NVFP4 partial into the receive windows of `ctx` for its NEXT launch."""
    M, Nn, K = _check(x, wt)
    if Nn != N.HIDDEN:
        raise ValueError("the AllReduce windows are laid out for N = 6144")
    view = ctx.push_view(local_rank)
    if two_shot is None:
        two_shot = ctx.nranks > 2
    with torch.cuda.device(x.device):
        N.check(N.cuda().fp4ar_gemm_nvfp4(C.byref(view), 1 if two_shot else 0, x.data_ptr(), wt.data_ptr(), M, Nn, K,
                                          C.c_float(gs_self), local_q.data_ptr() if local_q is not None else None, None,
                                          _stream()), "fp4ar_gemm_nvfp4(push)")


def gemm_all_reduce_add_rms_norm(ctx, x: torch.Tensor, wt: torch.Tensor, gs: Sequence[float], residual: torch.Tensor,
                                 weight: torch.Tensor, *, eps: float = 1e-6, weight_bias: float = 1.0,
                                 epilogue: int = N.EPI_NORM_BF16, qscale: float = 1.0, out: Optional[torch.Tensor] = None):
    """x @ wt.T summed over the tensor-parallel group, + residual, Gemma RMSNorm: two kernels, no BF16 partial in
    memory.  `gs` holds every rank's static scale.  Returns (normed output, updated residual)."""
    from ..parallel.context import make_args

    M = x.shape[0]
    two_shot = ctx.nranks > 2
    gemm_push(ctx, x, wt, float(gs[ctx.rank]), two_shot=two_shot)
    o = q = None
    if epilogue == N.EPI_NORM_BF16:
        o = out if out is not None else torch.empty(M, N.HIDDEN, dtype=torch.bfloat16, device=x.device)
    else:
        nb = N.QROW_BYTES if epilogue == N.EPI_NORM_NVFP4 else N.MXROW_BYTES
        q = out if out is not None else torch.empty(M, nb, dtype=torch.uint8, device=x.device)
    ctx.launch(make_args(x=None, out=o, rows=M, input=N.IN_PUSHED, gs=list(gs), epilogue=epilogue, res_in=residual,
                         res_out=residual, weight=weight, eps=eps, weight_bias=weight_bias, outq=q, qscale=qscale,
                         algo=N.ALGO_TWOSHOT if two_shot else N.ALGO_ONESHOT))
    return (o if o is not None else q), residual


def gemm_status() -> N.StatusWords:
    w = N.StatusWords()
    N.check(N.cuda().fp4ar_gemm_status(C.byref(w)), "fp4ar_gemm_status")
    return w


def gemm_reset() -> None:
    """After a GEMM whose status is not 0: synchronise, clear the status block and the hand-off flags of the partial
    tiles, so that later launches do not wait on what the failed one left behind."""
    N.check(N.cuda().fp4ar_gemm_reset(), "fp4ar_gemm_reset")


def gemm_plan(M: int, Nn: int, K: int, sms: int = 148, unit: Optional[int] = None):
    """The schedule a GEMM of this size takes on a device with `sms` SMs (host only): a dict with `pair`, `tile_n`,
    `stream_k`, `units`, `tiles`, and with `unit` given also `segments`: the work list of that unit as
    (tile, first K block, K blocks, kind) tuples; kind 0 whole tile, 1 leaves a partial, 2 adds the next unit's."""
    vals = [C.c_int() for _ in range(5)]
    lib = N.cuda()
    rc = lib.fp4ar_gemm_plan(M, Nn, K, sms, *[C.byref(v) for v in vals], 0, None, 0)
    if rc < 0:
        raise ValueError("unsupported GEMM shape")
    out = dict(zip(("pair", "tile_n", "stream_k", "units", "tiles"), (v.value for v in vals)))
    if unit is not None:
        cap = 64
        while True:
            buf = (C.c_int * (4 * cap))()
            n = lib.fp4ar_gemm_plan(M, Nn, K, sms, *[C.byref(v) for v in vals], unit, buf, cap)
            if n < 0:
                raise ValueError("unit out of range")
            if n <= cap:
                break
            cap = n
        out["segments"] = [tuple(buf[4 * i:4 * i + 4]) for i in range(n)]
    return out
