"""Stand-alone codec and norm ops on CUDA tensors (hand-written sm_100a kernels, csrc/kernels/codec_ops.cu).

These are the building blocks of the fused AllReduce exposed one by one, the way the reference project
exposes them as benchmark kernels (bench/codec/codec_bench.cu:139-590).  All functions launch on the
current CUDA stream and never fall back to PyTorch: a missing library or a non-CUDA tensor is an error.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .. import _native as N


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _req_layout(t: torch.Tensor, dtype, cols: int | None, name: str) -> torch.Tensor:
    """dtype, shape [rows, cols] and contiguity; the device is the caller's business."""
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if cols is not None and (t.dim() != 2 or t.shape[1] != cols):
        raise ValueError(f"{name} must have shape [rows, {cols}], got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _req(t: torch.Tensor, dtype, cols: int | None, name: str) -> torch.Tensor:
    _req_layout(t, dtype, cols, name)
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    return t


def encode(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 [rows, 6144] -> (NVFP4 rows [rows, 3456] uint8: 3072 value bytes then 384 scale bytes,
    FP32 row scales [rows])."""
    _req(x, torch.bfloat16, N.HIDDEN, "x")
    rows = x.shape[0]
    q = torch.empty(rows, N.QROW_BYTES, dtype=torch.uint8, device=x.device)
    rs = torch.empty(rows, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.cuda().fp4ar_encode(x.data_ptr(), rows, q.data_ptr(), N.QROW_BYTES, q.data_ptr() + N.VALUE_BYTES,
                                      N.QROW_BYTES, rs.data_ptr(), _stream()), "fp4ar_encode")
    return q, rs


def encode_static(x: torch.Tensor, gs: float) -> torch.Tensor:
    """BF16 [rows, 6144] -> NVFP4 rows [rows, 3456] with the static per-tensor scale gs (no row scale)."""
    _req(x, torch.bfloat16, N.HIDDEN, "x")
    rows = x.shape[0]
    q = torch.empty(rows, N.QROW_BYTES, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        N.check(N.cuda().fp4ar_encode_static(x.data_ptr(), rows, C.c_float(gs), q.data_ptr(), _stream()),
                "fp4ar_encode_static")
    return q


def _sources(qrows: Sequence[torch.Tensor], row_scales, gs):
    n = len(qrows)
    if not 1 <= n <= N.MAX_RANKS:
        raise ValueError("1..8 sources")
    pitch = qrows[0].shape[1]
    for q in qrows:
        _req(q, torch.uint8, pitch, "source")
        if q.shape != qrows[0].shape:
            raise ValueError("sources must have one shape")
    if pitch not in (N.QROW_BYTES, N.REC_STRIDE):
        raise ValueError("source rows must be 3456 B (NVFP4 rows) or 3584 B (receive records)")
    src = (C.c_void_p * n)(*[q.data_ptr() for q in qrows])
    rsp = (C.c_void_p * n)()
    gsa = (C.c_float * N.MAX_RANKS)()
    for i in range(n):
        r = row_scales[i] if row_scales is not None else None
        if r is not None:
            _req(r, torch.float32, None, "row_scales")
            rsp[i] = r.data_ptr()
        else:
            if gs is None:
                raise ValueError("a source without row scales needs a static scale")
            rsp[i] = None
            gsa[i] = float(gs[i])
    return n, src, pitch, rsp, gsa


def decode_sum(qrows: Sequence[torch.Tensor], row_scales=None, gs=None) -> torch.Tensor:
    """FP32 decode-accumulate of the sources in list order, BF16 [rows, 6144] out."""
    n, src, pitch, rsp, gsa = _sources(qrows, row_scales, gs)
    rows = qrows[0].shape[0]
    out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=qrows[0].device)
    with torch.cuda.device(out.device):
        N.check(N.cuda().fp4ar_decode_sum(n, src, pitch, rsp, gsa, rows, out.data_ptr(), _stream()), "fp4ar_decode_sum")
    return out


def reduce_reencode(qrows: Sequence[torch.Tensor], row_scales=None, gs=None) -> tuple[torch.Tensor, torch.Tensor]:
    """The two-shot owner step: decode-sum, re-encode the FP32 sum with its own row scale, and output the
    decode of that re-encoding.  Returns (records [rows, 3584] uint8, BF16 [rows, 6144])."""
    n, src, pitch, rsp, gsa = _sources(qrows, row_scales, gs)
    rows = qrows[0].shape[0]
    dev = qrows[0].device
    rec = torch.zeros(rows, N.REC_STRIDE, dtype=torch.uint8, device=dev)
    out = torch.empty(rows, N.HIDDEN, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        N.check(N.cuda().fp4ar_reduce_reencode(n, src, pitch, rsp, gsa, rows, rec.data_ptr(), out.data_ptr(), _stream()),
                "fp4ar_reduce_reencode")
    return rec, out


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                weight_bias: float = 1.0, epilogue: int = N.EPI_NORM_BF16, qscale: float = 1.0,
                inplace_residual: bool = False, out: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """z = x + residual; residual' = bf16(z); y = (bf16(z) * rinv) * (weight_bias + weight).
    Returns (y as BF16 [rows,6144] | NVFP4 rows [rows,3456] | MXFP8 rows [rows,6336], residual')."""
    _req(x, torch.bfloat16, N.HIDDEN, "x")
    _req(residual, torch.bfloat16, N.HIDDEN, "residual")
    if weight.dtype != torch.bfloat16 or weight.numel() != N.HIDDEN or not weight.is_cuda:
        raise ValueError("weight must be a CUDA BF16 tensor of 6144 elements")
    rows = x.shape[0]
    res_out = residual if inplace_residual else torch.empty_like(residual)
    given, out, outq = out, None, None
    if epilogue == N.EPI_NORM_BF16:
        out = given if given is not None else torch.empty_like(x)
    elif epilogue == N.EPI_NORM_NVFP4:
        outq = given if given is not None else torch.empty(rows, N.QROW_BYTES, dtype=torch.uint8, device=x.device)
    elif epilogue == N.EPI_NORM_MXFP8:
        outq = given if given is not None else torch.empty(rows, N.MXROW_BYTES, dtype=torch.uint8, device=x.device)
    else:
        raise ValueError("epilogue must be 1 (BF16), 2 (NVFP4) or 3 (MXFP8)")
    with torch.cuda.device(x.device):
        N.check(N.cuda().fp4ar_add_rmsnorm(x.data_ptr(), residual.data_ptr(), res_out.data_ptr(), weight.data_ptr(),
                                           C.c_float(eps), C.c_float(weight_bias), epilogue, C.c_float(qscale),
                                           out.data_ptr() if out is not None else None,
                                           outq.data_ptr() if outq is not None else None, rows, _stream()),
                "fp4ar_add_rmsnorm")
    return (out if out is not None else outq), res_out


def fill_sentinel(window: torch.Tensor, buffer_bytes: int, nbuffers: int = 2) -> None:
    """Overwrite a receive window with the not-yet-written patterns (0x88 values, 0xFF scales, -0.0 row scale)."""
    if window.dtype != torch.uint8 or not window.is_cuda or window.numel() < buffer_bytes * nbuffers:
        raise ValueError("window must be a CUDA uint8 tensor of at least buffer_bytes * nbuffers")
    with torch.cuda.device(window.device):
        N.check(N.cuda().fp4ar_fill_sentinel(window.data_ptr(), buffer_bytes, nbuffers, _stream()), "fp4ar_fill_sentinel")
