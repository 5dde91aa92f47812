"""numpy / torch front end of the host bit-exact model (csrc/oracle/oracle.cpp).

Every GPU result in this package is gated against these functions.  BF16 data is passed as
`uint16` bit patterns (numpy has no bfloat16); `bf16_bits()` / `from_bf16_bits()` convert torch tensors.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native as N

H = N.HIDDEN


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def bf16_bits(t) -> np.ndarray:
    """torch.bfloat16 tensor -> uint16 numpy array of its bit patterns."""
    import torch

    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def from_bf16_bits(a: np.ndarray):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    N.oracle().fp4ar_oracle_f32_to_bf16(_p(x), _p(out), x.size)
    return out


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    N.oracle().fp4ar_oracle_e4m3_encode_n(_p(x), _p(out), x.size)
    return out


def e2m1_encode(x: np.ndarray) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint8)
    N.oracle().fp4ar_oracle_e2m1_encode_n(_p(x), _p(out), x.size)
    return out


def e4m3_table() -> np.ndarray:
    o = N.oracle()
    return np.array([o.fp4ar_oracle_e4m3_decode(b) for b in range(256)], np.float32)


def e2m1_table() -> np.ndarray:
    o = N.oracle()
    return np.array([o.fp4ar_oracle_e2m1_decode(b) for b in range(16)], np.float32)


def canon_neg0(words: np.ndarray) -> np.ndarray:
    w = _c(words, np.uint32)
    out = np.empty_like(w)
    N.oracle().fp4ar_oracle_canon_neg0(_p(w), _p(out), w.size)
    return out


def encode(x_bits: np.ndarray, canon: bool = True):
    """[rows, 6144] BF16 bits -> (values [rows,3072] u8, scales [rows,384] u8, row_scale [rows] f32)."""
    x = _c(x_bits, np.uint16).reshape(-1, H)
    rows = x.shape[0]
    v = np.empty((rows, N.VALUE_BYTES), np.uint8)
    s = np.empty((rows, N.SCALE_BYTES), np.uint8)
    rs = np.empty(rows, np.float32)
    N.oracle().fp4ar_oracle_encode(_p(x), rows, _p(v), N.VALUE_BYTES, _p(s), N.SCALE_BYTES, _p(rs), int(canon))
    return v, s, rs


def encode_f32(x: np.ndarray, canon: bool = True):
    x = _c(x, np.float32).reshape(-1, H)
    rows = x.shape[0]
    v = np.empty((rows, N.VALUE_BYTES), np.uint8)
    s = np.empty((rows, N.SCALE_BYTES), np.uint8)
    rs = np.empty(rows, np.float32)
    N.oracle().fp4ar_oracle_encode_f32(_p(x), rows, _p(v), N.VALUE_BYTES, _p(s), N.SCALE_BYTES, _p(rs), int(canon))
    return v, s, rs


def encode_static(x_bits: np.ndarray, gs: float) -> np.ndarray:
    """[rows, 6144] BF16 bits -> NVFP4 rows [rows, 3456] (values then scales), static scale gs."""
    x = _c(x_bits, np.uint16).reshape(-1, H)
    rows = x.shape[0]
    q = np.empty((rows, N.QROW_BYTES), np.uint8)
    base = q.ctypes.data
    N.oracle().fp4ar_oracle_encode_static(_p(x), rows, C.c_float(gs), C.c_void_p(base), N.QROW_BYTES,
                                          C.c_void_p(base + N.VALUE_BYTES), N.QROW_BYTES)
    return q


def encode_static_f32(x: np.ndarray, gs: float) -> np.ndarray:
    """[rows, cols] FP32 -> NVFP4 rows [rows, cols/2 + cols/16] with the static scale gs (the GEMM epilogue's quantiser)."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols // 2 + cols // 16), np.uint8)
    base = q.ctypes.data
    N.oracle().fp4ar_oracle_encode_static_f32(_p(x), rows, cols, C.c_float(gs), C.c_void_p(base), q.shape[1],
                                              C.c_void_p(base + cols // 2), q.shape[1])
    return q


def decode_acc(acc: np.ndarray, v: np.ndarray, s: np.ndarray, rs) -> np.ndarray:
    """acc [rows,6144] f32 += decode(v, s, rs); rs is an array of row scales or one static scale."""
    assert acc.dtype == np.float32 and acc.flags.c_contiguous
    rows = acc.shape[0]
    v = _c(v, np.uint8); s = _c(s, np.uint8)
    if np.isscalar(rs):
        N.oracle().fp4ar_oracle_decode_acc(_p(acc), rows, _p(v), v.shape[1], _p(s), s.shape[1], None, C.c_float(rs))
    else:
        r = _c(rs, np.float32)
        N.oracle().fp4ar_oracle_decode_acc(_p(acc), rows, _p(v), v.shape[1], _p(s), s.shape[1], _p(r), C.c_float(0))
    return acc


def row_sumsq(z: np.ndarray) -> float:
    z = _c(z, np.float32)
    assert z.size == H
    return float(N.oracle().fp4ar_oracle_row_sumsq(_p(z)))


def allreduce(xs, *, algo: int = 0, input_kind: int = 0, gs=None, epi: int = 0, res_in=None, weight=None,
              eps: float = 1e-6, wbias: float = 1.0, qscale: float = 1.0, want_sum: bool = False) -> dict:
    """Bit-exact model of the fused operator.

    xs: list of per-rank inputs, BF16 bits [rows,6144] (input_kind 0) or NVFP4 rows [rows,3456] u8 (1).
    Returns a dict with the keys that the epilogue produces: out, res_out, outq, sum.
    """
    P = len(xs)
    if input_kind == 0:
        arrs = [_c(x, np.uint16).reshape(-1, H) for x in xs]
    else:
        arrs = [_c(x, np.uint8).reshape(-1, N.QROW_BYTES) for x in xs]
    rows = arrs[0].shape[0]
    ptrs = (C.c_void_p * P)(*[a.ctypes.data for a in arrs])
    gsa = _c(gs if gs is not None else np.ones(P), np.float32)
    out = np.zeros((rows, H), np.uint16) if epi <= 1 else None
    res_out = np.zeros((rows, H), np.uint16) if epi > 0 else None
    outq = None
    if epi == 2:
        outq = np.zeros((rows, N.QROW_BYTES), np.uint8)
    elif epi == 3:
        outq = np.zeros((rows, N.MXROW_BYTES), np.uint8)
    r_in = _c(res_in, np.uint16) if epi > 0 else None
    w = _c(weight, np.uint16) if epi > 0 else None
    sm = np.zeros((rows, H), np.float32) if want_sum else None
    rc = N.oracle().fp4ar_oracle_allreduce(
        P, rows, algo, input_kind, ptrs, _p(gsa), epi,
        _p(r_in) if r_in is not None else None, _p(w) if w is not None else None,
        C.c_float(eps), C.c_float(wbias), C.c_float(qscale),
        _p(out) if out is not None else None, _p(res_out) if res_out is not None else None,
        _p(outq) if outq is not None else None, _p(sm) if sm is not None else None)
    if rc != 0:
        raise ValueError(f"oracle rejected the arguments (code {rc})")
    return {"out": out, "res_out": res_out, "outq": outq, "sum": sm}


def add_rmsnorm(x_bits, res_in, weight, *, eps=1e-6, wbias=1.0, epi=1, qscale=1.0) -> dict:
    x = _c(x_bits, np.uint16).reshape(-1, H)
    rows = x.shape[0]
    r = _c(res_in, np.uint16); w = _c(weight, np.uint16)
    out = np.zeros((rows, H), np.uint16) if epi == 1 else None
    res_out = np.zeros((rows, H), np.uint16)
    outq = np.zeros((rows, N.QROW_BYTES if epi == 2 else N.MXROW_BYTES), np.uint8) if epi >= 2 else None
    rc = N.oracle().fp4ar_oracle_add_rmsnorm(rows, _p(x), _p(r), _p(w), C.c_float(eps), C.c_float(wbias), epi,
                                             C.c_float(qscale), _p(out) if out is not None else None, _p(res_out),
                                             _p(outq) if outq is not None else None)
    if rc != 0:
        raise ValueError(f"oracle rejected the arguments (code {rc})")
    return {"out": out, "res_out": res_out, "outq": outq}
