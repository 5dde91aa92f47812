"""PyTorch custom ops (`torch.ops.fp4ar.*`) over the fused AllReduce contexts.

The ops take the id of a registered context instead of the context object so that they are plain
functions of tensors and scalars: traceable by `torch.compile` / export through their fake
implementations, and recordable in CUDA graphs (a launch has no host-side per-call state).

    ctx_id = register_context(Fp4ArContext(max_rows, group))
    y = torch.ops.fp4ar.all_reduce(x, ctx_id)
    y = torch.ops.fp4ar.all_reduce_add_rms_norm(x, residual, weight, 1e-6, 1.0, ctx_id)     # residual updated in place
    yq = torch.ops.fp4ar.all_reduce_add_rms_norm_quant(x, residual, weight, 1e-6, 1.0, 2, qscale, ctx_id)
    y = torch.ops.fp4ar.all_reduce_nvfp4(xq, gs, ctx_id)                                   # producer already emitted NVFP4
    y = torch.ops.fp4ar.all_reduce_add_rms_norm_nvfp4(xq, gs, residual, weight, 1e-6, 1.0, ctx_id)
    y = torch.ops.fp4ar.linear_all_reduce_add_rms_norm(x, wt, gs, residual, weight, 1e-6, 1.0, ctx_id)   # row-parallel linear:
                                                           # tcgen05 GEMM pushing NVFP4 partials into the peers + AllReduce + norm

This is the op surface the reference project only plans (docs/INTEGRATION.md:18-23).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import _native as N
from . import codec as _codec

_CONTEXTS: Dict[int, object] = {}
_NEXT_ID = [1]


def register_context(ctx) -> int:
    cid = _NEXT_ID[0]
    _NEXT_ID[0] += 1
    _CONTEXTS[cid] = ctx
    return cid


def unregister_context(cid: int) -> None:
    _CONTEXTS.pop(cid, None)


def _ctx(cid: int):
    try:
        return _CONTEXTS[cid]
    except KeyError:
        raise RuntimeError(f"fp4ar: no context registered under id {cid}") from None


_lib = torch.library.Library("fp4ar", "DEF")
_lib.define("all_reduce(Tensor x, int ctx) -> Tensor")
_lib.define("all_reduce_nvfp4(Tensor xq, float[] gs, int ctx) -> Tensor")
_lib.define("all_reduce_add_rms_norm(Tensor x, Tensor(a!) residual, Tensor weight, float eps, float weight_bias, int ctx) -> Tensor")
_lib.define("all_reduce_add_rms_norm_nvfp4(Tensor xq, float[] gs, Tensor(a!) residual, Tensor weight, float eps, float weight_bias, int ctx) -> Tensor")
_lib.define("all_reduce_add_rms_norm_quant(Tensor x, Tensor(a!) residual, Tensor weight, float eps, float weight_bias, int out_kind, float qscale, int ctx) -> Tensor")
_lib.define("encode(Tensor x) -> (Tensor, Tensor)")
_lib.define("encode_static(Tensor x, float gs) -> Tensor")
_lib.define("decode_sum(Tensor[] qrows, Tensor[] row_scales) -> Tensor")
_lib.define("add_rms_norm(Tensor x, Tensor(a!) residual, Tensor weight, float eps, float weight_bias) -> Tensor")
_lib.define("linear_nvfp4(Tensor x, Tensor wt, float gs) -> Tensor")
_lib.define("linear_all_reduce_add_rms_norm(Tensor x, Tensor wt, float[] gs, Tensor(a!) residual, Tensor weight, float eps, "
            "float weight_bias, int ctx) -> Tensor")


def _all_reduce(x, ctx):
    return _ctx(ctx).all_reduce(x)


def _all_reduce_nvfp4(xq, gs, ctx):
    return _ctx(ctx).all_reduce(xq, gs=list(gs))


def _ar_norm(x, residual, weight, eps, weight_bias, ctx):
    y, _ = _ctx(ctx).all_reduce_add_rms_norm(x, residual, weight, eps=eps, weight_bias=weight_bias)
    return y


def _ar_norm_nvfp4(xq, gs, residual, weight, eps, weight_bias, ctx):
    y, _ = _ctx(ctx).all_reduce_add_rms_norm(xq, residual, weight, eps=eps, weight_bias=weight_bias, gs=list(gs))
    return y


def _ar_norm_quant(x, residual, weight, eps, weight_bias, out_kind, qscale, ctx):
    if out_kind not in (N.EPI_NORM_NVFP4, N.EPI_NORM_MXFP8):
        raise ValueError("out_kind must be 2 (NVFP4) or 3 (MXFP8)")
    y, _ = _ctx(ctx).all_reduce_add_rms_norm(x, residual, weight, eps=eps, weight_bias=weight_bias, epilogue=out_kind,
                                             qscale=qscale)
    return y


def _add_rms_norm(x, residual, weight, eps, weight_bias):
    y, _ = _codec.add_rmsnorm(x, residual, weight, eps, weight_bias, N.EPI_NORM_BF16, 1.0, inplace_residual=True)
    return y


def _linear_nvfp4(x, wt, gs):
    from . import gemm as _gemm

    return _gemm.gemm_nvfp4(x, wt, gs)


def _linear_ar_norm(x, wt, gs, residual, weight, eps, weight_bias, ctx):
    from . import gemm as _gemm

    y, _ = _gemm.gemm_all_reduce_add_rms_norm(_ctx(ctx), x, wt, list(gs), residual, weight, eps=eps, weight_bias=weight_bias)
    return y


_lib.impl("all_reduce", _all_reduce, "CUDA")
_lib.impl("all_reduce_nvfp4", _all_reduce_nvfp4, "CUDA")
_lib.impl("all_reduce_add_rms_norm", _ar_norm, "CUDA")
_lib.impl("all_reduce_add_rms_norm_nvfp4", _ar_norm_nvfp4, "CUDA")
_lib.impl("all_reduce_add_rms_norm_quant", _ar_norm_quant, "CUDA")
_lib.impl("encode", lambda x: _codec.encode(x), "CUDA")
_lib.impl("encode_static", lambda x, gs: _codec.encode_static(x, gs), "CUDA")
_lib.impl("decode_sum", lambda q, r: _codec.decode_sum(list(q), list(r)), "CUDA")
_lib.impl("add_rms_norm", _add_rms_norm, "CUDA")
_lib.impl("linear_nvfp4", _linear_nvfp4, "CUDA")
_lib.impl("linear_all_reduce_add_rms_norm", _linear_ar_norm, "CUDA")


def _bf16_rows(t):
    return t.new_empty((t.shape[0], N.HIDDEN), dtype=torch.bfloat16)


@torch.library.register_fake("fp4ar::all_reduce")
def _(x, ctx):
    return _bf16_rows(x)


@torch.library.register_fake("fp4ar::all_reduce_nvfp4")
def _(xq, gs, ctx):
    return _bf16_rows(xq)


@torch.library.register_fake("fp4ar::all_reduce_add_rms_norm")
def _(x, residual, weight, eps, weight_bias, ctx):
    return _bf16_rows(x)


@torch.library.register_fake("fp4ar::all_reduce_add_rms_norm_nvfp4")
def _(xq, gs, residual, weight, eps, weight_bias, ctx):
    return _bf16_rows(xq)


@torch.library.register_fake("fp4ar::all_reduce_add_rms_norm_quant")
def _(x, residual, weight, eps, weight_bias, out_kind, qscale, ctx):
    nb = N.QROW_BYTES if out_kind == N.EPI_NORM_NVFP4 else N.MXROW_BYTES
    return x.new_empty((x.shape[0], nb), dtype=torch.uint8)


@torch.library.register_fake("fp4ar::encode")
def _(x):
    return (x.new_empty((x.shape[0], N.QROW_BYTES), dtype=torch.uint8), x.new_empty((x.shape[0],), dtype=torch.float32))


@torch.library.register_fake("fp4ar::encode_static")
def _(x, gs):
    return x.new_empty((x.shape[0], N.QROW_BYTES), dtype=torch.uint8)


@torch.library.register_fake("fp4ar::decode_sum")
def _(qrows, row_scales):
    return _bf16_rows(qrows[0])


@torch.library.register_fake("fp4ar::linear_nvfp4")
def _(x, wt, gs):
    n = wt.shape[0]
    return x.new_empty((x.shape[0], n // 2 + n // 16), dtype=torch.uint8)


@torch.library.register_fake("fp4ar::linear_all_reduce_add_rms_norm")
def _(x, wt, gs, residual, weight, eps, weight_bias, ctx):
    return x.new_empty((x.shape[0], wt.shape[0]), dtype=torch.bfloat16)


@torch.library.register_fake("fp4ar::add_rms_norm")
def _(x, residual, weight, eps, weight_bias):
    return torch.empty_like(x)
