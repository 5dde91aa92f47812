"""CPU tests of the op surface: schemas, fake (meta) implementations, argument validation, window sizes."""
import ctypes as C

import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200.ops import allreduce as A  # noqa: F401  (registers torch.ops.fp4ar)


def test_fake_impls_give_shapes_without_a_gpu():
    with torch._subclasses.FakeTensorMode():
        x = torch.empty(37, 6144, dtype=torch.bfloat16)
        res = torch.empty(37, 6144, dtype=torch.bfloat16)
        w = torch.empty(6144, dtype=torch.bfloat16)
        xq = torch.empty(37, 3456, dtype=torch.uint8)
        assert torch.ops.fp4ar.all_reduce(x, 1).shape == (37, 6144)
        assert torch.ops.fp4ar.all_reduce_nvfp4(xq, [1.0, 2.0], 1).dtype == torch.bfloat16
        assert torch.ops.fp4ar.all_reduce_add_rms_norm(x, res, w, 1e-6, 1.0, 1).shape == (37, 6144)
        assert torch.ops.fp4ar.all_reduce_add_rms_norm_nvfp4(xq, [1.0, 2.0], res, w, 1e-6, 1.0, 1).shape == (37, 6144)
        assert torch.ops.fp4ar.all_reduce_add_rms_norm_quant(x, res, w, 1e-6, 1.0, 2, 1.0, 1).shape == (37, 3456)
        assert torch.ops.fp4ar.all_reduce_add_rms_norm_quant(x, res, w, 1e-6, 1.0, 3, 1.0, 1).shape == (37, 6336)
        q, rs = torch.ops.fp4ar.encode(x)
        assert q.shape == (37, 3456) and rs.shape == (37,)
        assert torch.ops.fp4ar.decode_sum([q, q], [rs, rs]).shape == (37, 6144)
        xk = torch.empty(37, 2048, dtype=torch.bfloat16)
        wt = torch.empty(6144, 2048, dtype=torch.bfloat16)
        assert torch.ops.fp4ar.linear_nvfp4(xk, wt, 0.5).shape == (37, 3456)
        y = torch.ops.fp4ar.linear_all_reduce_add_rms_norm(xk, wt, [0.5, 0.5], res, w, 1e-6, 1.0, 1)
        assert y.shape == (37, 6144) and y.dtype == torch.bfloat16


def test_unknown_context_id_is_an_error():
    with pytest.raises(RuntimeError):
        A._ctx(987654)


def test_window_bytes_and_argument_validation_without_a_gpu(cuda_lib):
    lib = cuda_lib
    assert lib.fp4ar_window_bytes(16384, 6144, 2) == 2 * 2 * 16384 * 3584   # 2 buffers x 2 sources x rows x slot
    assert lib.fp4ar_window_bytes(16384, 6144, 8) % (2 << 20) == 0
    assert lib.fp4ar_window_bytes(16384, 4096, 2) == 0      # only hidden 6144
    assert lib.fp4ar_window_bytes(16384, 6144, 3) == 0      # 1, 2, 4, 8 ranks
    assert lib.fp4ar_window_bytes(0, 6144, 2) == 0
    # a window that is too small or a null pointer is rejected before any CUDA call
    ctx = C.c_void_p()
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    assert lib.fp4ar_create(C.byref(ctx), 0, 2, 0, 1024, 6144, ptrs, 4096) == 1
    ptrs = (C.c_void_p * 2)(None, None)
    assert lib.fp4ar_create(C.byref(ctx), 0, 2, 0, 1024, 6144, ptrs, 1 << 30) == 1
    assert lib.fp4ar_launch(None, None, None) == 1
    assert b"sm_100a" in lib.fp4ar_build_info()


def test_kernel_table_holds_every_product_shape(cuda_lib):
    """Host-side check of the compiled-shape table (no GPU): three-warp teams for every shape, six-warp teams for the
    two-shot shapes of four and eight ranks (their default), nothing else."""
    lib = cuda_lib
    has = lambda *a: int(lib.fp4ar_has_kernel(*a))
    for P, algos in ((1, (0,)), (2, (0, 1)), (4, (0, 1)), (8, (0, 1))):
        for algo in algos:
            assert has(P, algo, 0, 0, 3) > 0, (P, algo)
    for P in (2, 4, 8):
        algo = 0 if P == 2 else 1
        for inp in (0, 1, 2):
            for epi in (0, 1, 2, 3):
                assert has(P, algo, inp, epi, 3) > 0, (P, algo, inp, epi)
                assert has(P, algo, inp, epi, 6) == (3 if P >= 4 else 0), (P, algo, inp, epi)
                assert has(P, algo, inp, epi, 2) == 0
    assert has(4, 0, 0, 0, 6) == 0 and has(1, 0, 0, 1, 6) == 0
    assert lib.fp4ar_default_team_warps(8, 1) == 6 and lib.fp4ar_default_team_warps(2, 0) == 3


def _unbound_context(nranks=2, max_rows=64):
    """A context object with only the fields the argument checks read (no GPU, no native context)."""
    from fp4_all_reduce_b200.parallel.context import Fp4ArContext

    ctx = Fp4ArContext.__new__(Fp4ArContext)
    ctx.nranks, ctx.max_rows, ctx.device, ctx._ctx = nranks, max_rows, torch.device("cuda", 0), None
    return ctx


def test_all_reduce_wrappers_reject_bad_tensors_before_any_launch():
    """Wrong dtype, width, strides, row count, scales or device never reach the kernel, which trusts its pointers."""
    ctx = _unbound_context()
    good = torch.zeros(8, 6144, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="bfloat16"):
        ctx.all_reduce(good.float())
    with pytest.raises(ValueError, match="shape"):
        ctx.all_reduce(torch.zeros(8, 4096, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="contiguous"):
        ctx.all_reduce(torch.zeros(8, 2 * 6144, dtype=torch.bfloat16)[:, ::2])
    with pytest.raises(ValueError, match="is on cpu"):
        ctx.all_reduce(good)                                        # a host tensor, context on cuda:0
    with pytest.raises(ValueError, match="shape"):
        ctx.all_reduce(torch.zeros(8, 3000, dtype=torch.uint8), gs=[1.0, 1.0])
    xq = torch.zeros(8, 3456, dtype=torch.uint8)
    with pytest.raises(ValueError, match="gs"):
        ctx.all_reduce(xq)                                          # NVFP4 rows without scales
    with pytest.raises(ValueError, match="gs"):
        ctx.all_reduce(xq, gs=[1.0])                                # one scale per rank
    with pytest.raises(ValueError, match="gs"):
        ctx.all_reduce(xq, gs=[1.0, 0.0])
    with pytest.raises(ValueError, match="max_rows"):
        ctx.all_reduce(torch.zeros(65, 6144, dtype=torch.bfloat16))


def test_companion_tensors_of_the_norm_call_are_checked():
    ctx = _unbound_context()
    ctx.device = torch.device("cpu")            # host tensors pass the device test, so every later check is reached
    x = torch.zeros(8, 6144, dtype=torch.bfloat16)
    res = torch.zeros(8, 6144, dtype=torch.bfloat16)
    w = torch.zeros(6144, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="epilogue"):
        ctx.all_reduce_add_rms_norm(x, res, w, epilogue=7)
    with pytest.raises(ValueError, match="residual must have 8 rows"):
        ctx.all_reduce_add_rms_norm(x, res[:7], w)
    with pytest.raises(ValueError, match="residual_out"):
        ctx.all_reduce_add_rms_norm(x, res, w, residual_out=torch.zeros(8, 6000, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="weight"):
        ctx.all_reduce_add_rms_norm(x, res, w[:100])
    with pytest.raises(ValueError, match="weight"):
        ctx.all_reduce_add_rms_norm(x, res, w.float())
    with pytest.raises(ValueError, match="out must be"):
        ctx.all_reduce_add_rms_norm(x, res, w, epilogue=2, out=torch.zeros(8, 3456, dtype=torch.int8))
    with pytest.raises(ValueError, match="out must have shape"):
        ctx.all_reduce_add_rms_norm(x, res, w, epilogue=3, out=torch.zeros(8, 3456, dtype=torch.uint8))
    with pytest.raises(ValueError, match="out must have 8 rows"):
        ctx.all_reduce(x, out=torch.zeros(9, 6144, dtype=torch.bfloat16))


def test_zero_row_call_and_poisoned_code_have_names():
    assert N.ERROR_NAMES[4] == "context poisoned"
    with pytest.raises(N.ContextPoisoned):
        N.check(4, "fp4ar_launch")
