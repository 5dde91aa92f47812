"""ctypes bindings of the two native libraries.

`oracle()` returns the host-only bit-exact model (always available: it is plain C++ and is built on
first use).  `cuda()` returns the CUDA library; it is built in-tree by `python -m
fp4_all_reduce_b200.build` and must exist on a GPU machine: the GPU ops raise instead of silently
falling back to PyTorch when it is missing.
"""
from __future__ import annotations

import ctypes as C
import functools
from pathlib import Path

from . import build as _build

_LIB = Path(__file__).resolve().parent / "lib"

MAX_RANKS = 8
HIDDEN = 6144
VALUE_BYTES = 3072
SCALE_BYTES = 384
QROW_BYTES = 3456
MXROW_BYTES = 6336
REC_STRIDE = 3584
REC_PAYLOAD = 3472

MODE_FUSED, MODE_XPORT, MODE_COMPUTE = 0, 1, 2
ALGO_AUTO, ALGO_ONESHOT, ALGO_TWOSHOT = -1, 0, 1
IN_BF16, IN_NVFP4, IN_PUSHED = 0, 1, 2
EPI_NONE, EPI_NORM_BF16, EPI_NORM_NVFP4, EPI_NORM_MXFP8 = 0, 1, 2, 3

ERROR_NAMES = {0: "ok", 1: "bad argument", 2: "unsupported combination", 3: "CUDA error", 4: "context poisoned"}


class Args(C.Structure):
    """Mirror of `fp4ar_args` (csrc/include/fp4ar.h)."""

    _fields_ = [
        ("x", C.c_void_p), ("out", C.c_void_p),
        ("rows", C.c_int), ("hidden", C.c_int), ("mode", C.c_int), ("algo", C.c_int),
        ("input", C.c_int), ("epilogue", C.c_int),
        ("gs", C.c_float * MAX_RANKS),
        ("res_in", C.c_void_p), ("res_out", C.c_void_p), ("weight", C.c_void_p),
        ("eps", C.c_float), ("weight_bias", C.c_float),
        ("outq", C.c_void_p), ("qscale", C.c_float),
        ("tune", C.c_int * 4),
    ]


class StatusWords(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("code", "row", "source", "detail", "cta", "call", "count", "pad")]


class PushView(C.Structure):
    _fields_ = [
        ("call_counter", C.c_void_p), ("buffer_bytes", C.c_size_t), ("cap", C.c_int), ("capo", C.c_int),
        ("nranks", C.c_int), ("rank", C.c_int), ("windows", C.c_void_p * MAX_RANKS),
    ]


@functools.lru_cache(maxsize=None)
def oracle() -> C.CDLL:
    path = _build.build_oracle()
    lib = C.CDLL(str(path))
    u8p, u16p, f32p, vp = C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.POINTER(C.c_float), C.c_void_p
    lib.fp4ar_oracle_e4m3_encode.argtypes = [C.c_float]; lib.fp4ar_oracle_e4m3_encode.restype = C.c_uint8
    lib.fp4ar_oracle_e4m3_decode.argtypes = [C.c_uint8]; lib.fp4ar_oracle_e4m3_decode.restype = C.c_float
    lib.fp4ar_oracle_e2m1_encode.argtypes = [C.c_float]; lib.fp4ar_oracle_e2m1_encode.restype = C.c_uint8
    lib.fp4ar_oracle_e2m1_decode.argtypes = [C.c_uint8]; lib.fp4ar_oracle_e2m1_decode.restype = C.c_float
    lib.fp4ar_oracle_bf16_rn.argtypes = [C.c_float]; lib.fp4ar_oracle_bf16_rn.restype = C.c_uint16
    lib.fp4ar_oracle_e4m3_encode_n.argtypes = [vp, vp, C.c_long]
    lib.fp4ar_oracle_e2m1_encode_n.argtypes = [vp, vp, C.c_long]
    lib.fp4ar_oracle_encode.argtypes = [vp, C.c_int, vp, C.c_long, vp, C.c_long, vp, C.c_int]
    lib.fp4ar_oracle_encode_f32.argtypes = [vp, C.c_int, vp, C.c_long, vp, C.c_long, vp, C.c_int]
    lib.fp4ar_oracle_encode_static.argtypes = [vp, C.c_int, C.c_float, vp, C.c_long, vp, C.c_long]
    lib.fp4ar_oracle_encode_static_f32.argtypes = [vp, C.c_int, C.c_int, C.c_float, vp, C.c_long, vp, C.c_long]
    lib.fp4ar_oracle_decode_acc.argtypes = [vp, C.c_int, vp, C.c_long, vp, C.c_long, vp, C.c_float]
    lib.fp4ar_oracle_f32_to_bf16.argtypes = [vp, vp, C.c_long]
    lib.fp4ar_oracle_canon_neg0.argtypes = [vp, vp, C.c_long]
    lib.fp4ar_oracle_row_sumsq.argtypes = [vp]; lib.fp4ar_oracle_row_sumsq.restype = C.c_float
    lib.fp4ar_oracle_allreduce.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(vp), vp, C.c_int, vp, vp,
                                           C.c_float, C.c_float, C.c_float, vp, vp, vp, vp]
    lib.fp4ar_oracle_allreduce.restype = C.c_int
    lib.fp4ar_oracle_add_rmsnorm.argtypes = [C.c_int, vp, vp, vp, C.c_float, C.c_float, C.c_int, C.c_float, vp, vp, vp]
    lib.fp4ar_oracle_add_rmsnorm.restype = C.c_int
    del u8p, u16p, f32p
    return lib


def cuda_library_path() -> Path:
    """In-tree library, or the file named by FP4AR_LIBRARY (for tuning builds with extra counters)."""
    import os

    override = os.environ.get("FP4AR_LIBRARY")
    return Path(override) if override else _LIB / "libfp4ar.so"


@functools.lru_cache(maxsize=None)
def cuda() -> C.CDLL:
    path = cuda_library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m fp4_all_reduce_b200.build` (needs nvcc; no GPU required)")
    lib = C.CDLL(str(path))
    vp, vpp = C.c_void_p, C.POINTER(C.c_void_p)
    lib.fp4ar_window_bytes.argtypes = [C.c_int, C.c_int, C.c_int]; lib.fp4ar_window_bytes.restype = C.c_size_t
    lib.fp4ar_create.argtypes = [vpp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vpp, C.c_size_t]
    lib.fp4ar_create_emulated.argtypes = [vpp, C.c_int, C.c_int, C.c_int, C.c_int, vpp, C.c_size_t]
    lib.fp4ar_launch.argtypes = [vp, C.POINTER(Args), vp]
    lib.fp4ar_status.argtypes = [vp, C.c_int, C.POINTER(StatusWords)]
    lib.fp4ar_set_timeout_ms.argtypes = [vp, C.c_int]
    lib.fp4ar_reset.argtypes = [vp]
    lib.fp4ar_destroy.argtypes = [vp]
    lib.fp4ar_get_push_view.argtypes = [vp, C.c_int, C.POINTER(PushView)]
    lib.fp4ar_ctas_per_rank.argtypes = [vp]
    lib.fp4ar_last_cuda_error.restype = C.c_char_p
    lib.fp4ar_build_info.restype = C.c_char_p
    lib.fp4ar_encode.argtypes = [vp, C.c_int, vp, C.c_long, vp, C.c_long, vp, vp]
    lib.fp4ar_encode_static.argtypes = [vp, C.c_int, C.c_float, vp, vp]
    lib.fp4ar_decode_sum.argtypes = [C.c_int, vpp, C.c_long, vpp, C.POINTER(C.c_float), C.c_int, vp, vp]
    lib.fp4ar_reduce_reencode.argtypes = [C.c_int, vpp, C.c_long, vpp, C.POINTER(C.c_float), C.c_int, vp, vp, vp]
    lib.fp4ar_add_rmsnorm.argtypes = [vp, vp, vp, vp, C.c_float, C.c_float, C.c_int, C.c_float, vp, vp, C.c_int, vp]
    lib.fp4ar_fill_sentinel.argtypes = [vp, C.c_size_t, C.c_int, vp]
    lib.fp4ar_selftest_scale_division.argtypes = [C.c_int, vp, vp]
    lib.fp4ar_selftest_scale_division.restype = C.c_int
    lib.fp4ar_selftest_conversions.argtypes = [C.c_int, C.c_uint, C.c_uint, vp, vp]
    lib.fp4ar_selftest_conversions.restype = C.c_int
    lib.fp4ar_gemm_nvfp4.argtypes = [C.POINTER(PushView), C.c_int, vp, vp, C.c_int, C.c_int, C.c_int, C.c_float, vp, vp, vp]
    lib.fp4ar_gemm_nvfp4.restype = C.c_int
    lib.fp4ar_gemm_status.argtypes = [C.POINTER(StatusWords)]
    lib.fp4ar_gemm_status.restype = C.c_int
    ip = C.POINTER(C.c_int)
    lib.fp4ar_gemm_plan.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, ip, ip, ip, ip, ip, C.c_int, ip, C.c_int]
    lib.fp4ar_gemm_plan.restype = C.c_int
    lib.fp4ar_gemm_reset.argtypes = []
    lib.fp4ar_gemm_reset.restype = C.c_int
    for name in ("fp4ar_create", "fp4ar_create_emulated", "fp4ar_launch", "fp4ar_status", "fp4ar_set_timeout_ms",
                 "fp4ar_reset", "fp4ar_destroy", "fp4ar_get_push_view", "fp4ar_ctas_per_rank", "fp4ar_encode",
                 "fp4ar_encode_static", "fp4ar_decode_sum", "fp4ar_reduce_reencode", "fp4ar_add_rmsnorm",
                 "fp4ar_fill_sentinel"):
        getattr(lib, name).restype = C.c_int
    return lib


class ContextPoisoned(RuntimeError):
    """A device-side wait of an earlier call gave up; the context refuses launches until its collective `reset()`."""


def check(rc: int, what: str) -> None:
    """Raise on a non-zero return code of the CUDA library."""
    if rc == 0:
        return
    if rc == 4:
        raise ContextPoisoned(f"{what} refused: an earlier call timed out waiting for a peer; read status(), then "
                              "call reset() on every rank")
    detail = ""
    if rc == 3:
        detail = ": " + (cuda().fp4ar_last_cuda_error() or b"").decode()
    raise RuntimeError(f"{what} failed: {ERROR_NAMES.get(rc, rc)}{detail}")
