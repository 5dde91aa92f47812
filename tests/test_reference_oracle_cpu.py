"""The host model of this repository against the reference project's OWN CPU oracle (its `namespace cpu`, compiled
untouched and called through baseline/ref_oracle_shim.cu), bit for bit, on the host.  Skipped when the reference
tree is not on the machine or the bridge cannot be built."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.utils import data as D

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import build_ref
    finally:
        sys.path.pop(0)
    ref_dir = build_ref.reference_dir()
    if not (ref_dir and Path(ref_dir).exists()) and not (ROOT / "baseline" / "_ref" / "libref_oracle.so").exists():
        pytest.skip("reference tree not present")
    lib_path = build_ref.build_host_oracle()
    if lib_path is None:
        pytest.skip("the bridge to the reference's CPU oracle could not be built")
    lib = C.CDLL(str(lib_path))
    lib.ref_cpu_allreduce.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    lib.ref_cpu_encode_rows.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    return lib


def _inputs(P, rows, special):
    xs = []
    for r in range(P):
        t = D.special_rows(rows, r) if special else D.partial(rows, r)
        xs.append(np.ascontiguousarray(O.bf16_bits(t)))
    return xs


def _finite_rows(xs):
    """Rows whose every element is finite in every rank: the two oracles only promise agreement there (the
    reference's CPU code and its GPU code themselves differ on NaN / Inf payload conventions)."""
    ok = np.ones(xs[0].shape[0], bool)
    for x in xs:
        ok &= np.isfinite(O.bf16_bits_to_f32(x)).all(axis=1)
    return ok


@pytest.mark.parametrize("special", [False, True])
def test_encode_matches_reference_cpu_oracle(ref, special):
    rows = 96
    x = _inputs(1, rows, special)[0]
    v = np.zeros((rows, N.VALUE_BYTES), np.uint8)
    s = np.zeros((rows, N.SCALE_BYTES), np.uint8)
    rs = np.zeros(rows, np.float32)
    assert ref.ref_cpu_encode_rows(rows, x.ctypes.data, v.ctypes.data, s.ctypes.data, rs.ctypes.data, 1) == 0
    mv, ms, mrs = O.encode(x, canon=True)
    ok = _finite_rows([x])
    assert ok.sum() >= rows // 2
    assert np.array_equal(v[ok], mv[ok]) and np.array_equal(s[ok], ms[ok])
    assert np.array_equal(rs[ok].view(np.uint32), mrs[ok].view(np.uint32))


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("two_shot", [0, 1])
@pytest.mark.parametrize("special", [False, True])
def test_allreduce_matches_reference_cpu_oracle(ref, P, two_shot, special):
    rows = 64
    xs = _inputs(P, rows, special)
    ptrs = (C.c_void_p * P)(*[x.ctypes.data for x in xs])
    out = np.zeros((rows, N.HIDDEN), np.uint16)
    assert ref.ref_cpu_allreduce(P, rows, ptrs, two_shot, out.ctypes.data) == 0
    mine = O.allreduce(xs, algo=two_shot, input_kind=0)["out"]
    ok = _finite_rows(xs)
    assert ok.sum() >= rows // 2
    # Where a sum of huge finite values overflows, both models produce NaN, but with the NaN encoding of the machine
    # they model (x86 default NaN has the sign bit set, the GPU's canonical NaN does not): compare NaN positions there
    # and bits everywhere else.
    a, b = out[ok], mine[ok]
    nan_a, nan_b = np.isnan(O.bf16_bits_to_f32(a)), np.isnan(O.bf16_bits_to_f32(b))
    assert np.array_equal(nan_a, nan_b)
    assert np.array_equal(a[~nan_a], b[~nan_b]), int(np.count_nonzero(a[~nan_a] != b[~nan_b]))
    assert (~nan_a).sum() >= a.size // 4
