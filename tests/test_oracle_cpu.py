"""CPU tests of the host bit-exact model against the independent numpy model (tests/ref_numpy.py).

Mirrors the reference project's unit level (tests/codec_test.cu:9-72 and the exhaustive primitive tests
T1-T5 of bench/codec/codec_bench.cu:29-134), with the roles shifted: there a GPU codec is checked against
a CPU oracle; here the C++ oracle itself is pinned first, on the CPU, and the GPU tests then use it.
"""
import numpy as np
import pytest
import torch

import ref_numpy as R
from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.utils import data as D


def all_bf16_as_f32():
    return R.bf16_to_f32(np.arange(65536, dtype=np.uint32).astype(np.uint16))


def test_e2m1_encode_all_bf16_and_midpoints():
    x = all_bf16_as_f32()
    got = O.e2m1_encode(x)
    want = R.e2m1_encode(x)
    assert np.array_equal(got, want)
    mids = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.5, 1e30, np.inf], np.float32)
    for s in (1, -1):
        assert np.array_equal(O.e2m1_encode(s * mids), R.e2m1_encode(s * mids))
    eps = np.float32(2.0 ** -20)
    near = np.concatenate([mids[:7] * (1 + eps), mids[:7] * (1 - eps)]).astype(np.float32)
    assert np.array_equal(O.e2m1_encode(near), R.e2m1_encode(near))
    assert O.e2m1_encode(np.array([np.nan], np.float32))[0] == 7
    assert O.e2m1_encode(np.array([-0.0], np.float32))[0] == 8


def test_e4m3_encode_dense_sweep():
    # every BF16 value >= 0 plus a dense FP32 sweep around every rounding boundary
    x = all_bf16_as_f32()
    x = x[((x >= 0) & ~np.signbit(x)) | np.isnan(x)]
    assert np.array_equal(O.e4m3_encode(x), R.e4m3_encode(x))
    vals = R.E4M3
    mids = ((vals[:-1] + vals[1:]) / 2).astype(np.float32)
    probe = []
    for m in mids:
        u = int(np.array([m], np.float32).view(np.uint32)[0])
        probe += [np.array([u + d], np.uint32).view(np.float32)[0] for d in (-2, -1, 0, 1, 2) if u + d > 0]
    probe = np.array(probe + [447.9, 448.0, 463.9, 464.0, 1e9, np.inf, 2.0 ** -10, 2.0 ** -11, 1e-30, 0.0], np.float32)
    assert np.array_equal(O.e4m3_encode(probe), R.e4m3_encode(probe))
    rng = np.random.default_rng(0)
    r = np.abs(rng.standard_normal(20000).astype(np.float32)) * np.float32(2.0) ** rng.integers(-12, 10, 20000)
    assert np.array_equal(O.e4m3_encode(r.astype(np.float32)), R.e4m3_encode(r.astype(np.float32)))
    assert O.e4m3_encode(np.array([np.nan], np.float32))[0] == 0x7F


def test_tables():
    t = O.e4m3_table()
    assert np.array_equal(t[:127], R.E4M3.astype(np.float32))
    assert np.isnan(t[127])
    assert np.array_equal(O.e2m1_table()[:8], R.E2M1.astype(np.float32))
    assert np.array_equal(O.e2m1_table()[8:], -R.E2M1.astype(np.float32))


def test_bf16_rounding():
    rng = np.random.default_rng(1)
    x = rng.standard_normal(100000).astype(np.float32) * np.float32(2.0) ** rng.integers(-30, 30, 100000).astype(np.float32)
    got = O.f32_to_bf16_bits(x)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want)
    assert np.array_equal(got, R.f32_to_bf16(x))


def test_canon_neg0_exhaustive_16bit():
    lo = np.arange(65536, dtype=np.uint32)
    for hi in (0x0000, 0x8888, 0x8080, 0x1234, 0xFFFF):
        w = lo | (np.uint32(hi) << 16)
        got = O.canon_neg0(w)
        want = w.copy()
        for k in range(8):
            nib = (w >> (4 * k)) & 15
            want = np.where(nib == 8, want & ~(np.uint32(15) << (4 * k)), want)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("src", [0, 1])
def test_encode_rows_match_numpy_model(src):
    x = D.special_rows(16, src)
    bits = O.bf16_bits(x)
    v, s, rs = O.encode(bits)
    f = R.bf16_to_f32(bits)
    for r in range(16):
        rv, rsb, rrs = R.encode_row(f[r])
        assert np.array_equal(v[r], rv), f"values differ in special row class {(r + 7 * src) % 16}"
        assert np.array_equal(s[r], rsb), f"scales differ in special row class {(r + 7 * src) % 16}"
        assert rs[r].tobytes() == np.float32(rrs).tobytes()
    # no encoder output may look like a sentinel
    words = v.view(np.uint32)
    assert not np.any(words == 0x88888888)
    assert not np.any(s & 0x80)
    assert not np.any(rs.view(np.uint32) == 0x80000000)


def test_encode_static_matches_numpy_model():
    x = D.partial(3, 0)
    bits = O.bf16_bits(x)
    f = R.bf16_to_f32(bits)
    gs = float(np.max(np.abs(f))) / 2688.0
    q = O.encode_static(bits, gs)
    inv = np.float32(1.0) / np.float32(gs)
    for r in range(3):
        rv, rsb, _ = R.encode_row(f[r], inv=inv)
        assert np.array_equal(q[r, :3072], rv)
        assert np.array_equal(q[r, 3072:], rsb)


def test_decode_acc_matches_exact_fma():
    xs = [D.special_rows(3, s) for s in range(2)] + [D.partial(3, 5)]
    enc = [O.encode(O.bf16_bits(x)) for x in xs]
    acc = np.zeros((3, 6144), np.float32)
    want = np.zeros((3, 6144), np.float32)
    for v, s, rs in enc:
        O.decode_acc(acc, v, s, rs)
        for r in range(3):
            want[r] = R.decode_acc_row(want[r], v[r], s[r], rs[r])
    a, b = acc.view(np.uint32), want.view(np.uint32)
    nan = np.isnan(acc) & np.isnan(want)
    assert np.array_equal(a[~nan], b[~nan])


def test_row_sumsq_order():
    rng = np.random.default_rng(3)
    z = (rng.standard_normal(6144) * 3).astype(np.float32)
    assert np.float32(O.row_sumsq(z)).tobytes() == np.float32(R.row_sumsq(z)).tobytes()


def _compose_oneshot(xs_bits):
    acc = np.zeros((xs_bits[0].shape[0], 6144), np.float32)
    for b in xs_bits:
        v, s, rs = O.encode(b)
        O.decode_acc(acc, v, s, rs)
    return acc


@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_allreduce_oneshot_is_composition(P):
    xs = [O.bf16_bits(D.gaussian_mags(8, s, 1)) for s in range(P)]
    r = O.allreduce(xs, algo=0, want_sum=True)
    acc = _compose_oneshot(xs)
    assert np.array_equal(r["sum"].view(np.uint32), acc.view(np.uint32))
    assert np.array_equal(r["out"], O.f32_to_bf16_bits(acc))


@pytest.mark.parametrize("P", [2, 4, 8])
def test_allreduce_twoshot_is_reencode_of_sum(P):
    xs = [O.bf16_bits(D.gaussian_mags(8, s, 2)) for s in range(P)]
    acc = _compose_oneshot(xs)
    v, s, rs = O.encode_f32(acc)
    acc2 = np.zeros_like(acc)
    O.decode_acc(acc2, v, s, rs)
    r = O.allreduce(xs, algo=1, want_sum=True)
    assert np.array_equal(r["sum"].view(np.uint32), acc2.view(np.uint32))
    assert np.array_equal(r["out"], O.f32_to_bf16_bits(acc2))


def test_allreduce_static_input():
    P = 2
    xs = [O.bf16_bits(D.partial(8, s)) for s in range(P)]
    gs = [float(np.max(np.abs(R.bf16_to_f32(x)))) / 2688.0 for x in xs]
    qs = [O.encode_static(x, g) for x, g in zip(xs, gs)]
    r = O.allreduce(qs, algo=0, input_kind=1, gs=gs, want_sum=True)
    acc = np.zeros((8, 6144), np.float32)
    for q, g in zip(qs, gs):
        O.decode_acc(acc, q[:, :3072], q[:, 3072:], float(np.float32(g)))
    assert np.array_equal(r["sum"].view(np.uint32), acc.view(np.uint32))


def test_norm_epilogue_against_float64():
    P = 2
    rows = 6
    xs = [O.bf16_bits(D.partial(rows, s)) for s in range(P)]
    res = O.bf16_bits(D.residual(rows))
    w = O.bf16_bits(D.norm_weight())
    r = O.allreduce(xs, algo=0, epi=1, res_in=res, weight=w, want_sum=True)
    z = r["sum"].astype(np.float64) + R.bf16_to_f32(res).astype(np.float64)
    assert np.array_equal(r["res_out"], O.f32_to_bf16_bits((r["sum"] + R.bf16_to_f32(res)).astype(np.float32)))
    zb = R.bf16_to_f32(r["res_out"]).astype(np.float64)
    rinv = 1.0 / np.sqrt((z * z).mean(axis=1, keepdims=True) + 1e-6)
    y = zb * rinv * (1.0 + R.bf16_to_f32(w).astype(np.float64))
    got = R.bf16_to_f32(r["out"]).astype(np.float64)
    # BF16 output: at most one ulp (2^-8 relative) away from the float64 evaluation
    assert np.all(np.abs(got - y) <= np.abs(y) * 2.0 ** -7 + 1e-30)
    # the stand-alone norm op is the same epilogue applied to a BF16 tensor
    x0 = O.f32_to_bf16_bits(r["sum"])
    a = O.add_rmsnorm(x0, res, w, epi=1)
    assert a["out"].shape == (rows, 6144)


def test_norm_quantised_outputs_decode_close_to_bf16_output():
    rows = 4
    xs = [O.bf16_bits(D.partial(rows, s)) for s in range(2)]
    res = O.bf16_bits(D.residual(rows)); w = O.bf16_bits(D.norm_weight())
    y = R.bf16_to_f32(O.allreduce(xs, epi=1, res_in=res, weight=w)["out"])
    qs = float(np.float32(2688.0 / np.max(np.abs(y))))      # the usual calibration: 448 * 6 / amax
    q4 = O.allreduce(xs, epi=2, res_in=res, weight=w, qscale=qs)["outq"]
    t4, t2 = O.e4m3_table(), O.e2m1_table()
    vals = q4[:, :3072]; sc = q4[:, 3072:]
    nib = np.stack([vals & 15, vals >> 4], axis=-1).reshape(rows, 6144)
    dec = t2[nib] * np.repeat(t4[sc], 16, axis=1) / np.float32(qs)
    rel = np.linalg.norm(dec - y) / np.linalg.norm(y)
    assert rel < 0.15
    q8 = O.allreduce(xs, epi=3, res_in=res, weight=w)["outq"]
    v8 = t4[q8[:, :6144]]
    e8 = q8[:, 6144:].astype(np.int32)
    dec8 = v8 * np.repeat(np.exp2((e8 - 127).astype(np.float32)), 32, axis=1)
    rel8 = np.linalg.norm(dec8 - y) / np.linalg.norm(y)
    assert rel8 < 0.04


def test_benchmark_config0_two_simulated_ranks():
    """Two simulated ranks, [1024 x 6144] partials of the benchmark distribution: round trip bit-exact with the
    composed codec, rel-L2 against the exact FP32 sum in the expected range."""
    rows = 1024
    xs = [O.bf16_bits(D.partial(rows, r)) for r in range(2)]
    r = O.allreduce(xs, algo=0, want_sum=True)
    assert np.array_equal(r["sum"].view(np.uint32), _compose_oneshot(xs).view(np.uint32))
    exact = sum(R.bf16_to_f32(x).astype(np.float32) for x in xs)
    got = R.bf16_to_f32(r["out"])
    rel = float(np.linalg.norm(got - exact) / np.linalg.norm(exact))
    assert 0.02 < rel < 0.2, rel
    rel2 = float(np.linalg.norm(R.bf16_to_f32(O.allreduce(xs, algo=1)["out"]) - exact) / np.linalg.norm(exact))
    assert rel < rel2 < 0.3


def test_software_models_of_the_device_selftests_match_the_host_model(cuda_lib):
    """The plain software encoders / decoders that the exhaustive GPU self-tests compare the hardware with
    (csrc/kernels/selftest.cu) agree with the host model on dense sweeps, so a GPU mismatch would point at the GPU side."""
    import ctypes as C

    from fp4_all_reduce_b200 import _native as NN

    lib = cuda_lib           # loading the library needs no GPU; only host functions are called
    lib.fp4ar_selftest_soft_model.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    rng = np.random.default_rng(5)
    # E4M3: every BF16-representable non-negative value, a dense log sweep, ties, the saturation edge, inf and NaN
    bits = np.arange(0, 0x7f81, dtype=np.uint32) << 16
    x = np.concatenate([bits.view(np.float32), np.exp(rng.uniform(-25, 8, 400000)).astype(np.float32),
                        np.array([447.9, 448.0, 463.9, 464.0, 479.9, 480.0, 1e9, np.inf, np.nan, 2.0 ** -9, 2.0 ** -10,
                                  1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9], np.float32)])
    out = np.zeros(x.size, np.uint32)
    assert lib.fp4ar_selftest_soft_model(0, x.ctypes.data, None, x.size, out.ctypes.data) == 0
    assert np.array_equal(out.astype(np.uint8), O.e4m3_encode(x))
    # E2M1: all BF16 values of both signs, midpoints, random
    allbf = (np.arange(0, 0x10000, dtype=np.uint32) << 16).view(np.float32)
    y = np.concatenate([allbf, rng.normal(0, 3, 400000).astype(np.float32),
                        np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -5.0, 6.0, 7.0, -0.0, 0.0], np.float32)])
    out = np.zeros(y.size, np.uint32)
    assert lib.fp4ar_selftest_soft_model(1, y.ctypes.data, None, y.size, out.ctypes.data) == 0
    assert np.array_equal(out.astype(np.uint8), O.e2m1_encode(y))
    # decode tables
    n16 = np.arange(16, dtype=np.uint32)
    out = np.zeros(16, np.uint32)
    assert lib.fp4ar_selftest_soft_model(2, None, n16.ctypes.data, 16, out.ctypes.data) == 0
    assert np.array_equal(out, O.e2m1_table().view(np.uint32))
    n256 = np.arange(256, dtype=np.uint32)
    out = np.zeros(256, np.uint32)
    assert lib.fp4ar_selftest_soft_model(3, None, n256.ctypes.data, 256, out.ctypes.data) == 0
    tab = O.e4m3_table()
    finite = ~np.isnan(tab)
    assert np.array_equal(out[finite], tab.view(np.uint32)[finite])
