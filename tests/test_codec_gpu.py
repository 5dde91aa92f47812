"""GPU tests of the stand-alone sm_100a codec / norm kernels against the host bit-exact model.

Counterpart of the reference project's row-kernel checks ("ORACLE" / "CHECK ... bit-exact" lines of
bench/codec/codec_bench.cu:808-828), including its special-row classes.
"""
import numpy as np
import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.ops import codec
from fp4_all_reduce_b200.utils import data as D

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _same_bf16(t, want_bits):
    got = O.bf16_bits(t)
    gn = (got & 0x7FFF) > 0x7F80
    wn = (want_bits & 0x7FFF) > 0x7F80
    return int(np.count_nonzero((got != want_bits) & ~(gn & wn)))


@pytest.mark.parametrize("dist,rows", [("special", 64), ("partial", 333), ("mags", 1024)])
def test_encode_bit_exact(dist, rows):
    x = {"special": lambda: D.special_rows(rows, 1), "partial": lambda: D.partial(rows, 0),
         "mags": lambda: D.gaussian_mags(rows, 2, 0)}[dist]()
    q, rs = codec.encode(x.to(DEV))
    torch.cuda.synchronize()
    v, s, r = O.encode(O.bf16_bits(x))
    qh = q.cpu().numpy()
    assert np.count_nonzero(qh[:, :3072] != v) == 0
    assert np.count_nonzero(qh[:, 3072:] != s) == 0
    assert np.array_equal(rs.cpu().numpy().view(np.uint32), r.view(np.uint32))


def test_encode_static_bit_exact():
    x = D.partial(500, 3)
    f = x.float()
    gs = float(np.float32(f.abs().max().item() / 2688.0))
    q = codec.encode_static(x.to(DEV), gs)
    torch.cuda.synchronize()
    assert np.count_nonzero(q.cpu().numpy() != O.encode_static(O.bf16_bits(x), gs)) == 0


@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_decode_sum_bit_exact(P):
    rows = 200
    xs = [D.special_rows(rows, s) if s % 2 else D.partial(rows, s) for s in range(P)]
    enc = [codec.encode(x.to(DEV)) for x in xs]
    out = codec.decode_sum([e[0] for e in enc], [e[1] for e in enc])
    torch.cuda.synchronize()
    want = O.allreduce([O.bf16_bits(x) for x in xs], algo=0)["out"]
    assert _same_bf16(out, want) == 0


@pytest.mark.parametrize("P", [2, 4, 8])
def test_reduce_reencode_bit_exact(P):
    rows = 160
    xs = [D.gaussian_mags(rows, s, 5) if s != 1 else D.special_rows(rows, s) for s in range(P)]
    enc = [codec.encode(x.to(DEV)) for x in xs]
    rec, out = codec.reduce_reencode([e[0] for e in enc], [e[1] for e in enc])
    torch.cuda.synchronize()
    bits = [O.bf16_bits(x) for x in xs]
    r = O.allreduce(bits, algo=1, want_sum=True)
    assert _same_bf16(out, r["out"]) == 0
    # the record is the encoding of the FP32 one-shot sum
    s1 = O.allreduce(bits, algo=0, want_sum=True)["sum"]
    v, s, rs = O.encode_f32(s1)
    rh = rec.cpu().numpy()
    ok = ~np.isnan(rs)
    assert np.count_nonzero(rh[ok][:, :3072] != v[ok]) == 0
    assert np.count_nonzero(rh[ok][:, 3072:3456] != s[ok]) == 0
    got_rs = rh[:, 3456:3472].copy().view(np.uint32).reshape(rows, 4)
    assert np.array_equal(got_rs[ok], np.repeat(rs.view(np.uint32)[:, None], 4, axis=1)[ok])


def test_decode_sum_static_scales():
    rows, P = 128, 2
    xs = [D.partial(rows, s) for s in range(P)]
    gs = [float(np.float32(x.float().abs().max().item() / 2688.0)) for x in xs]
    qs = [codec.encode_static(x.to(DEV), g) for x, g in zip(xs, gs)]
    out = codec.decode_sum(qs, None, gs)
    torch.cuda.synchronize()
    want = O.allreduce([q.cpu().numpy() for q in qs], algo=0, input_kind=1, gs=gs)["out"]
    assert _same_bf16(out, want) == 0


@pytest.mark.parametrize("epi", [1, 2, 3])
def test_add_rmsnorm_bit_exact(epi):
    rows = 300
    x = D.partial(rows, 7); res = D.residual(rows); w = D.norm_weight()
    qscale = 168.0
    y, ro = codec.add_rmsnorm(x.to(DEV), res.to(DEV), w.to(DEV), epilogue=epi, qscale=qscale)
    torch.cuda.synchronize()
    want = O.add_rmsnorm(O.bf16_bits(x), O.bf16_bits(res), O.bf16_bits(w), epi=epi, qscale=qscale)
    assert _same_bf16(ro, want["res_out"]) == 0
    if epi == 1:
        assert _same_bf16(y, want["out"]) == 0
    else:
        assert np.count_nonzero(y.cpu().numpy() != want["outq"]) == 0


def test_fill_sentinel_pattern():
    buf = 3584 * 5 + 512   # five slots and a tail, two buffers
    buf = (buf + 4095) // 4096 * 4096
    w = torch.zeros(2 * buf, dtype=torch.uint8, device=DEV)
    codec.fill_sentinel(w, buf, 2)
    torch.cuda.synchronize()
    h = w.cpu().numpy().reshape(2, buf)
    for b in range(2):
        for slot in range(5):
            r = h[b, slot * 3584:(slot + 1) * 3584]
            assert np.all(r[:3072] == 0x88) and np.all(r[3072:3456] == 0xFF)
            assert np.array_equal(r[3456:3472].view(np.uint32), np.full(4, 0x80000000, np.uint32))


def test_division_free_multiplier_is_the_ieee_quotient():
    """All 2^23 mantissas x 126 scale bytes for each of the 201 exponents of the supported range (2 x 10^11 cases)."""
    import ctypes as C
    cnt = torch.zeros(1, dtype=torch.int64, device=DEV)
    for e in range(27, 228):       # every exponent of the admitted range 2^-100 .. 2^100
        N.check(N.cuda().fp4ar_selftest_scale_division(e, cnt.data_ptr(), None), "selftest")
    torch.cuda.synchronize()
    assert int(cnt.item()) == 0


def test_hardware_conversions_match_software_models_exhaustively():
    """E4M3 block scale of x / 6 for all 2^31 non-negative floats, E2M1 value encode for all 2^32 floats in every
    nibble position, both decode tables and the -0 canonicalisation."""
    counters = torch.zeros(3, dtype=torch.int64, device=DEV)
    lib = N.cuda()
    N.check(lib.fp4ar_selftest_conversions(0, 0, 0, counters[0:].data_ptr(), None), "block scale")
    N.check(lib.fp4ar_selftest_conversions(1, 0, 0x80000000, counters[1:].data_ptr(), None), "value encode, positive")
    N.check(lib.fp4ar_selftest_conversions(1, 0x80000000, 0, counters[1:].data_ptr(), None), "value encode, negative")
    N.check(lib.fp4ar_selftest_conversions(2, 0, 0, counters[2:].data_ptr(), None), "decode tables")
    torch.cuda.synchronize()
    assert counters.tolist() == [0, 0, 0], counters.tolist()


def test_pair_encoders_agree_and_never_emit_a_sentinel():
    """2^28 pseudo-random BF16 pairs and 2^26 FP32 pairs in four classes (any finite value, tiny magnitudes, a narrow
    band, mostly zeros of both signs): the encoder with table-driven multipliers gives the words of the encoder with
    IEEE divisions, and no value word, scale byte or row scale equals its sentinel; 2^28 decode-accumulate cases over
    every pair of scale bytes equal scalar table arithmetic.  (The reference's T3-T5: bench/codec/codec_bench.cu:66-134.)"""
    lib = N.cuda()
    c = torch.zeros(6, dtype=torch.int64, device=DEV)
    N.check(lib.fp4ar_selftest_conversions(3, 12345, 1 << 28, c[0:].data_ptr(), None), "BF16 pairs")
    N.check(lib.fp4ar_selftest_conversions(4, 777, 1 << 26, c[2:].data_ptr(), None), "FP32 pairs")
    N.check(lib.fp4ar_selftest_conversions(5, 4242, 1 << 14, c[4:].data_ptr(), None), "decode-accumulate")
    torch.cuda.synchronize()
    assert c.tolist() == [0, 0, 0, 0, 0, 0], c.tolist()
