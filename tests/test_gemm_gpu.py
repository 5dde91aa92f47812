"""The tcgen05 GEMM with NVFP4 epilogue: accumulators against an FP32 matmul, quantised rows bit for bit
against the host quantiser applied to the kernel's own accumulators, and the fused GEMM -> push -> AllReduce
path on emulated ranks against the host model fed with the kernel's NVFP4 partials."""
import numpy as np
import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.ops import gemm as G
from fp4_all_reduce_b200.parallel.context import EmulatedGroup, make_args
from fp4_all_reduce_b200.utils import data as D

pytestmark = pytest.mark.gpu


def _xw(M, K, Nn, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    wt = (torch.randn(Nn, K, generator=g) / K ** 0.5).to(torch.bfloat16).cuda()
    return x, wt


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("M,K,Nn", [(128, 64, 256), (300, 512, 512), (1024, 2048, 6144), (77, 4096, 6144)])
def test_gemm_accumulators_and_quantised_rows(M, K, Nn, pair, monkeypatch):
    monkeypatch.setenv("FP4AR_GEMM_PAIR", str(pair))      # 1: two CTAs per 256 x 256 tile (tcgen05 cta_group::2)
    x, wt = _xw(M, K, Nn, 1)
    gs = G.calibrate_gs(x, wt)
    q, acc = G.gemm_nvfp4(x, wt, gs, want_acc=True)
    torch.cuda.synchronize()
    assert G.gemm_status().code == 0
    ref = x.float() @ wt.float().t()
    err = (acc - ref).abs().max().item()
    assert err <= 2e-3 * ref.abs().max().item() + 1e-4, err
    want = O.encode_static_f32(acc.cpu().numpy(), gs)
    assert np.count_nonzero(q.cpu().numpy() != want) == 0


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("P", [2, 4])
def test_gemm_push_then_allreduce_on_emulated_ranks(P, pair, monkeypatch):
    monkeypatch.setenv("FP4AR_GEMM_PAIR", str(pair))
    M, K = 256, 512
    g = EmulatedGroup(P, M)
    g.set_timeout_ms(500)
    xs, wts, gss, qs = [], [], [], []
    for r in range(P):
        x, wt = _xw(M, K, N.HIDDEN, 10 + r)
        xs.append(x); wts.append(wt)
        gss.append(G.calibrate_gs(x, wt))
    res = [D.residual(M).cuda() for _ in range(P)]
    res0 = res[0].clone()
    w = D.norm_weight().cuda()
    outs = [torch.zeros(M, N.HIDDEN, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    for call in range(3):                       # three calls: both window buffers and a reuse
        for r in range(P):
            res[r].copy_(res0)
            lq = torch.empty(M, N.QROW_BYTES, dtype=torch.uint8, device="cuda")
            G.gemm_push(g, xs[r], wts[r], gss[r], two_shot=P > 2, local_rank=r, local_q=lq)
            qs.append(lq)
        g.launch([make_args(x=None, out=outs[r], rows=M, input=N.IN_PUSHED, gs=gss, epilogue=N.EPI_NORM_BF16,
                            res_in=res[r], res_out=res[r], weight=w,
                            algo=N.ALGO_TWOSHOT if P > 2 else N.ALGO_ONESHOT) for r in range(P)])
        torch.cuda.synchronize()
        assert g.status(0).ok, g.status(0).describe()
        partials = [t.cpu().numpy() for t in qs[-P:]]
        exp = O.allreduce(partials, algo=1 if P > 2 else 0, input_kind=1, gs=gss, epi=1, res_in=O.bf16_bits(res0),
                          weight=O.bf16_bits(w))
        for r in range(P):
            assert np.array_equal(O.bf16_bits(outs[r]), exp["out"]), (call, r)
            assert np.array_equal(O.bf16_bits(res[r]), exp["res_out"]), (call, r)
    g.close()


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("M,K", [(1024, 2048), (2048, 512), (1000, 1024), (2300, 320)])
def test_gemm_stream_k_split(M, K, pair, monkeypatch):
    """Tile counts that do not fill the last wave of CTAs run with the K loop cut into equal ranges per CTA: a tile shared
    by two CTAs is summed from a partial accumulator.  Same checks as for whole tiles, over several calls (the partial
    slots and their flags are reused), inside a CUDA graph of back-to-back launches, and against the whole-tile walk."""
    Nn = N.HIDDEN
    x, wt = _xw(M, K, Nn, 3)
    gs = G.calibrate_gs(x, wt)
    ref = x.float() @ wt.float().t()
    tol = 2e-3 * ref.abs().max().item() + 1e-4
    monkeypatch.setenv("FP4AR_GEMM_PAIR", str(pair))
    monkeypatch.setenv("FP4AR_GEMM_STREAM_K", "0")
    q_plain, acc_plain = G.gemm_nvfp4(x, wt, gs, want_acc=True)
    torch.cuda.synchronize()
    monkeypatch.setenv("FP4AR_GEMM_STREAM_K", "1")
    for call in range(3):
        q, acc = G.gemm_nvfp4(x, wt, gs, want_acc=True)
        torch.cuda.synchronize()
        assert G.gemm_status().code == 0
        assert (acc - ref).abs().max().item() <= tol
        want = O.encode_static_f32(acc.cpu().numpy(), gs)
        assert np.count_nonzero(q.cpu().numpy() != want) == 0
        # the split changes the order of the FP32 additions, nothing else
        assert (acc - acc_plain).abs().max().item() <= 1e-5 * ref.abs().max().item() + 1e-6
    assert (q != q_plain).float().mean().item() < 0.01
    first = q.clone()
    st = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    outs = [torch.empty_like(q) for _ in range(3)]
    with torch.cuda.stream(st):
        G.gemm_nvfp4(x, wt, gs, out=outs[0])
        st.synchronize()
        with torch.cuda.graph(g, stream=st):
            for o in outs:
                G.gemm_nvfp4(x, wt, gs, out=o)
    for _ in range(2):
        for o in outs:
            o.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert G.gemm_status().code == 0
        for o in outs:
            assert torch.equal(o, first)


def test_gemm_reset_keeps_the_kernel_usable():
    x, wt = _xw(1024, 2048, N.HIDDEN, 5)
    gs = G.calibrate_gs(x, wt)
    q0 = G.gemm_nvfp4(x, wt, gs)
    G.gemm_reset()
    assert G.gemm_status().code == 0
    q1 = G.gemm_nvfp4(x, wt, gs)
    torch.cuda.synchronize()
    assert G.gemm_status().code == 0 and torch.equal(q0, q1)
