"""`torch.ops.fp4ar.*` on a GPU: every op against the host model, one op captured in a CUDA graph and replayed with
three input sets, one traced by `torch.compile(fullgraph=True)` through its fake implementation, and the fused
row-parallel linear + AllReduce + norm op on two GPUs.

The one-GPU tests use a one-rank context (the AllReduce degenerates to encode + decode of the rank's own row, the
epilogue and every launch path stay the same); the reference project only plans this op surface
(docs/INTEGRATION.md:18-23)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.ops import allreduce as A
from fp4_all_reduce_b200.utils import data as D

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ROWS = 96


def _bits_equal(t: torch.Tensor, want: np.ndarray) -> int:
    got = O.bf16_bits(t) if t.dtype == torch.bfloat16 else t.cpu().numpy()
    return int(np.count_nonzero(got != want))


@pytest.fixture(scope="module")
def one_rank():
    from fp4_all_reduce_b200.parallel.context import Fp4ArContext

    ctx = Fp4ArContext(ROWS, device=torch.device("cuda", 0))
    cid = A.register_context(ctx)
    yield ctx, cid
    A.unregister_context(cid)
    ctx.close()


def _inputs(seed=0):
    x = D.partial(ROWS, 0, seed_offset=seed).cuda()
    res = D.residual(ROWS, seed=77 + seed).cuda()
    w = D.norm_weight().cuda()
    return x, res, w


def test_every_allreduce_op_matches_the_host_model(one_rank):
    ctx, cid = one_rank
    x, res, w = _inputs()
    xb, rb, wb = O.bf16_bits(x), O.bf16_bits(res), O.bf16_bits(w)
    # plain AllReduce
    want = O.allreduce([xb])
    assert _bits_equal(torch.ops.fp4ar.all_reduce(x, cid), want["out"]) == 0
    # + residual + norm, BF16 out; the residual is updated in place
    want = O.allreduce([xb], epi=1, res_in=rb, weight=wb, eps=1e-6, wbias=1.0)
    r1 = res.clone()
    y = torch.ops.fp4ar.all_reduce_add_rms_norm(x, r1, w, 1e-6, 1.0, cid)
    assert _bits_equal(y, want["out"]) == 0 and _bits_equal(r1, want["res_out"]) == 0
    # quantised outputs
    for kind in (N.EPI_NORM_NVFP4, N.EPI_NORM_MXFP8):
        want = O.allreduce([xb], epi=kind, res_in=rb, weight=wb, eps=1e-6, wbias=1.0, qscale=168.0)
        r2 = res.clone()
        yq = torch.ops.fp4ar.all_reduce_add_rms_norm_quant(x, r2, w, 1e-6, 1.0, kind, 168.0, cid)
        assert _bits_equal(yq, want["outq"]) == 0 and _bits_equal(r2, want["res_out"]) == 0
    # NVFP4 input with a static scale
    gs = [float(np.float32(np.abs(O.bf16_bits_to_f32(xb)).max() / 2688.0))]
    xq = torch.ops.fp4ar.encode_static(x, gs[0])
    assert _bits_equal(xq, O.encode_static(xb, gs[0])) == 0
    want = O.allreduce([O.encode_static(xb, gs[0])], input_kind=1, gs=gs)
    assert _bits_equal(torch.ops.fp4ar.all_reduce_nvfp4(xq, gs, cid), want["out"]) == 0
    want = O.allreduce([O.encode_static(xb, gs[0])], input_kind=1, gs=gs, epi=1, res_in=rb, weight=wb, eps=1e-6, wbias=1.0)
    r3 = res.clone()
    y = torch.ops.fp4ar.all_reduce_add_rms_norm_nvfp4(xq, gs, r3, w, 1e-6, 1.0, cid)
    assert _bits_equal(y, want["out"]) == 0 and _bits_equal(r3, want["res_out"]) == 0
    assert ctx.status().ok


def test_codec_and_norm_ops_match_the_host_model():
    x, res, w = _inputs(1)
    xb = O.bf16_bits(x)
    q, rs = torch.ops.fp4ar.encode(x)
    v, s, rsw = O.encode(xb)
    assert np.array_equal(q.cpu().numpy()[:, :3072], v) and np.array_equal(q.cpu().numpy()[:, 3072:], s)
    assert np.array_equal(rs.cpu().numpy().view(np.uint32), np.asarray(rsw, np.float32).view(np.uint32))
    x2 = D.partial(ROWS, 1, seed_offset=1).cuda()
    q2, rs2 = torch.ops.fp4ar.encode(x2)
    want = O.allreduce([xb, O.bf16_bits(x2)])["out"]
    assert _bits_equal(torch.ops.fp4ar.decode_sum([q, q2], [rs, rs2]), want) == 0
    r = res.clone()
    y = torch.ops.fp4ar.add_rms_norm(x, r, w, 1e-6, 1.0)
    want = O.add_rmsnorm(xb, O.bf16_bits(res), O.bf16_bits(w), eps=1e-6, wbias=1.0, epi=1)
    assert _bits_equal(y, want["out"]) == 0 and _bits_equal(r, want["res_out"]) == 0


def test_fused_block_op_in_a_cuda_graph_replayed_with_three_input_sets(one_rank):
    """A launch carries no host-side per-call state, so a captured op replays correctly on new data in the same buffers."""
    ctx, cid = one_rank
    x, res, w = _inputs(2)
    wb = O.bf16_bits(w)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        y = torch.ops.fp4ar.all_reduce_add_rms_norm(x, res, w, 1e-6, 1.0, cid)     # warm-up outside the capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = torch.ops.fp4ar.all_reduce_add_rms_norm(x, res, w, 1e-6, 1.0, cid)
    torch.cuda.synchronize()
    for seed in (3, 4, 5):
        xn, rn, _ = _inputs(seed)
        x.copy_(xn); res.copy_(rn)
        graph.replay()
        torch.cuda.synchronize()
        want = O.allreduce([O.bf16_bits(xn)], epi=1, res_in=O.bf16_bits(rn), weight=wb, eps=1e-6, wbias=1.0)
        assert _bits_equal(y, want["out"]) == 0 and _bits_equal(res, want["res_out"]) == 0, seed
    assert ctx.status().ok


def test_op_traces_with_torch_compile_fullgraph(one_rank):
    """Dynamo traces the op through its fake implementation with no graph break (`backend="eager"`: the traced graph is
    run op by op, so nothing but this library's kernels executes) and the result equals the eager call."""
    ctx, cid = one_rank
    x, res, w = _inputs(6)

    def block(x, res, w):
        y = torch.ops.fp4ar.all_reduce_add_rms_norm(x, res, w, 1e-6, 1.0, cid)
        return y, torch.ops.fp4ar.all_reduce(y, cid)

    r_eager, r_comp = res.clone(), res.clone()
    y0, z0 = block(x, r_eager, w)
    y1, z1 = torch.compile(block, fullgraph=True, backend="eager")(x, r_comp, w)
    torch.cuda.synchronize()
    assert torch.equal(y0.view(torch.int16), y1.view(torch.int16)) and torch.equal(z0.view(torch.int16), z1.view(torch.int16))
    assert torch.equal(r_eager.view(torch.int16), r_comp.view(torch.int16))


@pytest.mark.multigpu
def test_linear_all_reduce_norm_op_on_two_gpus():
    """torch.ops.fp4ar.linear_all_reduce_add_rms_norm (tcgen05 GEMM pushing NVFP4 partials into the peer + AllReduce +
    norm) and the plain AllReduce ops on two ranks, bit for bit against the host model."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(ROOT, "tests", "custom_ops_worker.py")]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    recs = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert p.returncode == 0 and recs, p.stdout[-2000:] + p.stderr[-3000:]
    assert all(r["mismatches"] == 0 for r in recs), recs
    assert {r["op"] for r in recs} >= {"all_reduce", "all_reduce_add_rms_norm", "linear_all_reduce_add_rms_norm"}
