"""The comparison variants (flag push, pull, pull with NVFP4 input, two-shot pull, pull + pushed all-gather) on one
GPU (ranks emulated as CTA groups of one cooperative launch): bit-identical to the one-shot / two-shot host model,
across calls (both buffers, generation counter), in a CUDA graph, and with a row count that is not a multiple of
the tile."""

import numpy as np
import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.harness.gate import CellConfig, make_inputs
from fp4_all_reduce_b200.parallel.compare import TWO_SHOT, CompareEmulated

pytestmark = pytest.mark.gpu


def _mism(t, exp_bits):
    return int(np.count_nonzero(O.bf16_bits(t) != exp_bits))


@pytest.mark.parametrize("variant", ["flag_push", "pull", "pull_nvfp4", "pull_twoshot", "pull_rs_push_ag"])
@pytest.mark.parametrize("P", [1, 2, 4, 8])
def test_compare_variant_matches_host_model(variant, P):
    if variant in TWO_SHOT and P == 1:
        pytest.skip("two-shot needs at least two ranks")
    dev = torch.device("cuda", 0)
    rows = 203                                   # not a multiple of 4: the last tile is ragged
    cfg = CellConfig(nranks=P, rows=rows, algo=N.ALGO_TWOSHOT if variant in TWO_SHOT else N.ALGO_ONESHOT,
                     input=N.IN_NVFP4 if variant == "pull_nvfp4" else N.IN_BF16, dist="mags")
    sets = [make_inputs(cfg, s, dev) for s in range(3)]
    grp = CompareEmulated(P, 256, dev)
    grp.timeout_ms = 300                       # a broken hand-off ends in seconds, not minutes
    outs = [torch.zeros(rows, N.HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(P)]
    for call in range(7):                        # both buffers several times over, changing inputs
        s = sets[call % 3]
        for o in outs:
            o.zero_()
        grp.all_reduce(variant, s.xs, outs, gs=s.gs)
        torch.cuda.synchronize()
        assert grp.status().ok, grp.status().describe()
        for r in range(P):
            assert _mism(outs[r], s.exp["out"]) == 0, (variant, P, call, r)
    # a shorter call in between, then a captured graph of several calls
    short = [x[:57].contiguous() for x in sets[0].xs]
    souts = [torch.zeros(57, N.HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(P)]
    grp.all_reduce(variant, short, souts, gs=sets[0].gs)
    torch.cuda.synchronize()
    assert grp.status().ok, grp.status().describe()
    assert _mism(souts[0], sets[0].exp["out"][:57]) == 0
    st = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        grp.all_reduce(variant, sets[1].xs, outs, stream=st, gs=sets[1].gs)     # warm-up on the capture stream
        st.synchronize()
        with torch.cuda.graph(g, stream=st):
            for _ in range(3):
                grp.all_reduce(variant, sets[2].xs, outs, stream=st, gs=sets[2].gs)
    for _ in range(2):
        for o in outs:
            o.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert grp.status().ok, grp.status().describe()
        for r in range(P):
            assert _mism(outs[r], sets[2].exp["out"]) == 0


def test_compare_rejects_bad_arguments():
    dev = torch.device("cuda", 0)
    grp = CompareEmulated(2, 64, dev)
    x = [torch.zeros(65, N.HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    with pytest.raises(ValueError):
        grp.all_reduce("pull", x, x)
    with pytest.raises(KeyError):
        grp.all_reduce("nope", [t[:8].contiguous() for t in x], [t[:8].contiguous() for t in x])
