"""The bitwise gate on one GPU: every tensor-parallel degree runs as CTA groups of one cooperative launch
(real fused kernel, real Lamport protocol, windows in the same device memory).

Counterpart of the reference project's integration gate (harness/fp4ar_bench.cu:278-346, tests/gate.sh,
tests/negative_control.sh), which needs 2 or 4 GPUs; the multi-GPU form of this gate is
tests/test_allreduce_multigpu.py.
"""
import pytest
import torch

from fp4_all_reduce_b200 import _native as N
from fp4_all_reduce_b200.harness.gate import CellConfig, gate_cell_emulated, make_inputs, Outputs, args_for, mismatches
from fp4_all_reduce_b200.parallel.context import EmulatedGroup

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("P", [1, 2, 4, 8])
@pytest.mark.parametrize("inp", [N.IN_BF16, N.IN_NVFP4])
def test_allreduce_gate(P, inp):
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=413, input=inp, dist="mags"), reps=9)
    assert rec["pass"], rec
    if inp == N.IN_BF16:
        assert rec["rel_l2_vs_fp32"] < 0.2, rec


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("epi", [1, 2, 3])
def test_fused_norm_gate(P, epi):
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=300, epilogue=epi, dist="partial"), reps=6)
    assert rec["pass"], rec


@pytest.mark.parametrize("P,algo", [(2, 1), (4, 0), (8, 0)])
def test_other_algorithm_of_each_degree(P, algo):
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=257, algo=algo, dist="mags"), reps=6)
    assert rec["pass"], rec


@pytest.mark.parametrize("P", [2, 4])
def test_special_rows(P):
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=96, dist="special"), reps=3, graph_calls=0)
    assert rec["pass"], rec


@pytest.mark.parametrize("P", [2, 8])
@pytest.mark.parametrize("inp", [N.IN_NVFP4])
def test_fused_norm_nvfp4_input(P, inp):
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=222, input=inp, epilogue=1), reps=6)
    assert rec["pass"], rec


@pytest.mark.parametrize("negctl", ["stale", "flip"])
def test_negative_controls_turn_the_gate_red(negctl):
    rec = gate_cell_emulated(CellConfig(nranks=2, rows=128, dist="mags"), reps=3, negctl=negctl)
    assert not rec["pass"]
    assert rec["mism_first"] > 0 and rec["bad_calls_percall"] > 0 and rec["bad_graph_replays"] > 0


def test_alternating_rows_and_kinds_in_one_context():
    """Row counts, algorithms, inputs and epilogues alternate inside one context (one window, one call counter)."""
    g = EmulatedGroup(4, 512)
    dev = torch.device("cuda", 0)
    cells = [CellConfig(4, 512), CellConfig(4, 269, epilogue=1), CellConfig(4, 31, algo=0),
             CellConfig(4, 1), CellConfig(4, 300, input=N.IN_NVFP4), CellConfig(4, 512, epilogue=3)]
    prepared = [(c, make_inputs(c, i, dev), Outputs(c, dev, 4)) for i, c in enumerate(cells)]
    for _ in range(3):
        for c, inp, outs in prepared:
            outs.clear()
            g.launch([args_for(c, inp, outs, r, r) for r in range(4)])
            torch.cuda.synchronize()
            assert sum(mismatches(c, inp, outs, r) for r in range(4)) == 0, c
    assert g.status(0).ok
    g.close()


def test_modes_run_and_leave_the_window_armed():
    """Transport-only and compute-only modes are measurement modes: they must run, and a fused call after
    them must still be bit-exact (every slot they touched was re-armed)."""
    c = CellConfig(2, 200)
    g = EmulatedGroup(2, 200)
    dev = torch.device("cuda", 0)
    inp, outs = make_inputs(c, 0, dev), Outputs(c, dev, 2)
    for mode in (N.MODE_XPORT, N.MODE_FUSED, N.MODE_XPORT, N.MODE_FUSED):
        outs.clear()
        g.launch([args_for(c, inp, outs, r, r, mode=mode) for r in range(2)])
        torch.cuda.synchronize()
        if mode == N.MODE_FUSED:
            assert sum(mismatches(c, inp, outs, r) for r in range(2)) == 0
    assert g.status(0).ok
    g.close()


@pytest.mark.parametrize("P", [4, 8])
@pytest.mark.parametrize("lags", [33, 49, 50, 66, 67])
def test_two_shot_pipeline_depths(P, lags):
    """Every legal (owner lag, finish lag) pair gives the same bits; rows per team range from 0 to several."""
    for rows, epi in ((700, 0), (37, 1)):
        rec = gate_cell_emulated(CellConfig(nranks=P, rows=rows, epilogue=epi, lags=lags), reps=4, graph_calls=3, graph_reps=2)
        assert rec["pass"], (lags, rows, rec)


def test_norm_weight_bias_negative_control_turns_the_gate_red():
    """The fused-norm gate notices a weight bias that is off by 2^-7 (the reference's LN_NEGCTL control,
    bench/fused_norm/drv_norm.cu:188)."""
    rec = gate_cell_emulated(CellConfig(nranks=2, rows=96, epilogue=1), reps=3, graph_calls=2, graph_reps=2, negctl="bias")
    assert not rec["pass"]
    assert rec["mism_first"] > 0


@pytest.mark.parametrize("P", [4, 8])
@pytest.mark.parametrize("lags", [33, 50, 66, 67])
@pytest.mark.parametrize("inp,epi", [(N.IN_NVFP4, 0), (N.IN_NVFP4, 1), (N.IN_BF16, 2), (N.IN_NVFP4, 3)])
def test_two_shot_pipeline_depths_all_inputs_and_epilogues(P, lags, inp, epi):
    """Depth pairs x NVFP4 input x every epilogue with several rows per team (the record ring is one slot longer with
    NVFP4 input, and the quantised epilogues stage differently sized rows)."""
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=900, input=inp, epilogue=epi, lags=lags), reps=4, graph_calls=3,
                             graph_reps=2)
    assert rec["pass"], (P, lags, inp, epi, rec)


@pytest.mark.parametrize("P", [4, 8])
@pytest.mark.parametrize("tw", [3, 6])
@pytest.mark.parametrize("inp,epi", [(N.IN_BF16, 0), (N.IN_BF16, 1), (N.IN_BF16, 3), (N.IN_NVFP4, 0), (N.IN_NVFP4, 2)])
def test_both_team_widths_of_the_two_shot_shapes_are_bit_identical(P, tw, inp, epi):
    """Six-warp teams are the default of the two-shot shapes; the three-warp build of the same template stays selectable."""
    rec = gate_cell_emulated(CellConfig(nranks=P, rows=700, input=inp, epilogue=epi, team_warps=tw), reps=6, graph_calls=3,
                             graph_reps=2)
    assert rec["pass"], rec


def test_default_team_width_per_shape():
    lib = N.cuda()
    assert lib.fp4ar_default_team_warps(4, 1) == 6 and lib.fp4ar_default_team_warps(8, 1) == 6
    assert lib.fp4ar_default_team_warps(2, 0) == 3 and lib.fp4ar_default_team_warps(2, 1) == 3 and lib.fp4ar_default_team_warps(4, 0) == 3
