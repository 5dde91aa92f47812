"""Small host-side utilities: clock-sample summary, run-information fields, deterministic input generators."""
import numpy as np
import torch

from fp4_all_reduce_b200 import oracle as O
from fp4_all_reduce_b200.utils import data as D
from fp4_all_reduce_b200.utils.clocks import ClockSampler
from fp4_all_reduce_b200.utils.runinfo import run_info, sources_digest


def test_clock_summary_uses_busy_samples_and_collects_reasons():
    s = ClockSampler(0)
    # index, sm, max sm, power, active mask, hw_slowdown, hw_thermal, sw_thermal, sw_power_cap
    s._rows = [["0", "300", "1965", "120.0", "0x0", "Not Active", "Not Active", "Not Active", "Not Active"],
               ["0", "1950", "1965", "900.0", "0x4", "Not Active", "Not Active", "Not Active", "Active"],
               ["0", "1900", "1965", "950.0", "0x4", "Not Active", "Not Active", "Not Active", "Active"],
               ["0", "bad", "1965", "x", "", "", "", "", ""]]
    out = s.summary()
    assert out["sm_mhz"] == 1925.0 and out["sm_max_mhz"] == 1965.0 and out["power_w_max"] == 950.0
    assert out["reasons"] == ["sw_power_cap"] and out["samples"] == 3
    empty = ClockSampler(0)
    assert empty.summary() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    s._rows[1][6] = "Active"
    assert "hw_thermal_slowdown" in s.summary()["reasons"]


def test_run_info_fields():
    info = run_info()
    assert info["host"] and "time" in info and "torch" in info
    assert info["sources"] == sources_digest() and len(info["sources"]) == 16


def test_inputs_are_deterministic_and_ranks_differ():
    a, b = D.partial(64, 0), D.partial(64, 0)
    assert torch.equal(a, b) and a.dtype == torch.bfloat16 and a.shape == (64, 6144)
    assert not torch.equal(a, D.partial(64, 1))
    assert not torch.equal(a, D.partial(64, 0, seed_offset=1))
    sp = O.bf16_bits_to_f32(O.bf16_bits(D.special_rows(96, 0)))
    assert np.isnan(sp).any() or np.isinf(sp).any() or (np.abs(sp) > 1e30).any()      # the hostile classes are there
    assert (sp[0] == 0).all() or (sp == 0).all(axis=1).any()                          # and an all-zero row
    w = D.norm_weight()
    assert w.shape == (6144,) and abs(float(w.float().std()) - 0.02) < 0.005
