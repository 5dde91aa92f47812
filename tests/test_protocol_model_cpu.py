"""Randomised model check of the window hand-off protocol (two buffers, consumer-side re-arm, stores that land
late and out of order, ranks at arbitrary speeds).  The rules of the product never violate an invariant; taking
one rule away does; a rank that stops pushing makes the others give up instead of hanging."""
import pytest

from fp4_all_reduce_b200.harness.protocol_model import Model, check


@pytest.mark.parametrize("P", [2, 4, 8])
@pytest.mark.parametrize("two_shot,lo,lf", [(False, 0, 1), (True, 1, 2), (True, 2, 3), (True, 2, 4), (True, 3, 4)])
def test_product_rules_are_safe(P, two_shot, lo, lf):
    for rows in (1, 2, 3, 6):
        r = check(P, rows, 5, two_shot=two_shot, lag_o=lo, lag_f=lf, seeds=24 if P == 8 else 40)
        assert r["violations"] == 0, (rows, r["first"])


@pytest.mark.parametrize("variant", ["one_buffer", "no_drain"])
@pytest.mark.parametrize("two_shot,lo,lf", [(False, 0, 1), (True, 1, 2)])
def test_a_missing_rule_is_caught(variant, two_shot, lo, lf):
    r = check(2, 1, 6, two_shot=two_shot, lag_o=lo, lag_f=lf, seeds=150, variant=variant)
    assert r["violations"] > 0
    assert "landed on unconsumed" in r["first"] or "consumed" in r["first"] or "re-arm" in r["first"]


@pytest.mark.parametrize("two_shot", [False, True])
def test_a_rank_that_stops_pushing_ends_in_bounded_waits(two_shot):
    m = Model(4, 4, 3, two_shot=two_shot, lag_o=2, lag_f=3, seed=3, dead_rank=2, dead_call=1, wait_limit=300)
    out = m.run()
    assert out["gave_up"] > 0                     # the survivors' waits ran into their limit and were reported
    assert all(rank != 2 for rank, _call, _slot in m.gave_up)
    assert all(call >= 1 for _rank, call, _slot in m.gave_up)     # the call before the failure completed normally


@pytest.mark.parametrize("two_shot,lo,lf", [(False, 0, 1), (True, 1, 2)])
def test_a_call_without_exchange_must_not_advance_the_call_counter(two_shot, lo, lf):
    """Zero-row calls between real calls: safe when they launch nothing (what the runtime does), caught when they
    would flip the buffer parity without any rank having waited for its peers."""
    bad = check(2, 1, 7, two_shot=two_shot, lag_o=lo, lag_f=lf, seeds=150, variant="empty_call_bumps")
    assert bad["violations"] > 0, bad
    good = check(2, 1, 7, two_shot=two_shot, lag_o=lo, lag_f=lf, seeds=150, variant="empty_call_skipped")
    assert good["violations"] == 0, good["first"]
