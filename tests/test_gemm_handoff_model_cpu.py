"""The partial-tile hand-off of the stream-K GEMM under a random scheduler (no GPU): the product rules are safe over
overlapping launches, and removing either rule is caught."""
import pytest

from fp4_all_reduce_b200.harness import gemm_handoff_model as M


@pytest.mark.parametrize("units,launches", [(2, 4), (5, 3), (8, 6)])
def test_product_rules_are_safe(units, launches):
    assert M.check(units, launches, seeds=150) == 0


@pytest.mark.parametrize("variant", ["no_free_wait", "early_reset"])
def test_a_missing_rule_is_caught(variant):
    assert M.check(6, 6, seeds=150, variant=variant) > 0
