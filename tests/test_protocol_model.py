"""Exhaustive interleaving check of the push-based collective protocol (slot sets, tickets, packets or data + flag)."""
import pytest

from rexl3_b200.parallel.protocol_model import Protocol, explore


@pytest.mark.parametrize("p", [Protocol(ranks=2, collectives=5, sets=2), Protocol(ranks=3, collectives=3, sets=2),
                               Protocol(ranks=2, collectives=4, sets=2, flags=True), Protocol(ranks=3, collectives=2, sets=2, flags=True),
                               Protocol(ranks=2, collectives=4, sets=3), Protocol(ranks=4, collectives=3, sets=2)])
def test_two_slot_sets_are_safe_under_every_interleaving(p):
    assert explore(p) is None


def test_one_slot_set_has_a_write_after_read_hazard():
    bad = explore(Protocol(ranks=2, collectives=3, sets=1))
    assert bad is not None and ("holds ticket" in bad[0] or "later ticket" in bad[0])
    # the trace ends with the failing step and is a real schedule: it starts with somebody's first push
    assert bad[1][0][1][0] == "packet" and bad[1][-1][1][0] in ("read", "wait")


def test_flag_before_data_is_caught():
    bad = explore(Protocol(ranks=2, collectives=2, sets=2, flags=True, flag_first=True))
    assert bad is not None and "reads source" in bad[0]
