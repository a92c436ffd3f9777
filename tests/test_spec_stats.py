"""Speculation telemetry: per-position counters, margin bins, and the margin-made confidences in the step loop."""
import pytest

from rexl3_b200.engine import Engine, MockBackend, MockOptions, generate, harness
from rexl3_b200.sampling import GREEDY
from rexl3_b200.spec import MarginBins, PositionStats


def test_position_stats_columns():
    ps = PositionStats()
    ps.record(4, 3, 1)          # 4 offered, 3 rode, the first matched: the second was tested and failed, the third was never reached
    assert ps.offered[:5] == [1, 1, 1, 1, 0] and ps.verified[:4] == [1, 1, 1, 0] and ps.reached[:4] == [1, 1, 0, 0] and ps.accepted[:3] == [1, 0, 0]
    ps.record(2, 2, 2)
    assert ps.reached[:3] == [2, 2, 0] and ps.accepted[:3] == [2, 1, 0] and ps.rounds == 2 and ps.wasted_rows() == 1
    c = ps.conditional(prior=0.5, weight=2.0)
    assert abs(c[0] - (2 + 1) / (2 + 2)) < 1e-9 and abs(c[1] - (1 + 1) / (2 + 2)) < 1e-9 and abs(c[5] - 0.5) < 1e-9
    with pytest.raises(ValueError):
        ps.record(2, 3, 1)


def test_margin_bins_learn_and_round_trip():
    mb = MarginBins(prior=0.6, weight=4.0)
    assert mb.bin(-1) == 0 and mb.bin(0.49) == 0 and mb.bin(0.5) == 1 and mb.bin(1e9) == 31 and mb.bin(float("nan")) == 0
    assert abs(mb.probability(3.0) - 0.6) < 1e-9
    for _ in range(200):
        mb.record([6.0, 0.2, 6.0], 3, 1)        # the sure first pick lands, the unsure second fails, the third is never tested
    assert mb.probability(6.0) > 0.97 and mb.probability(0.2) < 0.05
    assert mb.reached[12] == 200 and mb.reached[0] == 200 and mb.accepted[0] == 0
    assert mb.probability(9.0) > 0.9            # no data above: never less sure than a measured smaller lead
    again = MarginBins.from_snapshot(mb.snapshot())
    assert again.probability(6.0) == mb.probability(6.0)
    with pytest.raises(ValueError):
        MarginBins.from_snapshot({"reached": [1] * 32, "accepted": [2] * 32})


def test_margins_become_confidences_under_the_scored_policy():
    """A drafter that reports margins only (a wrong pick has a small lead): after a few rounds the bins say so, and `scored` stops spending
    scarce verify rows (four streams, room for five drafts) behind an unsure pick; output equals the serial run and the per-position counters show fewer wasted rows than `legacy`."""
    p = harness.default_prompts(512, (5, 9, 14, 33))
    serial = generate(Engine(MockBackend(MockOptions()), spec="none"), p, 80, GREEDY)
    wasted = {}
    for policy in ("legacy", "scored"):
        eng = Engine(MockBackend(MockOptions(native_draft=True, margins=True, draft_error=0.4)), spec="self", max_drafts=4, budget_policy=policy, window_rows=9)
        assert generate(eng, p, 80, GREEDY) == serial
        ps = eng.position_stats["greedy"]
        assert ps.rounds > 0 and sum(ps.accepted) == eng.counters["accepted"]
        wasted[policy] = ps.wasted_rows() / max(1, sum(ps.verified))
        assert eng.margin_bins.probability(6.0) > 0.9 and eng.margin_bins.probability(0.2) < 0.2
    assert wasted["scored"] < wasted["legacy"] * 0.7, wasted
