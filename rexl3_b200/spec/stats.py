"""Speculation telemetry: what each draft position bought, and how well the drafter's own confidence predicts acceptance.

Per draft position j (0 = the draft right after the token being fed) and per population (greedy / sampled requests):
`offered` (the drafter produced it), `verified` (a row of the target forward was spent on it), `reached` (every earlier draft was accepted,
so it was tested against the target's sample), `accepted`.  accepted / reached is the conditional acceptance a budget needs;
offered - reached is draft work that could not count; verified - reached is verify rows computed and thrown away.

`MarginBins` keeps, per bin of the draft's margin (how far its pick leads the runner-up, in logits), how many picks were tested and how
many were accepted; `probability(margin)` is the smoothed ratio, which the `margin` / `scored` budget policies use as the pick's
confidence when the drafter gives none of its own.

Behaviour parity: reference crates/spec/src/stats.rs:1-80 (PositionStats, Mode, CONF_BINS), crates/spec/src/measured.rs (the frozen
priors this module's `snapshot()` / `from_snapshot()` stand for: a table measured on one deployment seeds the next).
"""
from __future__ import annotations

MAX_POSITIONS = 16
MARGIN_BINS = 32
MARGIN_WIDTH = 0.5
MODES = ("greedy", "sampled")


def mode_of(sampling) -> str:
    return "greedy" if sampling is None or sampling.temperature == 0.0 else "sampled"


class PositionStats:
    def __init__(self):
        self.rounds = 0
        self.offered = [0] * MAX_POSITIONS
        self.verified = [0] * MAX_POSITIONS
        self.reached = [0] * MAX_POSITIONS
        self.accepted = [0] * MAX_POSITIONS

    def record(self, offered: int, verified: int, accepted: int) -> None:
        """One sequence-round: the drafter offered `offered` drafts, `verified` of them rode in the window, the first `accepted` matched."""
        if not accepted <= verified <= offered:
            raise ValueError(f"accepted {accepted} verified {verified} offered {offered}")
        self.rounds += 1
        reached = min(verified, accepted + 1)
        for j in range(min(offered, MAX_POSITIONS)):
            self.offered[j] += 1
            self.verified[j] += 1 if j < verified else 0
            self.reached[j] += 1 if j < reached else 0
            self.accepted[j] += 1 if j < accepted else 0

    def conditional(self, prior: float = 0.7, weight: float = 8.0) -> list:
        """Smoothed accepted / reached per position."""
        return [(a + prior * weight) / (r + weight) for a, r in zip(self.accepted, self.reached)]

    def wasted_rows(self) -> int:
        return sum(v - r for v, r in zip(self.verified, self.reached))

    def snapshot(self) -> dict:
        return dict(rounds=self.rounds, offered=list(self.offered), verified=list(self.verified), reached=list(self.reached), accepted=list(self.accepted))


class MarginBins:
    def __init__(self, prior: float = 0.6, weight: float = 4.0):
        self.reached = [0] * MARGIN_BINS
        self.accepted = [0] * MARGIN_BINS
        self.prior, self.weight = prior, weight

    @staticmethod
    def bin(margin: float) -> int:
        if not margin == margin or margin <= 0:
            return 0
        return min(MARGIN_BINS - 1, int(margin / MARGIN_WIDTH))

    def record(self, margins, verified: int, accepted: int) -> None:
        """margins[j] of the picks that rode in the window; pick j was tested when picks 0..j-1 were accepted."""
        for j in range(min(verified, accepted + 1, len(margins))):
            b = self.bin(margins[j])
            self.reached[b] += 1
            self.accepted[b] += 1 if j < accepted else 0

    def probability(self, margin: float) -> float:
        """Smoothed acceptance of a pick with this margin.  Bins with little data lean on their neighbours below (a larger margin is never
        taken to be less certain than a smaller one that was measured)."""
        b = self.bin(margin)
        p = (self.accepted[b] + self.prior * self.weight) / (self.reached[b] + self.weight)
        lo = max(((self.accepted[i] + self.prior * self.weight) / (self.reached[i] + self.weight) for i in range(b) if self.reached[i] >= 8 * self.weight),
                 default=0.0)
        return min(0.999, max(p, lo if self.reached[b] < 8 * self.weight else 0.0))

    def confidences(self, margins) -> list:
        return [self.probability(m) for m in margins]

    def snapshot(self) -> dict:
        return dict(reached=list(self.reached), accepted=list(self.accepted))

    @staticmethod
    def from_snapshot(doc: dict, prior: float = 0.6, weight: float = 4.0) -> "MarginBins":
        m = MarginBins(prior, weight)
        if len(doc.get("reached", [])) != MARGIN_BINS or len(doc.get("accepted", [])) != MARGIN_BINS:
            raise ValueError(f"a margin table has {MARGIN_BINS} bins")
        m.reached, m.accepted = [int(x) for x in doc["reached"]], [int(x) for x in doc["accepted"]]
        if any(a > r or a < 0 for a, r in zip(m.accepted, m.reached)):
            raise ValueError("a margin table cannot hold more accepted than tested picks")
        return m
