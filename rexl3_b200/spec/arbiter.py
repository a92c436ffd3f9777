"""Draft-source selection for speculative rounds.

Each decode round, every stream can have its window filled from one of three sources: the backend's own draft head
("native"), the n-gram copy drafter ("copy"), or nothing.  This module picks the source and the draft count that
maximise committed tokens per millisecond of model time, from two inputs only: the cost figures the caller supplies
(what a draft step and a verify row cost) and the acceptance outcomes it reports back.  Acceptance is tracked per
draft depth as an exponentially decayed accept/offer ratio seeded with a prior, so a drafter that stops working
loses its slot within a few rounds; a source that is currently not chosen is still tried every so often (the probe
interval doubles each time a probe loses) so that a recovered drafter is noticed.  No GPU, no clock: everything
here is a pure function of its arguments and runs in the CPU tests.

Same role as the reference's crates/spec/src/arbiter.rs:27-130 (choice type, per-depth curve) and :255-394
(selection, feedback, probing).
"""
from __future__ import annotations

from dataclasses import dataclass, field

MAX_DEPTH = 8


@dataclass(frozen=True)
class Choice:
    kind: str = "none"      # "none" | "copy" | "native"
    n: int = 0

    def drafts(self) -> int:
        return 0 if self.kind == "none" else self.n


NONE = Choice()


class DepthCurve:
    """Conditional acceptance of the j-th draft given the j-1 before it were accepted, as a decayed ratio with a prior."""

    def __init__(self, prior, weight: float = 4.0, decay: float = 0.95, chain: float | None = None, fade: float = 1.0):
        if not prior or weight <= 0 or not 0 <= decay <= 1:
            raise ValueError("bad depth-curve parameters")
        self.prior = [prior[j] if j < len(prior) else prior[-1] * 0.95 ** (j + 1 - len(prior)) for j in range(MAX_DEPTH)]
        self.hits = [0.0] * MAX_DEPTH
        self.trials = [0.0] * MAX_DEPTH
        self.weight, self.decay, self.chain, self.fade = weight, decay, chain, fade

    def alpha(self, j: int) -> float:
        i = min(max(j, 1), MAX_DEPTH) - 1
        prior = self.alpha(i) * self.chain if (self.chain is not None and i > 0) else self.prior[i]
        return min(max((self.hits[i] + prior * self.weight) / (self.trials[i] + self.weight), 0.0), 0.999)

    def expected_tokens(self, d: int) -> float:
        s, p = 1.0, 1.0
        for j in range(1, d + 1):
            p *= self.alpha(j)
            s += p
        return s

    def conditional(self, d: int):
        return [self.alpha(j) for j in range(1, d + 1)]

    def observe(self, verified: int, accepted: int) -> None:
        v = min(verified, MAX_DEPTH)
        for j in range(1, v + 1):
            if accepted + 1 >= j:
                i = j - 1
                self.hits[i] = self.hits[i] * self.decay + (1.0 if accepted >= j else 0.0)
                self.trials[i] = self.trials[i] * self.decay + 1.0
        for i in range(v, MAX_DEPTH):
            self.hits[i] *= self.fade
            self.trials[i] *= self.fade


@dataclass
class StreamState:
    copy: DepthCurve
    native: DepthCurve
    since: dict = field(default_factory=lambda: {"copy": 0, "native": 0})
    gap: dict = field(default_factory=dict)


class Arbiter:
    """verify_ms(streams, rows) and native_ms(drafting streams, head rows) are callables supplied by the backend's cost tables."""

    def __init__(self, verify_ms, native_ms=None, probe_every: int = 16, probe_max_gap: int = 256, copy_prior=(0.55, 0.7, 0.75),
                 native_prior=(0.7, 0.6, 0.5)):
        self.verify_ms, self.native_ms = verify_ms, native_ms or (lambda drafting, rows: 0.0)
        self.probe_every, self.probe_max_gap = probe_every, probe_max_gap
        self.copy_prior, self.native_prior = copy_prior, native_prior
        self.streams = {}

    def state(self, sid) -> StreamState:
        st = self.streams.get(sid)
        if st is None:
            st = StreamState(DepthCurve(self.copy_prior, chain=0.9, fade=0.98), DepthCurve(self.native_prior, chain=0.9, fade=0.98))
            st.gap = {"copy": self.probe_every, "native": self.probe_every}
            self.streams[sid] = st
        return st

    def forget(self, sid) -> None:
        self.streams.pop(sid, None)

    def _rate(self, picks, offers) -> float:
        rows = len(picks) + sum(c.drafts() for c in picks.values())
        tokens = 0.0
        nat_streams = nat_rows = 0
        for sid, c in picks.items():
            st = self.state(sid)
            if c.kind == "copy":
                tokens += st.copy.expected_tokens(c.n)
            elif c.kind == "native":
                tokens += st.native.expected_tokens(c.n)
                nat_streams += 1
                nat_rows += c.n
            else:
                tokens += 1.0
        ms = self.verify_ms(len(picks), rows) + (self.native_ms(nat_streams, nat_rows) if nat_streams else 0.0)
        return tokens / max(ms, 1e-9)

    def choose(self, offers: dict, max_rows: int) -> dict:
        """offers: sid -> dict(copy=len of the copy proposal, native=max depth the head offers).  Returns sid -> Choice.

        Coordinate ascent from "nobody drafts": every step changes one stream's pick to the one that raises the round's
        rate most, until none does (deterministic; ties go to fewer rows).  Streams due for a probe get a one-deep probe.
        """
        picks = {sid: NONE for sid in offers}
        while True:
            base = self._rate(picks, offers)
            best = (base * (1 + 1e-9), None, None)
            rows_now = len(picks) + sum(c.drafts() for c in picks.values())
            for sid, off in offers.items():
                cur = picks[sid]
                cands = [Choice("copy", n) for n in range(1, off.get("copy", 0) + 1)] + \
                        [Choice("native", n) for n in range(1, off.get("native", 0) + 1)]
                for c in cands:
                    if c == cur or rows_now - cur.drafts() + c.drafts() > max_rows:
                        continue
                    picks[sid] = c
                    r = self._rate(picks, offers)
                    picks[sid] = cur
                    if r > best[0] or (r == best[0] and best[2] is not None and c.drafts() < best[2].drafts()):
                        best = (r, sid, c)
            if best[1] is None:
                break
            picks[best[1]] = best[2]
        # probing: a source not verified for `gap` rounds gets a cheap one-deep try
        rows_now = len(picks) + sum(c.drafts() for c in picks.values())
        for sid, off in offers.items():
            st = self.state(sid)
            if picks[sid].kind != "none":
                continue
            for src in ("native", "copy"):
                if off.get(src, 0) >= 1 and st.since[src] >= st.gap[src] and rows_now + 1 <= max_rows:
                    picks[sid] = Choice(src, 1)
                    rows_now += 1
                    break
        return picks

    def observe(self, sid, choice: Choice, accepted: int) -> None:
        st = self.state(sid)
        for src in ("copy", "native"):
            if choice.kind == src:
                curve = st.copy if src == "copy" else st.native
                was_probe = choice.n == 1 and st.since[src] >= st.gap[src]
                curve.observe(choice.n, accepted)
                st.since[src] = 0
                if was_probe:
                    st.gap[src] = self.probe_every if accepted >= 1 else min(self.probe_max_gap, st.gap[src] * 2)
            else:
                st.since[src] += 1
