"""Verify-row budget planning: how many draft rows each stream gets in a decode round.

Every stream gets its base row; extra rows go one at a time to the stream whose next draft is worth most (the value of
the j-th draft is the probability that drafts 1..j are all accepted, so values fall along a stream and greedy is
optimal); the budget that maximises expected committed tokens per millisecond of a measured cost model is chosen in
one pass over the nested allocation order.  Behaviour parity: reference crates/sched/src/lib.rs:374-912 (Demand,
allocate, CostModel, choose_budget, StepCost, DraftCost, RoundCost, plan_round, TreeDemand, plan_trees,
adaptive_block); TREE_MAX_ROWS / ATTN_ROW_BLOCK (:743-747).
"""
from __future__ import annotations

import bisect
import math
from dataclasses import dataclass

TREE_MAX_ROWS = 64
ATTN_ROW_BLOCK = 8
MIN_DRAFT_BLOCK, MAX_DRAFT_BLOCK, DEEP_BLOCK_STREAMS = 8, 16, 8


def clean_accept(a: float) -> float:
    """An acceptance probability usable for ranking: NaN and negatives count as 0, above 1 as 1."""
    if a != a or a < 0:
        return 0.0
    return min(a, 1.0)


@dataclass
class Demand:
    """What one stream could use this step: values[j] = P(drafts 1..j+1 all accepted), non-increasing."""
    values: list
    kv_tokens: int = 0

    @staticmethod
    def geometric(accept: float, drafts: int) -> "Demand":
        a = clean_accept(accept)
        return Demand([a ** (j + 1) for j in range(drafts)])

    @staticmethod
    def from_conditional(conditional, drafts: int) -> "Demand":
        vals, p = [], 1.0
        for j in range(drafts):
            c = clean_accept(conditional[j] if j < len(conditional) else (conditional[-1] if conditional else 0.0))
            p *= c
            vals.append(p)
        return Demand(vals)

    def with_kv_tokens(self, kv_tokens: int) -> "Demand":
        self.kv_tokens = kv_tokens
        return self

    def marginal(self, j: int) -> float:
        return self.values[j] if j < len(self.values) else 0.0

    def expected_tokens(self, k: int) -> float:
        return 1.0 + sum(self.values[:k])


def expected_tokens(accept: float, d: int) -> float:
    a = clean_accept(accept)
    return sum(a ** j for j in range(d + 1))


def allocation_order(demands) -> list:
    """Entry r = the stream that receives the (r+1)-th extra row; ties go to the lower stream index."""
    heads = [0] * len(demands)
    order = []
    total = sum(len(d.values) for d in demands)
    for _ in range(total):
        best, bi = -1.0, -1
        for i, d in enumerate(demands):
            if heads[i] < len(d.values) and d.values[heads[i]] > best:
                best, bi = d.values[heads[i]], i
        if bi < 0 or best <= 0.0:
            break
        order.append(bi)
        heads[bi] += 1
    return order


def allocate(demands, budget_rows: int) -> list:
    """Drafts per stream for a row budget.  Below the stream count the tail gets none (and must not be stepped)."""
    n = len(demands)
    out = [0] * n
    extra = budget_rows - n
    if extra <= 0:
        return out
    for s in allocation_order(demands)[:extra]:
        out[s] += 1
    return out


class CostModel:
    """Measured step time as a function of the rows in the step: piecewise linear between points, last slope beyond."""

    def __init__(self, points):
        pts = sorted((int(r), float(ms)) for r, ms in points)
        if not pts:
            raise ValueError("cost table is empty")
        if any(r <= 0 for r, _ in pts) or any(not (ms > 0 and math.isfinite(ms)) for _, ms in pts):
            raise ValueError("cost table needs positive rows and finite positive times")
        if len({r for r, _ in pts}) != len(pts):
            raise ValueError("cost table repeats a row count")
        self.rows = [r for r, _ in pts]
        self.msv = [m for _, m in pts]

    def ms(self, rows: int) -> float:
        r = max(1, rows)
        if len(self.rows) == 1:
            return self.msv[0] * r / self.rows[0]
        i = bisect.bisect_left(self.rows, r)
        if i == 0:
            return self.msv[0]
        if i >= len(self.rows):
            i = len(self.rows) - 1
        r0, r1, m0, m1 = self.rows[i - 1], self.rows[i], self.msv[i - 1], self.msv[i]
        return m0 + (m1 - m0) * (r - r0) / (r1 - r0)

    def max_rows(self) -> int:
        return self.rows[-1]


def choose_budget(cost: CostModel, demands, max_rows: int):
    """(row budget, drafts per stream) maximising expected committed tokens per ms of the verify step."""
    n = len(demands)
    if n == 0:
        return 0, []
    order = allocation_order(demands)
    drafts = [0] * n
    tokens = float(n)
    best = (tokens / cost.ms(n), n, list(drafts))
    rows = n
    for s in order:
        if rows + 1 > max_rows:
            break
        tokens += demands[s].marginal(drafts[s])
        drafts[s] += 1
        rows += 1
        rate = tokens / cost.ms(rows)
        if rate > best[0] * (1 + 1e-12):
            best = (rate, rows, list(drafts))
    return best[1], best[2]


class StepCost:
    """Verify-step time by (rows, streams): one rows->ms curve per measured stream count, interpolated between stream
    counts and extended past the last by its slope."""

    def __init__(self, curves: dict):
        self.curves = dict(sorted(curves.items()))
        if not self.curves:
            raise ValueError("empty step-cost grid")

    @staticmethod
    def rows_only(rows: CostModel) -> "StepCost":
        return StepCost({1: rows})

    @staticmethod
    def from_grid(points) -> "StepCost":
        by = {}
        for rows, streams, ms in points:
            by.setdefault(int(streams), []).append((rows, ms))
        return StepCost({s: CostModel(p) for s, p in by.items()})

    def ms(self, rows: int, streams: int) -> float:
        keys = list(self.curves)
        if len(keys) == 1:
            return self.curves[keys[0]].ms(rows)
        i = bisect.bisect_left(keys, streams)
        if i < len(keys) and keys[i] == streams:
            return self.curves[streams].ms(rows)
        if i == 0:
            i = 1
        if i >= len(keys):
            i = len(keys) - 1
        s0, s1 = keys[i - 1], keys[i]
        m0, m1 = self.curves[s0].ms(rows), self.curves[s1].ms(rows)
        return max(1e-9, m0 + (m1 - m0) * (streams - s0) / (s1 - s0))


@dataclass
class DraftCost:
    layers: CostModel            # by drafting streams
    head: CostModel              # by head rows
    fixed_ms: float = 0.0

    def ms(self, drafting: int, head_rows: int) -> float:
        if drafting <= 0:
            return 0.0
        return self.fixed_ms + self.layers.ms(drafting) + (self.head.ms(head_rows) if head_rows > 0 else 0.0)


@dataclass
class RoundShape:
    rows: int
    streams: int
    drafting: int = 0
    head_rows: int = 0
    kv_tokens: int = 0           # context tokens read by the round's attention (sum over rows / ATTN_ROW_BLOCK groups)


@dataclass
class RoundCost:
    step: StepCost
    draft: DraftCost | None = None
    kv_ms_per_token: float = 0.0

    def ms(self, s: RoundShape, draft_sunk: bool) -> float:
        t = self.step.ms(s.rows, s.streams) + self.kv_ms_per_token * s.kv_tokens
        if not draft_sunk and self.draft is not None:
            t += self.draft.ms(s.drafting, s.head_rows)
        return t


@dataclass
class Plan:
    drafts: list
    rows: int
    expected_tokens: float
    ms: float

    @property
    def rate(self) -> float:
        return self.expected_tokens / self.ms if self.ms > 0 else 0.0


def plan_round(cost: RoundCost, demands, max_rows: int, draft_sunk: bool) -> Plan:
    """The cheapest-per-token round among the nested greedy allocations.  With draft_sunk False the draft's own cost is
    counted, so the plan can be made BEFORE drafting (a plan with no drafts needs no draft round at all)."""
    n = len(demands)
    if n == 0:
        return Plan([], 0, 0.0, 0.0)
    order = allocation_order(demands)
    drafts = [0] * n
    tokens = float(n)

    def shape():
        kv = sum(d.kv_tokens * -(-(1 + k) // ATTN_ROW_BLOCK) for d, k in zip(demands, drafts))
        return RoundShape(n + sum(drafts), n, sum(1 for k in drafts if k > 0), sum(drafts), kv)

    ms = cost.ms(shape(), draft_sunk)
    best = Plan(list(drafts), n, tokens, ms)
    for s in order:
        if n + sum(drafts) + 1 > max_rows:
            break
        tokens += demands[s].marginal(drafts[s])
        drafts[s] += 1
        ms = cost.ms(shape(), draft_sunk)
        if tokens / ms > best.rate * (1 + 1e-12):
            best = Plan(list(drafts), n + sum(drafts), tokens, ms)
    return best


@dataclass
class TreeDemand:
    """Per-node probabilities of lying on the accepted path, in the order the tree search popped the nodes."""
    values: list
    kv_tokens: int = 0

    def expected_tokens(self, k: int) -> float:
        return 1.0 + sum(self.values[:k])


def plan_trees(cost: RoundCost, demands, max_rows: int) -> Plan:
    cap = min(max_rows, max(TREE_MAX_ROWS, len(demands)))
    return plan_round(cost, [Demand(list(d.values), d.kv_tokens) for d in demands], cap, True)


def adaptive_block(kept: int, last_level_kept: bool, streams: int) -> int:
    """Rows the draft block should run next round: the depth just kept plus a margin, inside [8, 16]; many streams fall
    back to the trained 8."""
    if streams > DEEP_BLOCK_STREAMS:
        return MIN_DRAFT_BLOCK
    want = kept + (5 if last_level_kept else 2)
    return max(MIN_DRAFT_BLOCK, min(MAX_DRAFT_BLOCK, want))
