"""GPU-free speculation logic: acceptance rule, acceptance statistics, copy (n-gram suffix) drafter, spec modes,
keyed draft pick.

A draft is accepted iff it equals the keyed sample at its position, so speculation changes speed and never an output
byte.  Behaviour parity: reference crates/spec/src/lib.rs:33-35 (accept), :37-78 (AcceptStats), :79-205 (CopyDrafter:
min_match 8, max_draft 7, KEEP_PER_GRAM 64, SCAN 32), crates/spec/src/mode.rs:9-35, crates/spec/src/draft_pick.rs:23-63.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..sampling import Sampling, choose

KEEP_PER_GRAM = 64
SCAN = 32


def accept(drafts, samples) -> int:
    """Number of drafts accepted: longest prefix with drafts[i] == samples[i]; committed tokens are samples[:a+1]."""
    a = 0
    for d, s in zip(drafts, samples):
        if d != s:
            break
        a += 1
    return a


class AcceptStats:
    """Exponentially weighted acceptance per successive draft; each proposed position is a Bernoulli trial until the first rejection."""

    def __init__(self, prior: float = 0.6, prior_trials: float = 4.0, decay: float = 0.9):
        self.hits = prior * prior_trials
        self.trials = prior_trials
        self.decay = decay
        self.prior_hits, self.prior_trials = self.hits, prior_trials

    def relax(self) -> None:
        """A round with no drafts for this stream: drift back toward the prior, so a stream budgeted zero drafts is tried again."""
        keep = 1.0 - self.decay
        self.hits = self.hits * self.decay + self.prior_hits * keep
        self.trials = self.trials * self.decay + self.prior_trials * keep

    def accept_rate(self) -> float:
        return 0.0 if self.trials <= 0 else min(max(self.hits / self.trials, 0.0), 0.999)

    def update(self, proposed: int, accepted: int) -> None:
        if proposed == 0:
            return
        trials = accepted + (1 if accepted < proposed else 0)
        self.hits = self.hits * self.decay + accepted
        self.trials = self.trials * self.decay + trials


def _gram_hash(g) -> int:
    h = 0xCBF29CE484222325
    for t in g:
        h = ((h ^ (t & 0xFFFFFFFF)) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


class CopyDrafter:
    """Copy-window drafter: continue the longest earlier match of the context's suffix (prompt lookup), indexed incrementally."""

    def __init__(self, min_match: int = 8, max_draft: int = 7):
        if min_match <= 0:
            raise ValueError("min_match must be positive")
        self.min_match, self.max_draft = min_match, max_draft
        self.index = {}
        self.indexed = 0

    def extend(self, tokens) -> None:
        n = self.min_match
        if len(tokens) + 1 < self.indexed:  # the sequence got shorter: reused for another one
            self.index.clear()
            self.indexed = 0
        for end in range(max(self.indexed, n), len(tokens) + 1):
            ends = self.index.setdefault(_gram_hash(tokens[end - n:end]), [])
            ends.append(end)
            if len(ends) > KEEP_PER_GRAM:
                del ends[:len(ends) - KEEP_PER_GRAM]
        self.indexed = len(tokens) + 1

    def _best(self, at, length: int, limit: int):
        n = self.min_match
        key = [at(i) for i in range(length - n, length)]
        ends = self.index.get(_gram_hash(key))
        if not ends:
            return None
        best = None
        seen = 0
        for end in reversed(ends):
            if end >= limit:
                continue
            if seen >= SCAN:
                break
            seen += 1
            if any(at(end - n + i) != key[i] for i in range(n)):
                continue  # hash collision
            m = n
            while m < end and m < 256 and at(end - 1 - m) == at(length - 1 - m):
                m += 1
            if best is None or m > best[0]:
                best = (m, end)
        return best

    def propose(self, tokens, max_tokens: int):
        n, length = self.min_match, len(tokens)
        mx = min(max_tokens, self.max_draft)
        if length < n + 1 or mx <= 0:
            return []
        self.extend(tokens)
        best = self._best(lambda i: tokens[i], length, length)
        if best is None:
            return []
        end = best[1]
        return list(tokens[end:min(length, end + mx)])

    def propose_after(self, committed, extra, max_tokens: int):
        """Copy branch of a draft tree: match the suffix of committed + extra; only `committed` is ever indexed."""
        n = self.min_match
        length = len(committed) + len(extra)
        if length < n + 1 or max_tokens <= 0:
            return 0, []
        self.extend(committed)
        at = lambda i: committed[i] if i < len(committed) else extra[i - len(committed)]  # noqa: E731
        best = self._best(at, length, len(committed))
        if best is None:
            return 0, []
        m, end = best
        return m, [at(i) for i in range(end, min(length, end + max_tokens))]


class NgramDrafter:
    """Statistical n-gram drafter over the sequence's own text (prompt and output so far): for the longest context order that has been
    seen (down from `order` - 1 tokens to 1), propose the continuation that followed it most often (ties: the most recent), token by token.
    Complements the copy drafter: it needs no long exact match, so it fires on short repeated patterns (lists, code idioms, formats).
    Indexed incrementally like the copy drafter; only committed tokens are ever indexed."""

    def __init__(self, order: int = 4, max_draft: int = 7, min_count: int = 2):
        if order < 2:
            raise ValueError("order must be at least 2")
        self.order, self.max_draft, self.min_count = order, max_draft, min_count
        self.tables = [dict() for _ in range(order)]      # tables[k]: k-token context -> {next token: [count, last position]}
        self.indexed = 0

    def extend(self, tokens) -> None:
        if len(tokens) < self.indexed:                     # the sequence got shorter: reused for another one
            self.tables = [dict() for _ in range(self.order)]
            self.indexed = 0
        for pos in range(max(self.indexed, 1), len(tokens)):
            nxt = tokens[pos]
            for k in range(1, self.order):
                if pos - k < 0:
                    break
                ent = self.tables[k].setdefault(tuple(tokens[pos - k:pos]), {}).setdefault(nxt, [0, 0])
                ent[0] += 1
                ent[1] = pos
        self.indexed = len(tokens)

    def _next(self, ctx):
        for k in range(min(self.order - 1, len(ctx)), 0, -1):
            cand = self.tables[k].get(tuple(ctx[-k:]))
            if not cand:
                continue
            tok, (count, _last) = max(cand.items(), key=lambda kv: (kv[1][0], kv[1][1]))
            if count >= self.min_count:
                return tok
        return None

    def propose(self, tokens, max_tokens: int):
        mx = min(max_tokens, self.max_draft)
        if mx <= 0 or len(tokens) < 2:
            return []
        self.extend(tokens)
        ctx, out = list(tokens[-(self.order - 1):]), []
        for _ in range(mx):
            t = self._next(ctx)
            if t is None:
                break
            out.append(t)
            ctx = (ctx + [t])[-(self.order - 1):]
        return out


SPEC_MODES = ("auto", "mtp", "copy", "ngram", "self", "none")


@dataclass(frozen=True)
class SpecMode:
    name: str = "auto"

    def __post_init__(self):
        if self.name not in SPEC_MODES:
            raise ValueError(f"--spec must be one of {'|'.join(SPEC_MODES)}, got {self.name!r}")

    @property
    def native(self) -> bool:
        return self.name in ("auto", "mtp", "self")

    @property
    def copy(self) -> bool:
        return self.name in ("auto", "copy")

    @property
    def ngram(self) -> bool:
        """The n-gram drafter takes over where the copy drafter offers nothing ("auto"), or is the only host drafter ("ngram")."""
        return self.name in ("auto", "ngram")

    @property
    def enabled(self) -> bool:
        return self.name != "none"


def draft_pick(values, ids, position: int, sampling: Sampling | None) -> int:
    """A drafter's pick at `position`: greedy when `sampling` is None or T == 0, else the keyed choice with the TARGET's
    noise at that position, so the draft agrees with the target wherever their kept candidates agree (Gumbel-max coupling)."""
    if sampling is None or sampling.temperature == 0.0:
        best = 0
        for i in range(1, len(values)):
            if values[i] > values[best] or (values[i] == values[best] and ids[i] < ids[best]):
                best = i
        return int(ids[best])
    return choose(values, ids, position, sampling)
