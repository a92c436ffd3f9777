"""The low-rank selector of a block drafter: which of a position's candidates follows the token picked before it.

A block drafter proposes T positions at once from one hidden state, so position p's candidates cannot see which token was picked at p - 1.
The selector adds that coupling afterwards: score(c) = unary[p][c] + sum_r pred[prev][r] * hidden[p][r] * succ[c][r], with `pred` / `succ`
two rank-r codebooks over the vocabulary and `hidden[p]` the draft's hidden state projected to the rank.  `selector_walk` picks one path
(greedy, or with the target's keyed noise so that the draft matches the target wherever the two distributions agree); `selector_lattice`
puts the same scores into a `spec.tree.Lattice` with per-parent edge terms, over which `best_first` grows a draft tree whose deeper
candidates are conditioned on their own parent.

Behaviour parity: reference crates/spec/src/lib.rs:207-300 (SelectorInputs, SelectorError, try_selector_walk, Walk::{Greedy, Keyed}).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..sampling import Sampling, SamplingError, choose
from .tree import Lattice


class SelectorError(ValueError):
    """Ragged inputs (`kind` = "shape") or a position without candidates / with a NaN score (`kind` = "sampling")."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"selector {'inputs' if kind == 'shape' else 'scoring'}: {message}")
        self.kind = kind


@dataclass
class SelectorInputs:
    candidates: list          # per position: candidate token ids
    unary: list               # per position: the draft head's logits of those candidates
    hidden: list              # per position: the draft hidden state projected to the rank, float [rank]
    predecessor: object       # callable(token id) -> float [rank]
    successor: object         # callable(token id) -> float [rank]


def _check(x: SelectorInputs) -> int:
    t = len(x.candidates)
    if len(x.unary) != t or len(x.hidden) != t:
        raise SelectorError("shape", f"{t} candidate lists, {len(x.unary)} unary rows, {len(x.hidden)} hidden rows")
    for p in range(t):
        if len(x.candidates[p]) != len(x.unary[p]):
            raise SelectorError("shape", f"position {p}: {len(x.candidates[p])} candidates but {len(x.unary[p])} unary scores")
    return t


def _scores(x: SelectorInputs, p: int, prev: int) -> list:
    a = np.asarray(x.predecessor(prev), dtype=np.float32)
    h = np.asarray(x.hidden[p], dtype=np.float32)
    if a.shape != h.shape:
        raise SelectorError("shape", f"position {p}: predecessor rank {a.size} but hidden rank {h.size}")
    ah = a * h
    out = []
    for c, u in zip(x.candidates[p], x.unary[p]):
        b = np.asarray(x.successor(int(c)), dtype=np.float32)
        if b.shape != ah.shape:
            raise SelectorError("shape", f"position {p}: successor rank {b.size} but hidden rank {ah.size}")
        acc = np.float32(0.0)
        for bb, aa in zip(b, ah):                   # summed in index order, in float32, as the walk on the device sums it
            acc = np.float32(acc + np.float32(bb * aa))
        out.append(float(np.float32(np.float32(u) + acc)))
    return out


def selector_walk(anchor: int, x: SelectorInputs, sampling: Sampling | None = None, first_position: int = 0) -> list:
    """One path from the verified anchor.  sampling None: greedy (highest score, ties to the lowest id).  Otherwise position p is drawn with
    the keyed sampler at absolute position first_position + p over all of its candidates, i.e. with the noise the target will use there."""
    t = _check(x)
    prev, path = int(anchor), []
    for p in range(t):
        scores = _scores(x, p, prev)
        s = Sampling(temperature=0.0, top_k=max(1, len(scores)), top_p=1.0) if sampling is None else \
            Sampling(seed=sampling.seed, temperature=sampling.temperature, top_k=max(1, len(scores)), top_p=sampling.top_p, min_p=sampling.min_p)
        try:
            if not scores:
                raise SamplingError("no candidates")
            tok = choose(scores, x.candidates[p], 0 if sampling is None else first_position + p, s)
        except SamplingError as e:
            raise SelectorError("sampling", f"position {p}: {e}")
        path.append(int(tok))
        prev = int(tok)
    return path


def selector_lattice(anchor: int, x: SelectorInputs) -> Lattice:
    """The selector's scores as a lattice for the tree search: unary per level, and edge[level][parent index][candidate index] = the coupling
    of a candidate with each possible parent (level 0's only parent is the anchor).  With Policy(edge=1, scale=1) a node's score is the
    walk's score given its own parent."""
    t = _check(x)
    edge = []
    for p in range(t):
        parents = [int(anchor)] if p == 0 else [int(c) for c in x.candidates[p - 1]]
        rows = []
        for prev in parents:
            sc = _scores(x, p, prev)
            rows.append([float(np.float32(s - np.float32(u))) for s, u in zip(sc, x.unary[p])])
        edge.append(rows)
    return Lattice([[int(c) for c in row] for row in x.candidates], [[float(u) for u in row] for row in x.unary], edge)
