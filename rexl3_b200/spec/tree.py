"""Draft trees: best-first search over a drafter's candidate lattice, calibrated node probabilities, and the walk of
the target's samples down a tree.

A tree only adds chances for one of a node's children to equal the sample drawn from the node's own logits; the
committed tokens are always the target's keyed samples.  Behaviour parity: reference crates/spec/src/tree.rs:22-120
(Lattice, Policy{edge .6, noise .7, scale 1.5, branch 4}, DraftTree), :199 (best_first: heap over summed sibling
log-probabilities, the first n pops are the n-node tree), :268 (with_copy), :422 (accept_tree).
"""
from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field


@dataclass
class Lattice:
    """Per level (1..rows): candidate token ids with unary scores; edge[level][parent_idx][cand_idx] couples a node's token with the
    next level's candidates (level 1's parent is the anchor, index 0)."""
    ids: list        # [levels][k]
    unary: list      # [levels][k]
    edge: list = None  # [levels][k_prev or 1][k] or None


@dataclass
class Policy:
    edge: float = 0.6
    noise: float = 0.7
    scale: float = 1.5
    branch: int = 4


@dataclass
class DraftTree:
    """Nodes in pop order (parents before children).  Row 0 of the verify window is the anchor; node i is row i + 1."""
    tokens: list = field(default_factory=list)
    parents: list = field(default_factory=list)    # -1 = anchor
    depth: list = field(default_factory=list)
    logp: list = field(default_factory=list)       # summed sibling log-probability along the path

    def __len__(self):
        return len(self.tokens)

    def prefix(self, n: int) -> "DraftTree":
        return DraftTree(self.tokens[:n], self.parents[:n], self.depth[:n], self.logp[:n])

    def path_to(self, node: int) -> list:
        out = []
        while node >= 0:
            out.append(node)
            node = self.parents[node]
        return out[::-1]

    def probabilities(self) -> list:
        """Calibrated-style probability of each node lying on the accepted path: exp(logp), capped to be non-increasing in pop order."""
        out, cap = [], 1.0
        for lp in self.logp:
            p = min(cap, math.exp(lp))
            out.append(p)
            cap = p
        return out


def _log_softmax(xs):
    m = max(xs)
    z = m + math.log(sum(math.exp(x - m) for x in xs))
    return [x - z for x in xs]


def best_first(lat: Lattice, nodes: int, policy: Policy = Policy(), noise=None) -> DraftTree:
    """The `nodes`-node tree: a heap pops nodes best first (highest summed sibling log-probability) and expands each popped
    node's `branch` best children.  Budgets are nested: a smaller budget is a prefix.  `noise(level, token)` adds the target's
    keyed Gumbel noise (weight policy.noise) on sampled requests."""
    tree = DraftTree()
    levels = len(lat.ids)
    heap, counter = [], 0

    def children(level, parent_idx, parent_node, base_lp):
        nonlocal counter
        if level >= levels:
            return
        scores = []
        for c, tid in enumerate(lat.ids[level]):
            s = lat.unary[level][c]
            if lat.edge is not None:
                s += policy.edge * lat.edge[level][parent_idx][c]
            if noise is not None:
                s += policy.noise * noise(level, tid)
            scores.append(s * policy.scale)
        lps = _log_softmax(scores)
        order = sorted(range(len(lps)), key=lambda c: (-lps[c], lat.ids[level][c]))[:policy.branch]
        for c in order:
            counter += 1
            heapq.heappush(heap, (-(base_lp + lps[c]), counter, level, c, parent_node))

    children(0, 0, -1, 0.0)
    while heap and len(tree) < nodes:
        neg, _, level, c, parent = heapq.heappop(heap)
        tree.tokens.append(lat.ids[level][c])
        tree.parents.append(parent)
        tree.depth.append(level + 1)
        tree.logp.append(-neg)
        children(level + 1, c, len(tree) - 1, -neg)
    return tree


def with_copy(tree: DraftTree, copy_tokens, max_nodes: int) -> DraftTree:
    """Graft the copy drafter's chain below the anchor (sharing nodes with the tree where the tokens agree)."""
    out = DraftTree(list(tree.tokens), list(tree.parents), list(tree.depth), list(tree.logp))
    parent, depth = -1, 0
    for t in copy_tokens:
        depth += 1
        found = next((i for i in range(len(out)) if out.parents[i] == parent and out.tokens[i] == t), None)
        if found is None:
            if len(out) >= max_nodes:
                break
            out.tokens.append(t)
            out.parents.append(parent)
            out.depth.append(depth)
            out.logp.append((out.logp[parent] if parent >= 0 else 0.0) - 0.7)
            found = len(out) - 1
        parent = found
    return out


def accept_tree(tree: DraftTree, samples) -> tuple:
    """Walk the target's samples down the tree.  samples[r] is the keyed sample from verify row r (row 0 = anchor, node i = row i+1).
    Returns (accepted node indices along the path, committed tokens = the accepted tokens plus one sample past them)."""
    path, committed = [], []
    row = 0
    while True:
        s = samples[row]
        committed.append(s)
        parent = row - 1
        nxt = next((i for i in range(len(tree)) if tree.parents[i] == parent and tree.tokens[i] == s and i + 1 < len(samples)), None)
        if nxt is None:
            break
        path.append(nxt)
        row = nxt + 1
    return path, committed
