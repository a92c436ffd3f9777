"""Prefix-cache index: chain-hashed 64-token blocks, longest strict prefix lookup, LRU / size-aware eviction with a
ghost set, cut planning and byte budgets.

Behaviour parity: reference crates/sched/src/prefix.rs:34-920 (PrefixIndex lookup/insert/evict, Chain, Ghost,
CutPolicy, plan_cuts, CacheBudget, Eviction::{Lru, SizeAware}).  Block size follows this engine's 64-token pages
(the reference uses 256).  A hit must be a STRICT prefix of the prompt so the model still runs at least one row and
"cached == cold" can hold bit for bit.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass

BLOCK_TOKENS = 64


def chain_hashes(tokens, block_tokens: int = BLOCK_TOKENS, namespace: bytes = b"") -> list:
    """Hash of every full block, each chained on the previous one: equal hash <=> equal prefix (and namespace)."""
    out, prev = [], hashlib.sha256(b"rexl3-prefix-v1|" + namespace).digest()[:16]
    for b in range(len(tokens) // block_tokens):
        h = hashlib.blake2b(prev, digest_size=16)
        h.update(struct.pack(f"<{block_tokens}I", *[int(t) & 0xFFFFFFFF for t in tokens[b * block_tokens:(b + 1) * block_tokens]]))
        prev = h.digest()
        out.append(prev)
    return out


def image_token(content_key: bytes, index: int) -> int:
    """A stable pseudo-token for position `index` of an image run, so image prompts can be prefix-cached by content."""
    return int.from_bytes(hashlib.sha256(content_key + struct.pack("<I", index)).digest()[:4], "little") | 0x80000000


@dataclass
class Entry:
    key: bytes
    parent: bytes | None
    depth: int                 # blocks from the root (1-based)
    handle: object             # what the backend needs to restore (page id, snapshot id, ...)
    nbytes: int
    children: int = 0
    hits: int = 0
    cost: float = 1.0          # recompute cost estimate (tokens) for size-aware eviction
    priority: float = 0.0


@dataclass
class CacheBudget:
    max_bytes: int
    max_entries: int = 1 << 30


class PrefixIndex:
    def __init__(self, budget: CacheBudget, eviction: str = "lru", block_tokens: int = BLOCK_TOKENS, ghost_capacity: int = 4096):
        if eviction not in ("lru", "size_aware"):
            raise ValueError(f"unknown eviction policy {eviction!r}")
        self.budget, self.eviction, self.block_tokens = budget, eviction, block_tokens
        self.entries: "OrderedDict[bytes, Entry]" = OrderedDict()   # LRU order: oldest first
        self.bytes = 0
        self.ghosts: "OrderedDict[bytes, int]" = OrderedDict()      # recently evicted keys -> depth
        self.ghost_capacity = ghost_capacity
        self.clock = 0.0      # GreedyDual inflation value
        self.stats = dict(lookups=0, hits=0, hit_blocks=0, inserts=0, evictions=0, ghost_hits=0)
        self.on_evict = None  # called with the Entry just before it leaves the index (a spill tier saves the block here)

    def __len__(self):
        return len(self.entries)

    # ---------------------------------------------------------------- lookup
    def lookup(self, hashes: list, prompt_tokens: int):
        """Longest cached chain that is a STRICT prefix of the prompt.  Returns the list of entries (root first)."""
        self.stats["lookups"] += 1
        max_blocks = (prompt_tokens - 1) // self.block_tokens  # strict: at least one token left to run
        chain = []
        for h in hashes[:max_blocks]:
            e = self.entries.get(h)
            if e is None:
                if h in self.ghosts:
                    self.stats["ghost_hits"] += 1
                break
            chain.append(e)
        if chain:
            self.stats["hits"] += 1
            self.stats["hit_blocks"] += len(chain)
            for e in chain:
                e.hits += 1
                self._touch(e)
        return chain

    def _touch(self, e: Entry) -> None:
        self.entries.move_to_end(e.key)
        if self.eviction == "size_aware":
            e.priority = self.clock + e.cost * max(1, e.hits) / max(1, e.nbytes)

    # ---------------------------------------------------------------- insert
    def insert(self, hashes: list, handles: list, nbytes_each: int, cost_each: float = None):
        """Insert blocks hashes[i] -> handles[i] (a chain from the root).  Existing blocks are kept (their handle wins) and the
        caller's duplicate handle is returned for release.  Returns (duplicates, evicted_handles)."""
        dup, evicted = [], []
        parent = None
        for i, (h, handle) in enumerate(zip(hashes, handles)):
            e = self.entries.get(h)
            if e is not None:
                if handle is not None and handle is not e.handle:
                    dup.append(handle)
                self._touch(e)
            else:
                e = Entry(h, parent, i + 1, handle, nbytes_each, cost=cost_each if cost_each is not None else float(self.block_tokens))
                self.entries[h] = e
                self.bytes += nbytes_each
                if parent is not None and parent in self.entries:
                    self.entries[parent].children += 1
                self.ghosts.pop(h, None)
                self.stats["inserts"] += 1
                self._touch(e)
            parent = h
        evicted.extend(self.evict_to_budget(protect=set(hashes)))
        return dup, evicted

    # ---------------------------------------------------------------- eviction
    def _victim(self, protect):
        leafs = [e for e in self.entries.values() if e.children == 0 and e.key not in protect]
        if not leafs:
            return None
        if self.eviction == "lru":
            return leafs[0]  # OrderedDict iteration order = least recently used first
        return min(leafs, key=lambda e: e.priority)

    def evict_one(self, protect=frozenset()):
        v = self._victim(protect)
        if v is None:
            return None
        if self.on_evict is not None:
            self.on_evict(v)
        del self.entries[v.key]
        self.bytes -= v.nbytes
        if v.parent is not None and v.parent in self.entries:
            self.entries[v.parent].children -= 1
        if self.eviction == "size_aware":
            self.clock = max(self.clock, v.priority)
        self.ghosts[v.key] = v.depth
        while len(self.ghosts) > self.ghost_capacity:
            self.ghosts.popitem(last=False)
        self.stats["evictions"] += 1
        return v.handle

    def evict_to_budget(self, protect=frozenset()):
        out = []
        while self.bytes > self.budget.max_bytes or len(self.entries) > self.budget.max_entries:
            h = self.evict_one(protect)
            if h is None:
                break
            out.append(h)
        return out

    def evict_bytes(self, need: int):
        """Free at least `need` bytes (memory pressure from admission); returns the evicted handles."""
        out, freed = [], 0
        while freed < need:
            before = self.bytes
            h = self.evict_one()
            if h is None:
                break
            freed += before - self.bytes
            out.append(h)
        return out

    def clear(self):
        out = [e.handle for e in self.entries.values()]
        self.entries.clear()
        self.bytes = 0
        return out

    def reach_tokens(self) -> int:
        return max((e.depth for e in self.entries.values()), default=0) * self.block_tokens


@dataclass
class CutPolicy:
    """Where snapshots are taken inside a long prefill so a cancelled prompt can resume and later prompts can share."""
    every_tokens: int = 4096
    align: int = BLOCK_TOKENS
    max_cuts: int = 64


def plan_cuts(start: int, end: int, policy: CutPolicy) -> list:
    """Aligned cut positions in (start, end): multiples of `every_tokens` rounded to the block size, at most max_cuts (the
    latest ones win, because they save the most recompute)."""
    if end <= start or policy.every_tokens <= 0:
        return []
    step = max(policy.align, policy.every_tokens // policy.align * policy.align)
    first = (start // step + 1) * step
    cuts = list(range(first, end, step))
    last_aligned = (end - 1) // policy.align * policy.align
    if last_aligned > start and last_aligned not in cuts and last_aligned < end:
        cuts.append(last_aligned)
    return sorted(cuts)[-policy.max_cuts:]
