"""CPU mock model: logits depend only on the context, state is deep (paged KV with refcounts, per-slot committed
tokens, pending windows), and it can be told to violate each exactness property so the harness is proven to catch it.

Behaviour parity: reference crates/engine/src/mock.rs:1-120 (MockBackend, MockOptions from ``key=value`` strings),
:24-36 (Fault::{WindowDependent, ChunkDependent, RollbackLeak}), :38-83 (Faults: panic / fatal / retryable at a
step, poisoned first token).
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass

import numpy as np

from ..sched import BlockPool
from ..spec.tree import Lattice
from .backend import Backend, BackendError, DraftOffer, RowOutput


@dataclass
class MockOptions:
    vocab: int = 512
    slots: int = 8
    max_rows: int = 64
    order: int = 0                 # 0: the next token depends on the WHOLE context (deep state); n > 0: on the last n tokens only (text repeats)
    blocks: int = 4096
    block_tokens: int = 64
    fault: str = ""                # "" | window_dependent | chunk_dependent | rollback_leak | prefix_stale
    native_draft: bool = False
    draft_error: float = 0.25      # probability a native draft token is wrong
    trees: bool = False            # step_tree / commit_path are offered
    lattice: bool = False          # the native drafter offers four candidates per level (a wrong first one keeps the right one second)
    margins: bool = False          # the native drafter reports each pick's lead over its runner-up instead of a confidence
    panic_at_step: int = -1
    fatal_at_step: int = -1
    group_lost_at_step: int = -1   # a fatal error that names a lost rank of a multi-rank group (what a peer wait that ran out reports)
    retryable_from_step: int = -1
    nan_at_step: int = -1
    eos: int = -1                  # token the model emits after `eos_after` generated tokens (-1: never)
    eos_after: int = 0
    latency_ms: float = 0.0

    @staticmethod
    def parse(text: str) -> "MockOptions":
        """``key=value,key=value`` as accepted by ``--mock`` on the server command line; unknown keys are refused by name."""
        o = MockOptions()
        for item in filter(None, (t.strip() for t in text.split(","))):
            k, _, v = item.partition("=")
            if not hasattr(o, k):
                raise ValueError(f"unknown mock option {k!r}")
            cur = getattr(o, k)
            setattr(o, k, (v.lower() in ("1", "true", "yes", "on")) if isinstance(cur, bool) else type(cur)(v))
        return o


def _h(data: bytes) -> int:
    return int.from_bytes(hashlib.blake2b(data, digest_size=8).digest(), "little")


class MockBackend(Backend):
    name = "mock"

    def __init__(self, opts: MockOptions | None = None):
        self.o = opts or MockOptions()
        self.vocab_size = self.o.vocab
        self.max_rows = self.o.max_rows
        self.max_slots = self.o.slots
        self.pool = BlockPool(self.o.blocks, self.o.block_tokens)
        self.ctx = {}          # slot -> committed tokens
        self.blocks = {}       # slot -> block ids
        self.pending = {}      # slot -> tokens fed by the last window (beyond the committed ones)
        self.leak = {}         # slot -> junk leaked by a faulty rollback
        self.steps = 0
        self.error = None
        self.generated = {}
        self.media = {}        # slot -> {prompt position: pseudo-token of the image row there}

    def score_last(self, slot, tokens, chunk):
        """A full row consistent with `_row`: the candidates' values at their ids, a low floor elsewhere."""
        r = self._row(list(tokens), 64)
        row = np.full(self.o.vocab, -30.0, dtype=np.float32)
        row[r.ids.astype(np.int64)] = r.values
        return row

    # ---------------------------------------------------------------- the "model"
    def _row(self, context, count: int, salt: int = 0) -> RowOutput:
        o = self.o
        tail = context[-o.order:] if o.order > 0 else context
        key = struct.pack(f"<{len(tail)}I", *[t & 0xFFFFFFFF for t in tail]) + struct.pack("<q", salt)
        rng = np.random.default_rng(_h(key))
        full = min(64, o.vocab)   # the row does not depend on how many candidates are asked for
        ids = rng.choice(o.vocab, size=full, replace=False).astype(np.uint32)
        vals = np.sort(rng.normal(0, 2.0, size=full).astype(np.float32))[::-1].copy()
        vals[0] += 1.5  # a clear favourite most of the time
        order = np.lexsort((ids, -vals.astype(np.float64)))
        n = min(count, full)
        return RowOutput(ids[order][:n].copy(), vals[order][:n].copy())

    def _ensure_blocks(self, slot: int, tokens: int) -> None:
        have = self.blocks.setdefault(slot, [])
        need = self.pool.blocks_for(tokens) - len(have)
        if need > 0:
            got = self.pool.alloc(need)
            if got is None:
                raise BackendError("mock KV pool exhausted", fatal=False)
            have.extend(got)

    def _tick(self) -> None:
        self.steps += 1
        o = self.o
        if self.steps == o.panic_at_step:
            raise RuntimeError("mock panic")
        if self.steps == o.fatal_at_step:
            raise BackendError("mock fatal device error", fatal=True)
        if self.steps == o.group_lost_at_step:
            raise BackendError("mock: device status code 3 (peer timed out)", fatal=True, group_lost=True)
        if o.retryable_from_step >= 0 and self.steps >= o.retryable_from_step:
            self.error = BackendError("mock retryable error", fatal=False)

    # ---------------------------------------------------------------- Backend
    def prefill_slice(self, slot, start, tokens, candidates, last):
        self._tick()
        ctx = self.ctx.setdefault(slot, [])
        if start != len(ctx):
            raise BackendError(f"prefill at {start} but slot {slot} holds {len(ctx)} tokens", fatal=False)
        seen = self.media.get(slot)
        ctx.extend(tokens if not seen else [seen.get(start + j, t) for j, t in enumerate(tokens)])
        self.pending.pop(slot, None)
        self._ensure_blocks(slot, len(ctx))
        if not last:
            return None
        salt = len(tokens) if self.o.fault == "chunk_dependent" else 0
        return self._row(ctx + self.leak.get(slot, []), candidates, salt)

    def step(self, reqs, candidates):
        self._tick()
        out = []
        total_rows = sum(len(r.tokens) for r in reqs)
        for r in reqs:
            ctx = self.ctx.setdefault(r.slot, [])
            if r.first_position != len(ctx):
                raise BackendError(f"window at {r.first_position} but slot {r.slot} holds {len(ctx)} tokens", fatal=False)
            self._ensure_blocks(r.slot, len(ctx) + len(r.tokens))
            self.pending[r.slot] = list(r.tokens)
            rows = []
            for j in range(len(r.tokens)):
                c = ctx + list(r.tokens[:j + 1]) + self.leak.get(r.slot, [])
                salt = total_rows if self.o.fault == "window_dependent" else 0
                row = self._row(c, candidates, salt)
                if self.steps == self.o.nan_at_step:
                    row.values[0] = np.nan
                if self.o.eos >= 0 and self.generated.get(r.slot, 0) + j >= self.o.eos_after:
                    row.ids[0] = self.o.eos
                rows.append(row)
            out.append(rows)
        return out

    def commit(self, slot, keep):
        ctx = self.ctx[slot]
        pend = self.pending.pop(slot, [])
        # the window fed [last, d1..dk]; the first `keep` of those rows become part of the context, the rest never happened
        kept = pend[:keep]
        if self.o.fault == "rollback_leak" and len(pend) > len(kept):
            self.leak[slot] = [pend[len(kept)]]
        self.generated[slot] = self.generated.get(slot, 0) + keep
        ctx.extend(kept)

    def supports_trees(self):
        return self.o.trees

    def supports_media(self):
        return True

    def set_media(self, slot, media):
        """The mock "sees" an image through its rows: every placeholder position reads as a pseudo-token made from that row's embedding."""
        if media is None:
            self.media.pop(slot, None)
            return
        emb = np.asarray(media.embeds, dtype=np.float32)
        self.media[slot] = {int(r): _h(emb[i].tobytes()) & 0x7FFFFFFF for i, r in enumerate(media.rows)}

    def step_tree(self, reqs, candidates):
        self._tick()
        out = []
        total_rows = sum(len(r.tokens) for r in reqs)
        for r in reqs:
            ctx = self.ctx.setdefault(r.slot, [])
            if r.first_position != len(ctx):
                raise BackendError(f"tree window at {r.first_position} but slot {r.slot} holds {len(ctx)} tokens", fatal=False)
            if r.parents[0] != -1 or any(not 0 <= r.parents[i] < i for i in range(1, len(r.tokens))):
                raise BackendError("tree rows must follow their parents", fatal=False)
            self._ensure_blocks(r.slot, len(ctx) + len(r.tokens))
            self.pending[r.slot] = (list(r.tokens), list(r.parents))
            paths, rows = [], []
            for j in range(len(r.tokens)):
                paths.append((paths[r.parents[j]] if j else []) + [r.tokens[j]])
                salt = total_rows if self.o.fault == "window_dependent" else 0
                row = self._row(ctx + paths[j] + self.leak.get(r.slot, []), candidates, salt)
                if self.o.eos >= 0 and self.generated.get(r.slot, 0) + len(paths[j]) - 1 >= self.o.eos_after:
                    row.ids[0] = self.o.eos
                rows.append(row)
            out.append(rows)
        return out

    def commit_path(self, slot, rows):
        toks, parents = self.pending.pop(slot)
        prev = 0
        for r in rows:
            if parents[r] != prev:
                raise BackendError(f"commit_path: row {r} does not follow row {prev}", fatal=False)
            prev = r
        kept = [toks[0]] + [toks[r] for r in rows]
        if self.o.fault == "rollback_leak" and len(toks) > len(kept):
            self.leak[slot] = [next(toks[i] for i in range(1, len(toks)) if i not in rows)]
        self.generated[slot] = self.generated.get(slot, 0) + len(kept)
        self.ctx[slot].extend(kept)

    def release(self, slot):
        self.ctx.pop(slot, None)
        self.pending.pop(slot, None)
        self.leak.pop(slot, None)
        self.generated.pop(slot, None)
        self.media.pop(slot, None)
        b = self.blocks.pop(slot, None)
        if b:
            self.pool.release(b)

    def take_error(self):
        e, self.error = self.error, None
        return e

    def supports_native_draft(self):
        return self.o.native_draft

    def propose_batch(self, asks):
        out = {}
        for a in asks:
            ctx, toks = list(a.context), []
            lat_ids, lat_val, margins = [], [], []
            for j in range(a.max_drafts):
                row = self._row(ctx, 4)
                t = int(row.ids[0])
                if (_h(struct.pack("<qq", len(ctx), t)) % 1000) / 1000.0 < self.o.draft_error:
                    t = (t + 1) % self.o.vocab
                # a wrong pick comes with a small lead, a right one with a large lead (what a margin is good for)
                margins.append(0.2 if t != int(row.ids[0]) else 6.0)
                toks.append(t)
                if self.o.lattice:
                    # candidates of this level: the drafter's pick first, then the model's own order; deeper levels follow the model's pick
                    rest = [int(x) for x in row.ids[:4] if int(x) != t]
                    lat_ids.append(([t] + rest)[:4])
                    lat_val.append([float(x) for x in row.values[:4]])
                    ctx.append(int(row.ids[0]))
                else:
                    ctx.append(t)
            out[a.slot] = DraftOffer(toks, [0.7] * len(toks) if not self.o.margins else [], Lattice(lat_ids, lat_val) if self.o.lattice else None,
                                     margins if self.o.margins else [])
        return out

    # prefix cache: blocks are shared by refcount
    def prefix_block_tokens(self):
        return self.o.block_tokens

    def prefix_bytes_per_block(self):
        return self.o.block_tokens * 1024

    def prefix_commit(self, slot, blocks):
        ids = self.blocks.get(slot, [])[:blocks]
        ctx = self.ctx[slot]
        handles = []
        for i, b in enumerate(ids):
            self.pool.retain([b])
            handles.append(("blk", b, tuple(ctx[i * self.o.block_tokens:(i + 1) * self.o.block_tokens])))
        return handles

    def prefix_restore(self, slot, handles):
        ctx = self.ctx.setdefault(slot, [])
        assert not ctx
        ids = []
        for _, b, toks in handles:
            self.pool.retain([b])
            ids.append(b)
            ctx.extend(toks)
        if self.o.fault == "prefix_stale" and ctx:
            ctx[-1] = (ctx[-1] + 1) % self.o.vocab
        self.blocks[slot] = ids
        return len(ctx)

    def prefix_release(self, handles):
        for _, b, _ in handles:
            self.pool.release([b])

    def prefix_export(self, handle):
        import struct
        return struct.pack(f"<{len(handle[2])}i", *handle[2])

    def prefix_import(self, payload):
        import struct
        got = self.pool.alloc(1)
        if got is None:
            return None
        return ("blk", got[0], struct.unpack(f"<{len(payload) // 4}i", payload))
