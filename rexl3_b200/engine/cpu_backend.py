"""CPU reference backend: the fp32 PyTorch executor over dequantized EXL3 weights behind the engine's Backend contract.

Runs the CPU plumbing configuration (tiny Llama-style decoder) without a GPU and serves as the oracle for the device
backend.  Each sequence is computed on its own, so row invariance holds by construction.
"""
from __future__ import annotations

import torch

from ..models.dense import HostWeights, ReferenceDense
from ..sampling import top_candidates
from .backend import Backend, BackendError, RowOutput


class CpuDenseBackend(Backend):
    name = "cpu-reference"

    def __init__(self, weights: HostWeights, max_slots: int = 8, max_rows: int = 64, dtype=torch.float32):
        self.model = ReferenceDense(weights, device="cpu", dtype=dtype)
        self.cfg = weights.cfg
        self.vocab_size = weights.cfg.vocab
        self.max_slots, self.max_rows = max_slots, max_rows
        self.len = {}
        self.pending = {}
        self.last_logits = None

    def _rows(self, logits: torch.Tensor, candidates: int):
        out = []
        for r in logits.numpy():
            ids, vals = top_candidates(r, candidates)
            out.append(RowOutput(ids, vals))
        return out

    def prefill_slice(self, slot, start, tokens, candidates, last):
        if start != self.len.get(slot, 0):
            raise BackendError(f"prefill at {start} but slot {slot} holds {self.len.get(slot, 0)} tokens")
        logits = self.model.forward_seq(slot, tokens, start)
        self.len[slot] = start + len(tokens)
        self.last_logits = logits[-1:].clone()
        return self._rows(logits[-1:], candidates)[0] if last else None

    def step(self, reqs, candidates):
        out = []
        for r in reqs:
            if r.first_position != self.len.get(r.slot, 0):
                raise BackendError(f"window at {r.first_position} but slot {r.slot} holds {self.len.get(r.slot, 0)} tokens")
            logits = self.model.forward_seq(r.slot, r.tokens, r.first_position)
            self.pending[r.slot] = len(r.tokens)
            out.append(self._rows(logits, candidates))
        return out

    def commit(self, slot, keep):
        keep = min(keep, self.pending.pop(slot, 0))
        self.len[slot] = self.len.get(slot, 0) + keep
        self.model.truncate(slot, self.len[slot])

    def release(self, slot):
        self.len.pop(slot, None)
        self.pending.pop(slot, None)
        self.model.reset(slot)

    def score_rows(self, slot, start, tokens):
        logits = self.model.forward_seq(slot, tokens, start)
        self.model.truncate(slot, start)
        return logits.numpy()

    def score_last(self, slot, tokens, chunk):
        row = None
        for a in range(0, len(tokens), chunk):
            row = self.model.forward_seq(slot, tokens[a:a + chunk], a)[-1]
        return row.numpy().astype("float32")


class CpuHybridBackend(CpuDenseBackend):
    """The fp32 hybrid (Mamba2 / delta-net + attention) oracle behind the Backend contract.  A recurrent state cannot be truncated, so a
    window is undone the way the reference's record / commit scheme does it: the state before the window is kept (a snapshot), and a
    commit that keeps fewer rows than were fed restores it and replays the kept rows.  Prompt scoring undoes its rows the same way."""
    name = "cpu-hybrid-reference"

    def __init__(self, weights: HostWeights, max_slots: int = 8, max_rows: int = 64, dtype=torch.float32):
        from ..models.hybrid import ReferenceHybrid
        self.model = ReferenceHybrid(weights, device="cpu", dtype=dtype)
        self.cfg = weights.cfg
        self.vocab_size = weights.cfg.vocab
        self.max_slots, self.max_rows = max_slots, max_rows
        self.len, self.pending, self.last_logits = {}, {}, None
        self._before = {}          # slot -> (snapshot before the window in flight, its tokens, its first position)

    def step(self, reqs, candidates):
        out = []
        for r in reqs:
            if r.first_position != self.len.get(r.slot, 0):
                raise BackendError(f"window at {r.first_position} but slot {r.slot} holds {self.len.get(r.slot, 0)} tokens")
            self._before[r.slot] = (self.model.snapshot(r.slot), list(r.tokens), r.first_position)
            logits = self.model.forward_seq(r.slot, r.tokens, r.first_position)
            self.pending[r.slot] = len(r.tokens)
            out.append(self._rows(logits, candidates))
        return out

    def commit(self, slot, keep):
        fed = self.pending.pop(slot, 0)
        before = self._before.pop(slot, None)
        keep = min(keep, fed)
        if keep < fed:
            snap, tokens, pos = before
            self.model.restore(slot, snap)
            if keep:
                self.model.forward_seq(slot, tokens[:keep], pos)         # replay of the accepted prefix
        self.len[slot] = self.len.get(slot, 0) + keep

    def release(self, slot):
        self._before.pop(slot, None)
        super().release(slot)

    def score_rows(self, slot, start, tokens):
        snap = self.model.snapshot(slot)
        logits = self.model.forward_seq(slot, tokens, start)
        self.model.restore(slot, snap)
        return logits.numpy()

    # ---- prefix cache: a block is restorable only where a slice ended (the handle of that block carries a full snapshot)
    BLOCK = 64

    def prefix_block_tokens(self):
        return self.BLOCK

    def prefix_needs_cuts(self) -> bool:
        return True

    def prefix_bytes_per_block(self):
        return self.cfg.state_bytes_per_slot() + self.cfg.kv_bytes_per_token(4) * self.BLOCK

    def prefix_commit(self, slot, blocks):
        snap = self.model.snapshot(slot) if self.len.get(slot, 0) == blocks * self.BLOCK else None
        return [("hyb", i, snap if i == blocks - 1 else None) for i in range(blocks)]

    def prefix_restore(self, slot, handles):
        best = max((i for i, h in enumerate(handles) if h[2] is not None), default=-1)
        if best < 0:
            return 0
        self.model.restore(slot, handles[best][2])
        self.len[slot] = (best + 1) * self.BLOCK
        return self.len[slot]

    def prefix_release(self, handles):
        pass
