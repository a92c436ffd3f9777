"""The contract between the engine's step loop and a model runtime.

A backend serves fixed sequence *slots*.  Every state-changing call is one of: ``prefill_slice`` (append prompt tokens
to a slot), ``step`` (a window of rows over several slots: each slot feeds ``[last, d1..dk]`` at consecutive positions),
``commit`` (keep the first ``keep`` rows of the slot's last window; the rest never become visible) and ``release``.
Rows come back as the top candidates (value desc, id asc) - the engine never sees full logits except on the score path.

Contract sentence: every row's output is bit-identical to what the same backend returns for that row in a one-row step.
Behaviour parity: reference crates/engine/src/lib.rs:212-432 (trait Backend and its optional methods).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class RowRequest:
    slot: int
    tokens: list           # [last, d1 .. dk]
    first_position: int    # absolute position of tokens[0]


@dataclass
class TreeRequest:
    """One sequence's rows of a tree window: row 0 is the anchor (the last committed token), row i > 0 a draft node whose parent row is
    `parents[i]` < i (`parents[0]` = -1).  Row i is the token at position first_position + depth(i)."""
    slot: int
    tokens: list
    parents: list
    first_position: int

    def depths(self) -> list:
        d = [0] * len(self.tokens)
        for i in range(1, len(self.tokens)):
            d[i] = d[self.parents[i]] + 1
        return d


@dataclass
class MediaInputs:
    """What a prompt with images carries beside its tokens (the prompt holds one run of the placeholder token per image).
    rows: indices of the placeholder tokens in the prompt, ascending; embeds: [len(rows), d_model] rows that replace those tokens'
    embeddings (a vision tower's output, any float dtype, host or device tensor); pos3: int32 [len(prompt), 3] (T, H, W) positions for a model
    with M-RoPE sections, or None (plain positions); rope_delta: what decode rows add to their position on every axis (the text after an
    image continues at 1 + the largest position the image used, which is less than the token count); keys: one content digest per image
    with (first row index into `rows`, count), from which the prefix cache's block hashes are made."""
    rows: np.ndarray
    embeds: object
    pos3: np.ndarray | None = None
    rope_delta: int = 0
    keys: list = field(default_factory=list)      # [(first, count, digest bytes)]

    def hash_tokens(self, prompt: list) -> list:
        """The prompt with every placeholder replaced by a pseudo-token made from its image's content and the index inside the image: equal
        block hashes then mean equal text AND equal images (reference crates/sched/src/lib.rs:300-360, image_token / prefix_hashes)."""
        from ..sched.prefix import image_token
        out = list(prompt)
        for first, count, digest in self.keys:
            for j in range(count):
                out[int(self.rows[first + j])] = image_token(digest, j)
        return out


@dataclass
class RowOutput:
    ids: np.ndarray        # uint32 [count], ordered (value desc, id asc)
    values: np.ndarray     # float32 [count]


class BackendError(Exception):
    """`group_lost`: the error means a rank of a multi-rank group stopped answering (a peer wait ran out or was aborted); the server
    then reports the state `group_lost` (reference crates/model/src/lockstep.rs:29-38, StateLost)."""

    def __init__(self, message: str, fatal: bool = False, group_lost: bool = False):
        super().__init__(message)
        self.fatal = fatal
        self.group_lost = group_lost


@dataclass
class DraftAsk:
    slot: int
    context: list          # committed tokens of the sequence
    max_drafts: int
    sampling: object = None


@dataclass
class DraftOffer:
    tokens: list = field(default_factory=list)
    conf: list = field(default_factory=list)       # optional per-draft confidence (probability it is accepted given the ones before)
    lattice: object = None                         # optional spec.tree.Lattice: per level the drafter's candidate ids and scores (level 0 = first draft)
    margin: list = field(default_factory=list)     # optional per draft: how far the pick leads the drafter's runner-up, in logits


class Backend:
    """Base class; a runtime overrides what it supports."""

    vocab_size: int = 0
    max_rows: int = 64            # rows one window may hold
    max_slots: int = 8
    name: str = "backend"

    # ---- required
    def prefill_slice(self, slot: int, start: int, tokens: list, candidates: int, last: bool):
        """Append `tokens` at positions start.. of `slot`.  Returns the last row's RowOutput when `last`, else None."""
        raise NotImplementedError

    def step(self, reqs: list, candidates: int) -> list:
        """One window.  Returns, per request, a list of RowOutput (one per fed token)."""
        raise NotImplementedError

    def commit(self, slot: int, keep: int) -> None:
        raise NotImplementedError

    def release(self, slot: int) -> None:
        raise NotImplementedError

    # ---- optional
    def prefill_slices(self, items: list, candidates: int) -> list:
        """Batched short prompts: items = [(slot, start, tokens, last)].  Default: one after another."""
        return [self.prefill_slice(s, st, t, candidates, last) for s, st, t, last in items]

    def step_verified(self, reqs: list, candidates: int, greedy: list) -> list:
        """`greedy[i]` says request i samples at T == 0 (a backend may return a single candidate per row for those)."""
        return self.step(reqs, candidates)

    def propose_batch(self, asks: list) -> dict:
        """Native drafter: slot -> DraftOffer.  Default: no native drafter."""
        return {}

    def supports_native_draft(self) -> bool:
        return False

    def supports_trees(self) -> bool:
        """True: `step_tree` / `commit_path` are implemented (reference crates/engine/src/lib.rs:212-432, step_tree / commit_path /
        supports_trees)."""
        return False

    def step_tree(self, reqs: list, candidates: int) -> list:
        """One window of draft trees (reqs: TreeRequest).  Returns, per request, one RowOutput per row; a row's output is what a one-row step
        returns after the tokens on the row's path from the anchor."""
        raise NotImplementedError

    def commit_path(self, slot: int, rows: list) -> None:
        """Keep the anchor and the rows `rows` (a path: each row's parent is the one before, the first row's parent the anchor) of the slot's
        last tree window; every other row never happened."""
        raise NotImplementedError

    def supports_media(self) -> bool:
        """True: `set_media` is implemented (prompts whose placeholder rows take a vision tower's embeddings)."""
        return False

    def set_media(self, slot: int, media) -> None:
        """The MediaInputs of the prompt that `slot` is about to prefill (None clears); `release` forgets them."""
        raise NotImplementedError

    def supports_rollback(self) -> bool:
        """False: rows fed to `step` cannot be rejected afterwards (recurrent state), so the engine plans no draft rows."""
        return True

    def take_error(self):
        """A BackendError raised asynchronously by the last call (device status words), or None."""
        return None

    def score_rows(self, slot: int, start: int, tokens: list) -> np.ndarray:
        """Full-vocabulary logits of every fed row (prompt scoring / logprobs).  Optional."""
        raise NotImplementedError

    def score_last(self, slot: int, tokens: list, chunk: int) -> np.ndarray:
        """Full-vocabulary float32 logits of the position after `tokens` (prefilled into the empty `slot` in chunks).  Default: built on
        `score_rows`.  The caller releases the slot."""
        row = None
        for a in range(0, len(tokens), chunk):
            row = self.score_rows(slot, a, tokens[a:a + chunk])[-1]
            self.commit_scored(slot, a + len(tokens[a:a + chunk]))
        return np.asarray(row, dtype=np.float32)

    def commit_scored(self, slot: int, length: int) -> None:
        """Hook for `score_last`'s default: make the scored chunk part of the slot's context (backends whose `score_rows` rolls back)."""

    # prefix cache (optional): handles are opaque to the engine
    def prefix_block_tokens(self) -> int:
        return 0                   # 0 = no prefix cache support

    def prefix_restore(self, slot: int, handles: list) -> int:
        """Make `slot` start with the cached blocks `handles`; returns the number of tokens restored."""
        return 0

    def prefix_commit(self, slot: int, blocks: int) -> list:
        """Handles of the slot's first `blocks` full blocks (the backend retains them for the cache)."""
        return []

    def prefix_release(self, handles: list) -> None:
        pass

    def prefix_needs_cuts(self) -> bool:
        """True for backends with recurrent state: a block can be cached only if a prefill slice ENDED at its last token (that is when the
        state can be snapshotted), so the engine ends a slice at the prompt's last full-block boundary.  `prefix_restore` of such a backend
        may restore fewer blocks than it is given (down to the deepest one that carries a snapshot) and returns what it restored."""
        return False

    def prefix_export(self, handle) -> bytes | None:
        """The block's cached state as bytes (for a spill tier), or None when this backend cannot export."""
        return None

    def prefix_import(self, payload: bytes):
        """A new handle holding an exported block again (the caller owns one reference), or None (no room, or not supported)."""
        return None

    def prefix_bytes_per_block(self) -> int:
        return 0

    def quiesce(self) -> None:
        """Wait for all device work (used before measuring and at shutdown)."""

    def stats(self) -> dict:
        return {}
