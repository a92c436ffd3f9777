"""Family-neutral lockstep control plane for multi-rank backends (tensor or expert parallel): rank 0 owns the scheduler and the
sampler; every state-changing backend call is numbered and broadcast to the followers BEFORE the leader applies it, and each
follower replays it on its own backend instance (own block pool, own graphs), so all ranks launch the same kernels in the same
order and meet inside the fused collectives.  Parity: reference crates/model/src/lockstep.rs:1-46 (numbered calls, followers replay
on one thread, a lost or out-of-order message means the group state is lost).

Transport: one pickled broadcast per call over a CPU (gloo) group.  A follower that sees a gap in the numbering, or a timeout of
the group, raises `GroupLost`; so does the leader when a broadcast fails.  Failure tests drive this with host-side faults only.
"""
from __future__ import annotations

import torch.distributed as dist

from .backend import Backend, DraftAsk

REPLAYED = ("prefill_slice", "prefill_slices", "step", "step_verified", "commit", "release", "propose_batch", "prefix_restore", "prefix_commit",
            "prefix_release", "quiesce")


class GroupLost(RuntimeError):
    pass


class _Tail:
    """Stands in for a token list on a follower: the drafter needs only its length and its last token."""

    def __init__(self, n: int, last: int):
        self.n, self.last = n, last

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        if i != -1:
            raise IndexError("only the last token travels to followers")
        return self.last


def _pack(name, args):
    if name == "propose_batch":
        return (name, ([(a.slot, len(a.context), a.context[-1], a.max_drafts) for a in args[0]],))
    return (name, args)


def _unpack(name, args):
    if name == "propose_batch":
        return ([DraftAsk(s, _Tail(n, last), m) for s, n, last, m in args[0]],)
    return args


class LockstepLeader(Backend):
    """Wraps rank 0's backend.  `drop_next` (tests) swallows one message to show that followers detect the gap."""

    def __init__(self, inner: Backend, ctrl_group, src: int = 0):
        self.inner, self.ctrl, self.src = inner, ctrl_group, src
        self.seq = 0
        self.drop_next = False
        self.vocab_size, self.max_rows, self.max_slots = inner.vocab_size, inner.max_rows, inner.max_slots
        self.name = inner.name + "+lockstep"

    def _send(self, name, args):
        self.seq += 1
        if self.drop_next:
            self.drop_next = False
            return
        try:
            dist.broadcast_object_list([(self.seq,) + _pack(name, args)], src=self.src, group=self.ctrl)
        except Exception as e:      # a dead follower surfaces here as a transport error or timeout
            raise GroupLost(f"lockstep broadcast {self.seq} ({name}) failed: {e}") from e

    def __getattr__(self, name):
        # anything not replayed (stats, take_error, prefix_block_tokens, ...) goes straight to the inner backend
        return getattr(self.inner, name)

    def stop(self):
        self._send("stop", ())


def _replayed(name):
    def call(self, *args):
        self._send(name, args)
        return getattr(self.inner, name)(*args)
    call.__name__ = name
    return call


for _n in REPLAYED:
    setattr(LockstepLeader, _n, _replayed(_n))
# capability probes must reflect the inner backend, not the Backend defaults
for _n in ("supports_native_draft", "take_error", "prefix_block_tokens", "prefix_bytes_per_block", "stats", "score_rows"):
    setattr(LockstepLeader, _n, (lambda n: lambda self, *a: getattr(self.inner, n)(*a))(_n))


def follow(inner: Backend, ctrl_group, src: int = 0) -> int:
    """Follower loop: replay until the leader says stop.  Returns the number of calls replayed."""
    expect = 0
    while True:
        box = [None]
        try:
            dist.broadcast_object_list(box, src=src, group=ctrl_group)
        except Exception as e:
            raise GroupLost(f"lockstep receive after call {expect} failed: {e}") from e
        seq, name, args = box[0]
        expect += 1
        if seq != expect:
            raise GroupLost(f"lockstep numbering gap: got call {seq}, expected {expect}")
        if name == "stop":
            return expect - 1
        getattr(inner, name)(*_unpack(name, args))
