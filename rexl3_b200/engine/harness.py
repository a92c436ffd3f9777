"""Exactness harness, generic over a backend factory: the five checks every model runtime must pass, plus the
prefix-cache check.

row_invariance, serial_batched_equals_solo, drafted_equals_serial, chunked_prefill_equals_whole,
rollback_equals_replay (behaviour parity: reference crates/engine/src/harness.rs:1-9,43-150) and cached_equals_cold
(crates/sched/src/prefix.rs:5-12).  Each check returns None on success or a human-readable reason; the mock backend can
be told to violate each property, which proves the harness catches it.
"""
from __future__ import annotations

import numpy as np

from ..sampling import Sampling
from ..sched import CacheBudget, PrefixIndex
from .backend import DraftOffer
from .core import Engine, generate

SAMPLING = Sampling(seed=1234, temperature=0.8, top_k=20, top_p=0.9)


def default_prompts(vocab: int, lengths=(3, 70, 150), seed: int = 0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


def _run(make_backend, prompts, n, sampling=SAMPLING, **kw):
    eng = Engine(make_backend(), **kw)
    return generate(eng, prompts, n, sampling), eng


def _diff(name, a, b):
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            j = next((k for k, (u, v) in enumerate(zip(x, y)) if u != v), min(len(x), len(y)))
            return f"{name}: sequence {i} differs at generated token {j}: {x[j:j + 4]} vs {y[j:j + 4]}"
    return None


def row_invariance(make_backend, vocab, n=24):
    """A request's tokens do not depend on which other requests share its windows."""
    p = default_prompts(vocab)
    solo, _ = _run(make_backend, [p[1]], n, spec="none")
    both, _ = _run(make_backend, [p[0], p[1], p[2]], n, spec="none")
    return _diff("row_invariance", solo, [both[1]])


def serial_batched_equals_solo(make_backend, vocab, n=24):
    p = default_prompts(vocab, (5, 9, 33, 64))
    batched, _ = _run(make_backend, p, n, spec="none")
    solo = [_run(make_backend, [q], n, spec="none")[0][0] for q in p]
    return _diff("serial_batched_equals_solo", batched, solo)


def drafted_equals_serial(make_backend, vocab, n=48):
    p = default_prompts(vocab)
    # repetitive prompt so the copy drafter proposes something
    p.append((p[1][:20] * 6)[:110])
    serial, _ = _run(make_backend, p, n, spec="none")
    drafted, eng = _run(make_backend, p, n, spec="auto", max_drafts=4)
    return _diff("drafted_equals_serial", serial, drafted)


def chunked_prefill_equals_whole(make_backend, vocab, n=8):
    p = default_prompts(vocab, (150, 67))
    whole, _ = _run(make_backend, p, n, spec="none", prefill_chunk=4096, prefill_policy="serial")
    for chunk in (64, 37):
        cut, _ = _run(make_backend, p, n, spec="none", prefill_chunk=chunk, prefill_policy="serial")
        d = _diff(f"chunked_prefill_equals_whole(chunk={chunk})", whole, cut)
        if d:
            return d
    return None


class _WrongDrafts:
    """Wraps a backend with a native drafter that is right for one token and then wrong, so every round rolls back."""

    def __init__(self, inner, vocab):
        self.inner, self.vocab = inner, vocab

    def __getattr__(self, k):
        return getattr(self.inner, k)

    def supports_native_draft(self):
        return True

    def propose_batch(self, asks):
        return {a.slot: DraftOffer([(a.context[-1] * 7 + 3 + j) % self.vocab for j in range(a.max_drafts)]) for a in asks}


def rollback_equals_replay(make_backend, vocab, n=32):
    """After partly (here: mostly) rejected windows the state equals a serial replay."""
    p = default_prompts(vocab)
    serial, _ = _run(make_backend, p, n, spec="none")
    rolled, _ = _run(lambda: _WrongDrafts(make_backend(), vocab), p, n, spec="self", max_drafts=3)
    return _diff("rollback_equals_replay", serial, rolled)


def cached_equals_cold(make_backend, vocab, n=16):
    """A prefix-cache hit gives the same reply as an uncached run."""
    rng = np.random.default_rng(5)
    shared = rng.integers(0, vocab, size=200).tolist()
    a, b = shared + [1, 2, 3], shared + [4, 5]
    cold, _ = _run(make_backend, [a, b], n, spec="none")
    be = make_backend()
    if be.prefix_block_tokens() <= 0:
        return None
    eng = Engine(be, spec="none", prefix=PrefixIndex(CacheBudget(1 << 40), block_tokens=be.prefix_block_tokens()))
    first = generate(eng, [a], n, SAMPLING)
    second = generate(eng, [b], n, SAMPLING)
    if eng.counters["cached_tokens"] <= 0:
        return "cached_equals_cold: the second prompt did not hit the cache"
    return _diff("cached_equals_cold", cold, [first[0], second[0]])


def trees_equal_serial(make_backend, vocab, n=48):
    """Tree windows (best-first trees over the drafter's lattice, the copy chain grafted in) commit the serial run's tokens; a backend
    without tree support passes trivially (its rounds stay chains)."""
    from .core import TreeConfig
    p = default_prompts(vocab)
    p.append((p[1][:20] * 6)[:110])
    serial, _ = _run(make_backend, p, n, spec="none")
    for nodes in (3, 12):
        treed, eng = _run(make_backend, p, n, spec="auto", max_drafts=4, trees=TreeConfig(max_nodes=nodes))
        d = _diff(f"trees_equal_serial[{nodes} nodes]", serial, treed)
        if d is not None:
            return d
    return None


ALL = (row_invariance, serial_batched_equals_solo, drafted_equals_serial, chunked_prefill_equals_whole, rollback_equals_replay,
       cached_equals_cold, trees_equal_serial)


def run_all(make_backend, vocab) -> dict:
    return {f.__name__: f(make_backend, vocab) for f in ALL}
