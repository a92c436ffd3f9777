"""Multi-GPU self test of the tensor-parallel path, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m rexl3_b200.parallel.selftest

Rank 0 runs the engine over the TP backend (the others follow), generates greedily for a few prompts with graphs on,
and checks every generated token against an fp32 reference forward of the same sequence: the chosen token's reference
logit must be within a small margin of the reference maximum (the two paths sum in different orders, so exact ties may
break differently).  Prints `TP_SELFTEST_OK ranks=N` on success.
"""
from __future__ import annotations

import dataclasses
import sys

import numpy as np
import torch


def failure_main(leave_after: int) -> int:
    """Failure detection without a GPU fault: the last rank leaves between two steps (its stream drained, nothing in flight).  The leader
    must notice within seconds - either its next control broadcast fails on the host, or the kernels of its next step give up their
    bounded peer waits and report through the status words - and must NOT hang.  Prints TP_FAILURE_DETECTED on the leader."""
    import os
    import time
    from ..engine import BackendError, Engine, Request, StepError
    from ..engine.tp_backend import DenseTpBackend, follow
    from ..models import dense
    from ..sampling import GREEDY
    from . import runtime
    ctx = runtime.init(timeout_s=15)
    cfg = dataclasses.replace(dense.CONFIGS["test-hd128"], n_kv=4, name="tp-selftest")
    w = dense.random_weights(cfg, seed=11)
    shard, group = runtime.build_dense_tp(ctx, cfg, num_pages=32, max_rows=256, max_slots=4, max_blocks_per_seq=6, weights=w)
    if ctx.rank == ctx.world - 1 and ctx.rank != 0:
        follow(shard, 4, ctx.ctrl, leave_after=leave_after)
        torch.cuda.synchronize()
        os._exit(0)                      # gone: no goodbye message, no collective in flight
    if ctx.rank != 0:
        try:
            follow(shard, 4, ctx.ctrl)
        except Exception:
            pass
        os._exit(0)
    be = DenseTpBackend(shard, 4, ctx.ctrl)
    eng = Engine(be, None, window_rows=64, prefill_chunk=256, spec="none")
    eng.submit(Request("r", np.random.default_rng(3).integers(0, cfg.vocab, size=40).tolist(), 200, GREEDY))
    t0 = time.time()
    detected = ""
    try:
        for _ in range(400):
            if not eng.has_work():
                break
            for ev in eng.step():
                if ev.kind == "error":
                    detected = f"engine error event: {ev.message}"
            if detected:
                break
    except (StepError, BackendError, RuntimeError) as e:
        detected = f"{e.__class__.__name__}: {e}"
    dt = time.time() - t0
    if detected and dt < 60:
        print(f"TP_FAILURE_DETECTED after {dt:.1f} s: {detected[:200]}", flush=True)
        os._exit(0)
    print(f"the leader did not notice the lost rank ({dt:.1f} s, {detected!r})", file=sys.stderr, flush=True)
    os._exit(1)


def main() -> int:
    if "--leave-after" in sys.argv:
        return failure_main(int(sys.argv[sys.argv.index("--leave-after") + 1]))
    from ..engine.tp_backend import DenseTpBackend, follow
    from ..models import dense
    from . import runtime
    ctx = runtime.init(timeout_s=120)
    cfg = dataclasses.replace(dense.CONFIGS["test-hd128"], n_kv=4, name="tp-selftest")
    if cfg.n_q % ctx.world or cfg.n_kv % ctx.world:
        print(f"selftest model does not split over {ctx.world} ranks", file=sys.stderr)
        return 2
    w = dense.random_weights(cfg, seed=11)
    # --streams N: N concurrent sequences, so the decode windows have N rows (above 16 rows they leave the packet format for f32 rows
    # with flags, or for the in-switch reduction where an NVLS buffer is bound)
    streams = int(sys.argv[sys.argv.index("--streams") + 1]) if "--streams" in sys.argv else 3
    slots, max_blocks = max(4, streams), 6
    shard, group = runtime.build_dense_tp(ctx, cfg, num_pages=8 * slots, max_rows=256, max_slots=slots, max_blocks_per_seq=max_blocks, weights=w)
    if ctx.rank == 0:
        print(f"tp selftest: {streams} streams, NVLS buffer {'bound' if group.mm_mc_base else 'not bound'}", flush=True)
    rc = 0
    if ctx.rank != 0:
        follow(shard, slots, ctx.ctrl)
    else:
        be = DenseTpBackend(shard, slots, ctx.ctrl)
        try:
            rc = _lead(be, cfg, w, ctx, streams)
        finally:
            be.stop()
    runtime.shutdown(ctx, group)
    if ctx.rank == 0 and rc == 0:
        print(f"TP_SELFTEST_OK ranks={ctx.world}")
    return rc


def _lead(be, cfg, w, ctx, streams: int = 3) -> int:
    from ..engine import Engine, Request
    from ..models import dense
    from ..sampling import GREEDY
    rc = 0
    eng = Engine(be, None, window_rows=64, prefill_chunk=256, spec="none")
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in ([70, 33, 129] + [20 + 7 * i for i in range(max(0, streams - 3))])[:max(1, streams)]]
    new = 12
    for i, p in enumerate(prompts):
        eng.submit(Request(f"r{i}", p, new, GREEDY))
    out = {f"r{i}": [] for i in range(len(prompts))}
    for _ in range(400):
        if not eng.has_work():
            break
        for ev in eng.step():
            if ev.kind == "tokens":
                out[ev.id].extend(ev.tokens)
            elif ev.kind == "error":
                print("engine error:", ev.message, file=sys.stderr)
                rc = 1
    be.sync_all()
    ref = dense.ReferenceDense(w, device=ctx.device)
    worst = 0.0
    for i, p in enumerate(prompts):
        got = out[f"r{i}"]
        if len(got) != new:
            print(f"r{i}: {len(got)} tokens, wanted {new}", file=sys.stderr)
            rc = 1
            continue
        seq = p + got
        logits = ref.forward_seq(i, seq[:-1], 0)
        for j, t in enumerate(got):
            row = logits[len(p) - 1 + j]
            gap = float(row.max() - row[t]) / float(row.abs().max())
            worst = max(worst, gap)
            if gap > 0.02:
                print(f"r{i} token {j}: chose {t}, reference margin {gap:.4f}", file=sys.stderr)
                rc = 1
    st = be.stats()
    print(f"tp selftest: worst margin {worst:.5f}, graph replays {st['graph_replays']}, control bytes {be.ctrl_bytes}")
    if rc == 0 and "--trees" in sys.argv:
        rc = _lead_trees(be, cfg, prompts, out, new)
    return rc


def _lead_trees(be, cfg, prompts, serial: dict, new: int) -> int:
    """Tree rounds over the tensor-parallel group: the same prompts again with verify windows of draft trees.  The drafter knows the run
    above and hides the right token at a hashed rank of each level (or leaves it out), so accepted paths run through second and third
    candidates - private pages, ancestor copies and path moves on every rank.  The tokens must equal the first run's, bit for bit."""
    import hashlib
    from ..engine import DraftOffer, Engine, Request, TreeConfig
    from ..sampling import GREEDY
    from ..spec.tree import Lattice
    want = [serial[f"r{i}"] for i in range(len(prompts))]

    def propose(asks):
        offers = {}
        for a in asks:
            i = next(k for k, p in enumerate(prompts) if a.context[:len(p)] == p and len(a.context) - len(p) <= new)
            g = len(a.context) - len(prompts[i])
            ids = []
            for j in range(a.max_drafts):
                hsh = int.from_bytes(hashlib.blake2b(f"{i}.{g}.{j}".encode(), digest_size=8).digest(), "little")
                cand = [(hsh >> (8 * k)) % cfg.vocab for k in range(1, 5)]
                if g + j < len(want[i]) and hsh % 5 < 4:
                    cand[hsh % 5] = want[i][g + j]
                ids.append(cand)
            offers[a.slot] = DraftOffer([c[0] for c in ids], [], Lattice(ids, [[3.0, 2.0, 1.0, 0.0]] * len(ids)))
        return offers
    if not be.supports_trees():
        print("the tensor-parallel backend offers no tree windows", file=sys.stderr)
        return 1
    be.supports_native_draft = lambda: True
    be.propose_batch = propose
    eng = Engine(be, None, window_rows=64, prefill_chunk=256, spec="self", max_drafts=4, trees=TreeConfig(max_nodes=10))
    for i, p in enumerate(prompts):
        eng.submit(Request(f"t{i}", p, new, GREEDY))
    got = {f"t{i}": [] for i in range(len(prompts))}
    rc = 0
    for _ in range(400):
        if not eng.has_work():
            break
        for ev in eng.step():
            if ev.kind == "tokens":
                got[ev.id].extend(ev.tokens)
            elif ev.kind == "error":
                print("engine error (trees):", ev.message, file=sys.stderr)
                rc = 1
    be.sync_all()
    for i in range(len(prompts)):
        if got[f"t{i}"] != want[i]:
            print(f"trees: sequence {i} gave {got[f't{i}']}, the serial run {want[i]}", file=sys.stderr)
            rc = 1
    st = be.stats()
    if eng.counters.get("tree_rounds", 0) == 0 or eng.counters["accepted"] < 6 or st.get("tree_moves", 0) == 0:
        print(f"trees: nothing was exercised ({eng.counters}, {st})", file=sys.stderr)
        rc = 1
    print(f"tp selftest trees: rounds {eng.counters.get('tree_rounds')}, accepted {eng.counters['accepted']}, path moves {st.get('tree_moves')}, "
          f"row copies {st.get('tree_copies')}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
