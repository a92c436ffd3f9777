"""Tensor-parallel boot gate: before any rank allocates its shard, every rank states what it is about to run as a flat dict of facts
(model config, pack fingerprint, kernel-library hash, the flags that shape the lockstep schedule), the facts are gathered over the
CPU control group, and every rank refuses to start unless all of them agree.  A group whose ranks differ would not fail at boot: it
would deadlock in a collective or, worse, decode garbage.  Role of the reference's TP boot gate (facts compared across ranks,
crates/model/src/families/nemotron_h_omni/tp_boot.rs).
"""
from __future__ import annotations

import hashlib
import json
import os


class BootGateError(RuntimeError):
    pass


def file_sha256(path: str, limit: int | None = None) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        left = limit
        while True:
            chunk = f.read(8 << 20 if left is None else min(8 << 20, left))
            if not chunk:
                break
            h.update(chunk)
            if left is not None:
                left -= len(chunk)
                if left <= 0:
                    break
    return h.hexdigest()


def collect_facts(cfg, *, world: int, pack: str | None = None, flags: dict | None = None, libraries=None) -> dict:
    """What this rank is about to run.  `flags`: the serve options every rank must share (slots, window rows, prefill chunk, KV dtype,
    graphs on/off, collective schedule...)."""
    from dataclasses import asdict, is_dataclass
    facts = {"world": int(world)}
    c = asdict(cfg) if is_dataclass(cfg) else dict(cfg)
    facts["config"] = hashlib.sha256(json.dumps(c, sort_keys=True, default=str).encode()).hexdigest()[:16]
    facts["model"] = c.get("name", "?")
    if pack:
        from ..format import verify
        facts["pack_fingerprint"] = verify.fingerprint(pack)[:16]
    if libraries is None:
        from ..ops import lib as oplib
        libraries = [oplib.LIB_PATH]
    for p in libraries:
        facts["lib:" + os.path.basename(p)] = file_sha256(p)[:16] if os.path.exists(p) else "missing"
    for k, v in sorted((flags or {}).items()):
        facts["flag:" + k] = v
    return facts


def compare(all_facts: list) -> list:
    """Differences against rank 0, as readable lines (empty = the group agrees)."""
    out = []
    base = all_facts[0]
    for r, f in enumerate(all_facts[1:], start=1):
        for k in sorted(set(base) | set(f)):
            if base.get(k) != f.get(k):
                out.append(f"rank {r}: {k} = {f.get(k)!r}, rank 0 has {base.get(k)!r}")
    return out


def gate(facts: dict, group=None) -> list:
    """Gather every rank's facts over `group` (a CPU process group) and raise BootGateError on every rank if any differ.
    Returns the gathered list (rank order)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    gathered = [None] * world
    dist.all_gather_object(gathered, facts, group=group)
    diffs = compare(gathered)
    if diffs:
        raise BootGateError("tensor-parallel boot gate: the ranks do not agree: " + "; ".join(diffs[:6]) + (f" (+{len(diffs) - 6} more)" if len(diffs) > 6 else ""))
    return gathered
