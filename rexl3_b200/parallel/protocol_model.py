"""A CPU model of the push-based collective protocol, explored exhaustively over every interleaving of a few ranks.

What is modelled (the rules `ops/csrc/tp.cuh` and `comm.cu` implement on the GPU): every rank runs the same numbered sequence of
collectives.  In collective c a rank (1) pushes its contribution into slot set `c % sets` of EVERY rank (peers and itself), either as
self-validating packets carrying the ticket c, or as plain data followed by a flag write of ticket c; (2) waits until its own slot set
holds ticket c from every source; (3) reads the contributions one source at a time; then moves on to c + 1.  Nothing else orders the
ranks: a fast rank may start pushing c + 1 (and, with enough sets, c + 2) while a slow one is still reading c.

The safety property: when a rank reads source s in collective c, that slot still holds s's contribution for c (a later push must not
have overwritten it: the write-after-read hazard).  `explore` walks every reachable state (depth-first, memoised) and returns the first
violating trace or None.  Two slot sets are safe and one is not; with flags, publishing the flag before the data is not.  The model is
how a change to the slot / ticket scheme is checked before any GPU runs it.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Protocol:
    ranks: int = 2
    collectives: int = 4
    sets: int = 2                 # slot sets alternating per collective
    flags: bool = False           # False: self-validating packets (data and ticket in one store); True: data store, then flag store
    flag_first: bool = False      # (mutation) publish the flag before the data


def _program(p: Protocol, r: int) -> list:
    """The step list of rank r: tuples (op, collective, other rank)."""
    prog = []
    for c in range(p.collectives):
        for dst in range(p.ranks):
            if p.flags:
                steps = [("data", c, dst), ("flag", c, dst)]
                prog += steps[::-1] if p.flag_first else steps
            else:
                prog.append(("packet", c, dst))
        prog.append(("wait", c, r))
        for src in range(p.ranks):
            prog.append(("read", c, src))
    return prog


def explore(p: Protocol, max_states: int = 2_000_000):
    """-> None when no interleaving violates the property, else (message, trace) with the trace as a list of (rank, step)."""
    progs = [_program(p, r) for r in range(p.ranks)]
    R, S = p.ranks, p.sets
    # memory: data[dst][set][src] and flag[dst][set][src] hold the ticket last written (-1: never)
    init_mem = tuple(-1 for _ in range(R * S * R * 2))
    idx = lambda kind, dst, st, src: ((kind * R + dst) * S + st) * R + src  # noqa: E731  kind 0 = data, 1 = flag
    start = (tuple(0 for _ in range(R)), init_mem)
    seen = {start}
    stack = [(start, [])]
    while stack:
        (pcs, mem), trace = stack.pop()
        if all(pcs[r] == len(progs[r]) for r in range(R)):
            continue
        progressed = False
        for r in range(R):
            if pcs[r] == len(progs[r]):
                continue
            op, c, other = progs[r][pcs[r]]
            st = c % S
            m = list(mem)
            if op == "packet":
                m[idx(0, other, st, r)] = c
                m[idx(1, other, st, r)] = c
            elif op == "data":
                m[idx(0, other, st, r)] = c
            elif op == "flag":
                m[idx(1, other, st, r)] = c
            elif op == "wait":
                if any(mem[idx(1, r, st, src)] < c for src in range(R)):
                    continue                                   # not enabled yet
                if any(mem[idx(1, r, st, src)] > c for src in range(R)):
                    return (f"rank {r} waiting for collective {c} finds a later ticket in its slot set: the contribution it needs is gone",
                            trace + [(r, progs[r][pcs[r]])])
            elif op == "read":
                if mem[idx(0, r, st, other)] != c:
                    return (f"rank {r} reads source {other} in collective {c} but the slot holds ticket {mem[idx(0, r, st, other)]}",
                            trace + [(r, progs[r][pcs[r]])])
            progressed = True
            nxt = (tuple(pcs[i] + (1 if i == r else 0) for i in range(R)), tuple(m))
            if nxt not in seen:
                if len(seen) >= max_states:
                    raise RuntimeError("state budget exceeded: shrink the model")
                seen.add(nxt)
                stack.append((nxt, trace + [(r, progs[r][pcs[r]])]))
        if not progressed:
            return ("deadlock: no rank can take a step", trace)
    return None
