"""Routing state, free of I/O: backends with probe / admin state and in-flight counts, the sticky affinity map, the choice.

Choice: the affinity key's sticky backend if it is routable and not overloaded past `max_skew` requests above the least
loaded one; else the least-outstanding backend, ties broken by rendezvous hash of (key, backend) so that several routers
agree.  Health: K consecutive probe failures take a backend out, M consecutive successes bring it back; the data path
takes it out at once on a refused connection or an engine-unavailable 503.
Behaviour parity: reference crates/router/src/main.rs:14-43, affinity.rs:1-25, backend.rs.
"""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field

from .keying import fnv64, rendezvous


@dataclass
class Backend:
    name: str
    url: str
    admin: str = "enabled"             # enabled | draining | disabled
    healthy: bool = True
    fails: int = 0
    oks: int = 0
    inflight: int = 0
    served: int = 0
    failed: int = 0
    uid: int = field(default=0)

    def __post_init__(self):
        self.uid = fnv64(self.name.encode())

    @property
    def routable(self) -> bool:
        return self.healthy and self.admin == "enabled"


class AffinityMap:
    """key -> backend name, bounded LRU with an idle TTL."""

    def __init__(self, cap: int = 65536, ttl_s: float = 1800.0, clock=time.monotonic):
        self.cap, self.ttl, self.clock = max(1, cap), ttl_s, clock
        self.map: "OrderedDict[int, tuple]" = OrderedDict()
        self.evicted_capacity = self.evicted_ttl = 0

    def get(self, key: int):
        e = self.map.get(key)
        if e is None:
            return None
        name, t = e
        if self.clock() - t > self.ttl:
            del self.map[key]
            self.evicted_ttl += 1
            return None
        self.map.move_to_end(key)
        self.map[key] = (name, self.clock())
        return name

    def put(self, key: int, name: str) -> None:
        self.map[key] = (name, self.clock())
        self.map.move_to_end(key)
        while len(self.map) > self.cap:
            self.map.popitem(last=False)
            self.evicted_capacity += 1

    def forget_backend(self, name: str) -> None:
        for k in [k for k, (n, _) in self.map.items() if n == name]:
            del self.map[k]

    def __len__(self):
        return len(self.map)


class Fleet:
    def __init__(self, backends=(), max_skew: int = 8, fail_after: int = 3, recover_after: int = 2, affinity: AffinityMap | None = None):
        self.backends: "OrderedDict[str, Backend]" = OrderedDict((b.name, b) for b in backends)
        self.max_skew, self.fail_after, self.recover_after = max_skew, fail_after, recover_after
        self.affinity = affinity or AffinityMap()
        self.counters = dict(requests=0, sticky_hits=0, sticky_moves=0, failovers=0, no_backend=0)

    # ---- selection
    def choose(self, key, exclude=()):
        cands = [b for b in self.backends.values() if b.routable and b.name not in exclude]
        if not cands:
            self.counters["no_backend"] += 1
            return None
        least = min(b.inflight for b in cands)
        if key is not None:
            name = self.affinity.get(key)
            b = self.backends.get(name) if name else None
            if b is not None and b.routable and b.name not in exclude and b.inflight - least <= self.max_skew:
                self.counters["sticky_hits"] += 1
                return b
            if b is not None:
                self.counters["sticky_moves"] += 1
        best = [b for b in cands if b.inflight == least]
        pick = max(best, key=lambda b: rendezvous(key or 0, b.uid)) if len(best) > 1 else best[0]
        if key is not None:
            self.affinity.put(key, pick.name)
        return pick

    def begin(self, b: Backend) -> None:
        b.inflight += 1
        self.counters["requests"] += 1

    def end(self, b: Backend, ok: bool) -> None:
        b.inflight = max(0, b.inflight - 1)
        if ok:
            b.served += 1
        else:
            b.failed += 1

    # ---- health
    def probe_result(self, name: str, ok: bool) -> None:
        b = self.backends.get(name)
        if b is None:
            return
        if ok:
            b.oks, b.fails = b.oks + 1, 0
            if not b.healthy and b.oks >= self.recover_after:
                b.healthy = True
        else:
            b.fails, b.oks = b.fails + 1, 0
            if b.healthy and b.fails >= self.fail_after:
                b.healthy = False

    def data_path_down(self, name: str) -> None:
        """A refused connection or an engine-unavailable 503: out at once, the prober brings it back."""
        b = self.backends.get(name)
        if b is not None:
            b.healthy, b.oks, b.fails = False, 0, self.fail_after

    # ---- admin
    def add(self, name: str, url: str) -> Backend:
        if name in self.backends:
            raise ValueError(f"backend {name!r} exists")
        b = Backend(name, url.rstrip("/"))
        self.backends[name] = b
        return b

    def remove(self, name: str) -> None:
        if self.backends.pop(name, None) is None:
            raise KeyError(name)
        self.affinity.forget_backend(name)

    def set_admin(self, name: str, state: str) -> None:
        if state not in ("enabled", "draining", "disabled"):
            raise ValueError(state)
        self.backends[name].admin = state

    def health(self) -> dict:
        return {"ok": any(b.routable for b in self.backends.values()),
                "backends": [dict(name=b.name, url=b.url, healthy=b.healthy, admin=b.admin, inflight=b.inflight, served=b.served, failed=b.failed)
                             for b in self.backends.values()]}
