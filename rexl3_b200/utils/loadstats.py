"""Process-wide load-stage timers: seconds, bytes and calls per (component, stage), filled while a pack is read, decoded and uploaded, and
rendered as `rexl3_load_stage_seconds / _bytes / _calls` metric lines.  Role of the reference's loader phase timers
(crates/exl3/src/loadstats.rs:1-12): a slow boot says which stage of which component took the time."""
from __future__ import annotations

import threading
import time
from contextlib import contextmanager

_lock = threading.Lock()
_stats = {}          # (component, stage) -> [seconds, bytes, calls]


@contextmanager
def stage(component: str, name: str, nbytes: int = 0):
    t = time.perf_counter()
    try:
        yield
    finally:
        add(component, name, time.perf_counter() - t, nbytes)


def add(component: str, name: str, seconds: float, nbytes: int = 0) -> None:
    with _lock:
        s = _stats.setdefault((component, name), [0.0, 0, 0])
        s[0] += seconds
        s[1] += int(nbytes)
        s[2] += 1


def snapshot() -> dict:
    with _lock:
        return {k: tuple(v) for k, v in _stats.items()}


def reset() -> None:
    with _lock:
        _stats.clear()


def render() -> str:
    lines = []
    for (c, s), (sec, nb, calls) in sorted(snapshot().items()):
        lab = f'{{component="{c}",stage="{s}"}}'
        lines += [f"rexl3_load_stage_seconds{lab} {sec:g}", f"rexl3_load_stage_bytes{lab} {nb}", f"rexl3_load_stage_calls{lab} {calls}"]
    return "\n".join(lines) + ("\n" if lines else "")
