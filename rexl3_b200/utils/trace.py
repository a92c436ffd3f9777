"""Opt-in host-side tracing with no cost when off.

* `REXL3_TP_TRACE=1`: a timeline of the tensor-parallel control plane.  Every leader / follower event becomes one line
  `TPTRACE <L|F> <ns> <rank> <tag> <arg>` on stderr, written by a flusher thread so the step loop only appends to a queue (the
  reference's host timeline, crates/model/src/hosttrace.rs:1-10).
* `REXL3_NVTX=1`: NVTX ranges around the engine's phases (draft / verify / prefill / sample) for a profiler's timeline.
"""
from __future__ import annotations

import os
import queue
import sys
import threading
import time
from contextlib import contextmanager

TP_TRACE = os.environ.get("REXL3_TP_TRACE", "") not in ("", "0")
NVTX = os.environ.get("REXL3_NVTX", "") not in ("", "0")

_q: "queue.SimpleQueue | None" = None
_out = None


def _flusher():
    while True:
        item = _q.get()
        if item is None:
            break
        (_out or sys.stderr).write(item)
        if _q.empty():
            (_out or sys.stderr).flush()


def enable_tp_trace(stream=None) -> None:
    """Turn the TP timeline on (tests pass a stream; production sets REXL3_TP_TRACE)."""
    global TP_TRACE, _q, _out
    TP_TRACE, _out = True, stream
    if _q is None:
        _q = queue.SimpleQueue()
        threading.Thread(target=_flusher, daemon=True, name="tptrace").start()


def tp_event(role: str, rank: int, tag: str, arg=0) -> None:
    if not TP_TRACE:
        return
    if _q is None:
        enable_tp_trace(_out)
    _q.put(f"TPTRACE {role} {time.monotonic_ns()} {rank} {tag} {arg}\n")


def flush_tp_trace(timeout_s: float = 1.0) -> None:
    t = time.monotonic() + timeout_s
    while _q is not None and not _q.empty() and time.monotonic() < t:
        time.sleep(0.001)
    time.sleep(0.005)
    (_out or sys.stderr).flush()


@contextmanager
def nvtx_range(name: str):
    if not NVTX:
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
