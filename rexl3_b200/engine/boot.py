"""Boot phase registry: named phases of bringing an engine up (scan, plan, load, graphs, ready), with wall time and an outcome, so that
a slow or failed boot says where it was.  Shown under `/health` and logged one line per phase.  Parity: the reference's boot phase
registry in crates/engine (phases are data, not log archaeology)."""
from __future__ import annotations

import sys
import time
from contextlib import contextmanager


class BootPhases:
    def __init__(self, log=None):
        self.phases = []                 # dict(name, seconds, ok, detail)
        self.current = None
        self.t0 = time.monotonic()
        self.log = log if log is not None else (lambda s: print(s, file=sys.stderr, flush=True))

    @contextmanager
    def phase(self, name: str, **detail):
        t = time.monotonic()
        self.current = name
        try:
            yield
        except BaseException as e:
            self.phases.append(dict(name=name, seconds=round(time.monotonic() - t, 3), ok=False, detail={**detail, "error": f"{e.__class__.__name__}: {e}"}))
            self.log(f"rexl3 level=error event=boot_phase name={name} ok=false seconds={time.monotonic() - t:.3f} error={e!r}")
            self.current = None
            raise
        self.phases.append(dict(name=name, seconds=round(time.monotonic() - t, 3), ok=True, detail=detail))
        self.log(f"rexl3 event=boot_phase name={name} ok=true seconds={time.monotonic() - t:.3f}")
        self.current = None

    def report(self) -> dict:
        return {"total_seconds": round(time.monotonic() - self.t0, 3), "current": self.current, "phases": list(self.phases)}
