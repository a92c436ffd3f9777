"""Group-aware supervisor: a tensor-parallel group is one unit - any rank that exits takes the attempt down, the exit codes of ALL
ranks classify the attempt, and the whole group is restarted (with backoff) or stopped.  The policy is pure and tested without
a process; `supervise` drives it over a runner.  Exit-code map (parity: reference crates/cluster/src/supervise.rs:1-25):

  0 clean stop -> no restart | 70 group lost / fatal backend error -> restart all, backoff | 101 engine-thread panic -> restart once,
  the second in a row stops | 134, 137, 143, 128+n killed -> restart all, backoff | 1 before ready: refused boot -> refusal;
  after ready -> restart | 2, 3 usage error / memory guard -> refusal | 75 GPU lock not free -> restart, backoff.
Give-up: two refusals in a row (exit status 78), or more than `max_failures` failed attempts inside `window_s` (exit status 75).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field


@dataclass
class Attempt:
    codes: list                 # exit code per rank (None: still running when the attempt was torn down)
    ready: bool                 # the group reached /health/ready before the first exit
    runtime_s: float = 0.0


@dataclass
class Policy:
    backoff_s: list = field(default_factory=lambda: [1.0, 2.0, 5.0, 15.0, 30.0])
    window_s: float = 600.0
    max_failures: int = 5


def classify(a: Attempt) -> str:
    """-> "clean" | "restart" | "restart_once" | "refusal"."""
    codes = [c for c in a.codes if c is not None]
    if codes and all(c == 0 for c in codes):
        return "clean"
    bad = [c for c in codes if c != 0]
    if any(c in (2, 3) for c in bad):
        return "refusal"
    if any(c == 1 for c in bad) and not a.ready:
        return "refusal"
    if any(c == 101 for c in bad) and not any(c in (70, 134, 137, 143) or c > 128 for c in bad):
        return "restart_once"
    return "restart"


def supervise(run_attempt, policy: Policy | None = None, sleep=time.sleep, clock=time.monotonic, log=print, max_attempts: int = 1_000_000) -> int:
    """`run_attempt()` starts every rank, waits for the first exit, stops the rest and returns an Attempt.  Returns the supervisor's
    exit status: 0 clean stop, 78 refused twice in a row, 75 too many failures in the window."""
    p = policy or Policy()
    failures = []          # times of failed attempts inside the window
    last = None
    streak = 0
    for n in range(max_attempts):
        a = run_attempt()
        kind = classify(a)
        log(f"rexl3-cluster event=attempt_end n={n} kind={kind} codes={a.codes} ready={a.ready}")
        if kind == "clean":
            return 0
        now = clock()
        failures = [t for t in failures if now - t <= p.window_s] + [now]
        if kind == "refusal" and last == "refusal":
            return 78
        if kind == "restart_once" and last == "restart_once":
            return 78
        if len(failures) > p.max_failures:
            return 75
        streak = streak + 1 if a.runtime_s < 60 else 1       # a group that ran for a while starts the backoff ladder again
        sleep(p.backoff_s[min(streak - 1, len(p.backoff_s) - 1)])
        last = kind
    return 75


class LocalRunner:
    """Runs the ranks of a group as child processes of this host (one NVLink box).  The first exit tears the others down by pid."""

    def __init__(self, commands, ready_probe=None, log_dir: str = "", max_runtime_s: float = 0.0, on_start=None):
        """`on_start(pids)`: called with the ranks' pids once they are started (the CLI records them in the group's state file)."""
        self.commands, self.ready_probe, self.log_dir, self.max_runtime_s = commands, ready_probe, log_dir, max_runtime_s
        self.on_start = on_start

    def __call__(self) -> Attempt:
        import os
        import signal
        import subprocess
        procs = []
        t0 = time.monotonic()
        for r, (env, argv) in enumerate(self.commands):
            out = open(os.path.join(self.log_dir, f"rank{r}.log"), "ab") if self.log_dir else None
            procs.append(subprocess.Popen(argv, env={**os.environ, **env}, stdout=out, stderr=subprocess.STDOUT if out else None, start_new_session=True))
        if self.on_start is not None:
            self.on_start([p.pid for p in procs])
        ready = False
        try:
            while True:
                codes = [p.poll() for p in procs]
                if any(c is not None for c in codes):
                    break
                if not ready and self.ready_probe is not None:
                    ready = bool(self.ready_probe())
                if self.max_runtime_s and time.monotonic() - t0 > self.max_runtime_s:
                    procs[0].send_signal(signal.SIGTERM)      # rank 0 first: the followers exit 0 on its shutdown
                    self.max_runtime_s = 0.0
                time.sleep(0.2)
        finally:
            for p in procs:
                if p.poll() is None:
                    p.send_signal(signal.SIGTERM)
            for p in procs:
                try:
                    p.wait(timeout=15)
                except subprocess.TimeoutExpired:
                    p.kill()
                    p.wait()
        final = [p.returncode if p.returncode is None or p.returncode >= 0 else 128 - p.returncode for p in procs]
        return Attempt(final, ready, time.monotonic() - t0)
