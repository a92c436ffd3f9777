"""The engine thread: the only thread that touches the model.  HTTP handlers talk to it through a command queue and get
tokens back over per-request asyncio queues.

FIFO admission with a bounded queue, queue / request deadlines, consecutive-error counters (degraded after
``unready_after``, exit after ``exit_after``), a progress heartbeat a watchdog can check, graceful drain.  "Never a zombie":
a fatal backend error ends the loop and fails every request.  Behaviour parity: reference crates/server/src/runtime.rs:1-11,
:603 (spawn_with), :772-900 (run loop), :1001-1252 (enqueue / admit / route), main.rs:978-990 (watchdog).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass, field

from ..engine import Engine, Request, StepError
from ..sched import AdmitError


@dataclass
class RuntimeConfig:
    queue_depth: int = 64
    queue_timeout_s: float = 300.0
    request_timeout_s: float = 1800.0
    unready_after: int = 3
    exit_after: int = 10
    idle_sleep_s: float = 0.002
    shutdown_grace_s: float = 8.0


@dataclass
class Ticket:
    id: str
    loop: asyncio.AbstractEventLoop
    out: asyncio.Queue
    t_submit: float = field(default_factory=time.monotonic)
    t_first: float | None = None
    closed: bool = False

    def post(self, msg) -> None:
        if not self.closed:
            self.loop.call_soon_threadsafe(self.out.put_nowait, msg)


class Metrics:
    """Process-wide counters and 1 ms * 2^k latency histograms, rendered as Prometheus text."""

    BUCKETS = [0.001 * 2 ** k for k in range(18)]

    def __init__(self):
        self.lock = threading.Lock()
        self.counters = {}
        self.gauges = {}
        self.hist = {}
        self.t_boot = time.time()

    def inc(self, name, v=1.0, **labels):
        with self.lock:
            k = (name, tuple(sorted(labels.items())))
            self.counters[k] = self.counters.get(k, 0.0) + v

    def set(self, name, v, **labels):
        with self.lock:
            self.gauges[(name, tuple(sorted(labels.items())))] = float(v)

    def observe(self, name, v):
        with self.lock:
            h = self.hist.setdefault(name, [[0] * (len(self.BUCKETS) + 1), 0.0, 0])
            i = next((j for j, b in enumerate(self.BUCKETS) if v <= b), len(self.BUCKETS))
            h[0][i] += 1
            h[1] += v
            h[2] += 1

    @staticmethod
    def _lab(labels):
        return "{" + ",".join(f'{k}="{v}"' for k, v in labels) + "}" if labels else ""

    def render(self) -> str:
        with self.lock:
            lines = []
            for (n, l), v in sorted(self.counters.items()):
                lines.append(f"rexl3_{n}{self._lab(l)} {v:g}")
            for (n, l), v in sorted(self.gauges.items()):
                lines.append(f"rexl3_{n}{self._lab(l)} {v:g}")
            for n, (counts, total, cnt) in sorted(self.hist.items()):
                acc = 0
                for b, c in zip(self.BUCKETS, counts):
                    acc += c
                    lines.append(f'rexl3_{n}_bucket{{le="{b:g}"}} {acc}')
                lines.append(f'rexl3_{n}_bucket{{le="+Inf"}} {cnt}')
                lines.append(f"rexl3_{n}_sum {total:g}")
                lines.append(f"rexl3_{n}_count {cnt}")
            lines.append(f"rexl3_uptime_seconds {time.time() - self.t_boot:g}")
            return "\n".join(lines) + "\n"


class EngineHandle:
    """Owns the engine thread.  States: loading -> ready -> (degraded) -> draining -> stopped | failed."""

    def __init__(self, make_engine, cfg: RuntimeConfig | None = None, metrics: Metrics | None = None):
        self.cfg = cfg or RuntimeConfig()
        self.metrics = metrics or Metrics()
        for kind in ("Backend", "Fatal", "BackendShape"):        # error counters exist from the start: a dashboard sees 0, not "no data"
            self.metrics.inc("step_errors_total", 0.0, kind=kind)
        self.cmd: "queue.Queue" = queue.Queue()
        self.state = "loading"
        self.error = ""
        self.tickets = {}
        self.pending = 0                 # queued + running requests; written by HTTP threads and by the engine thread, always under _plock
        self._plock = threading.Lock()
        self.heartbeat = time.monotonic()
        self.engine: Engine | None = None
        self.consecutive_errors = 0
        self._make = make_engine
        self._ready = threading.Event()
        self.thread = threading.Thread(target=self._run, name="rexl3-engine", daemon=True)
        self.thread.start()

    # ------------------------------------------------------------------ called from HTTP handlers
    def wait_ready(self, timeout: float | None = None) -> bool:
        self._ready.wait(timeout)
        return self.state in ("ready", "degraded")

    def submit(self, req: Request, loop: asyncio.AbstractEventLoop) -> Ticket:
        if self.state not in ("ready", "degraded"):
            raise RuntimeError(self.state)
        with self._plock:
            if self.pending >= self.cfg.queue_depth:
                raise OverflowError("queue full")
            self.pending += 1
        t = Ticket(req.id, loop, asyncio.Queue())
        if req.deadline is None:
            req.deadline = time.monotonic() + self.cfg.request_timeout_s
        self.cmd.put(("submit", req, t))
        return t

    def score(self, tokens: list, loop: asyncio.AbstractEventLoop) -> "asyncio.Future":
        """Full-vocabulary logits after `tokens`, computed by the engine thread between steps.  The future resolves to a float32 array or
        raises (AdmitError when every slot is busy, a backend error)."""
        if self.state not in ("ready", "degraded"):
            raise RuntimeError(self.state)
        fut = loop.create_future()
        self.cmd.put(("score", tokens, (loop, fut)))
        return fut

    def cancel(self, rid: str) -> None:
        self.cmd.put(("cancel", rid, None))

    def drain(self) -> None:
        self.cmd.put(("drain", None, None))

    def wedged(self, stale_s: float = 60.0) -> bool:
        """True when there is work but the loop has made no progress for `stale_s` (a watchdog aborts the process on this)."""
        return self.state in ("ready", "degraded") and self.pending > 0 and time.monotonic() - self.heartbeat > stale_s

    # ------------------------------------------------------------------ the engine thread
    def _done_one(self) -> None:
        with self._plock:
            self.pending = max(0, self.pending - 1)

    def _fail_all(self, message: str) -> None:
        for t in list(self.tickets.values()):
            t.post(("error", message))
        self.tickets.clear()
        with self._plock:
            self.pending = 0

    def _run(self) -> None:
        try:
            self.engine = self._make()
            self.state = "ready"
        except Exception as e:  # boot failure: report, never serve
            self.state, self.error = "failed", f"{e.__class__.__name__}: {e}"
            self._ready.set()
            return
        self._ready.set()
        eng, m = self.engine, self.metrics
        draining, t_drain = False, 0.0
        while True:
            try:
                while True:
                    kind, a, b = self.cmd.get_nowait() if (eng.has_work() or draining) else self.cmd.get(timeout=0.05)
                    if kind == "submit":
                        if draining:
                            b.post(("error", "draining"))
                            self._done_one()
                            continue
                        try:
                            eng.submit(a)
                            self.tickets[a.id] = b
                            m.inc("requests_total")
                        except (ValueError, AdmitError) as e:
                            code = "context_length_exceeded" if isinstance(e, AdmitError) and e.kind in ("ContextTooLong", "NeverFits") else "invalid"
                            b.post(("refused", code, str(e)))
                            self._done_one()
                    elif kind == "score":
                        loop, fut = b
                        try:
                            row = eng.score_prompt(a)
                            loop.call_soon_threadsafe(lambda f=fut, r=row: f.done() or f.set_result(r))
                            m.inc("decisions_total", status="completed")
                        except Exception as e:   # the caller's problem (no slot, too long), never the loop's
                            loop.call_soon_threadsafe(lambda f=fut, e=e: f.done() or f.set_exception(e))
                            m.inc("decisions_total", status="refused")
                    elif kind == "cancel":
                        eng.cancel(a)
                    elif kind == "drain":
                        draining, t_drain = True, time.monotonic()
                        self.state = "draining"
                    elif kind == "stop":
                        self._fail_all("stopped")
                        self.state = "stopped"
                        return
            except queue.Empty:
                pass
            if eng.events:                      # a cancel finishes a request outside step(): deliver it now
                self._route(eng.take_events())
            if draining and (not eng.has_work() or time.monotonic() - t_drain > self.cfg.shutdown_grace_s):
                self._fail_all("draining")
                self.state = "stopped"
                return
            if not eng.has_work():
                self.heartbeat = time.monotonic()
                continue
            try:
                t0 = time.perf_counter()
                events = eng.step()
                m.observe("step_seconds", time.perf_counter() - t0)
                self.consecutive_errors = 0
                if self.state == "degraded":
                    self.state = "ready"
            except StepError as e:
                events = eng.take_events()
                m.inc("step_errors_total", kind=e.kind)
                self.consecutive_errors += 1
                if e.fatal or self.consecutive_errors >= self.cfg.exit_after:
                    self._route(events)
                    self._fail_all(str(e))
                    # a lost rank takes the whole group down (fail-stop): health answers 503 `group_lost` until a supervisor restarts all ranks
                    self.state, self.error = ("group_lost" if getattr(e, "group_lost", False) else "failed"), str(e)
                    if self.state == "group_lost":
                        m.inc("tp_group_lost_total")
                        m.set("tp_group_up", 0)
                    return
                if self.consecutive_errors >= self.cfg.unready_after:
                    self.state = "degraded"
            except Exception as e:  # a bug in the loop must not leave a zombie that accepts requests
                self._fail_all(f"internal error: {e.__class__.__name__}: {e}")
                self.state, self.error = "failed", f"{e.__class__.__name__}: {e}"
                return
            self.heartbeat = time.monotonic()
            self._route(events)
            c = eng.counters
            m.set("active_sequences", eng.active_count())
            m.set("queued_requests", len(eng.waiting))
            for k in ("decode_tokens", "prefill_tokens", "drafted", "accepted", "rounds", "cached_tokens", "spilled_blocks", "unspilled_blocks"):
                m.set(f"engine_{k}_total", c.get(k, 0))
            m.set("round_streams_total", c.get("round_streams", 0))
            m.set("round_draft_streams_total", c.get("round_draft_streams", 0))
            m.set("round_verify_rows_total", c.get("rows", 0))
            for phase, ns in eng.phase_ns.items():
                m.set("round_phase_seconds_total", ns / 1e9, phase=phase)
            for j in range(len(eng.spec_pos["offered"])):
                for k in ("offered", "reached", "accepted"):
                    m.set(f"spec_position_{k}_total", eng.spec_pos[k][j], position=str(j + 1))
            for mode, ps in getattr(eng, "position_stats", {}).items():
                m.set("spec_rounds_by_mode_total", ps.rounds, mode=mode)
                m.set("spec_verify_rows_wasted_total", ps.wasted_rows(), mode=mode)
            mb = getattr(eng, "margin_bins", None)
            if mb is not None:
                for b in range(len(mb.reached)):
                    if mb.reached[b]:
                        m.set("spec_margin_reached_total", mb.reached[b], bin=str(b))
                        m.set("spec_margin_accepted_total", mb.accepted[b], bin=str(b))
            for k in ("tree_rounds", "tree_nodes", "tree_depth_kept"):        # draft-tree rounds: windows, nodes verified, accepted path lengths
                m.set(f"spec_{k}_total", c.get(k, 0))
            self._backend_metrics(eng.backend)
            if eng.admission is not None:
                m.set("admission_bytes_capacity", getattr(eng.admission, "capacity", 0))
                m.set("admission_bytes_used", getattr(eng.admission, "used", 0))
            if eng.prefix is not None:
                m.set("prefix_cache_bytes", eng.prefix.bytes)
                m.set("prefix_cache_entries", len(eng.prefix))
                m.set("prefix_cache_reach_tokens", eng.prefix.reach_tokens())
                for k in ("lookups", "hits", "hit_blocks", "inserts", "evictions", "ghost_hits"):
                    m.set(f"prefix_cache_{k}_total", eng.prefix.stats[k])
            if getattr(eng, "spill", None) is not None:
                m.set("prefix_spill_bytes", eng.spill.bytes)
                m.set("prefix_spill_entries", len(eng.spill))

    def _backend_metrics(self, backend) -> None:
        """Gauges a backend offers through `stats()`: CUDA-graph cache, KV pool, control-plane traffic of a tensor-parallel group."""
        m = self.metrics
        m.set("slots_total", getattr(backend, "max_slots", 0))
        try:
            st = backend.stats() if hasattr(backend, "stats") else {}
        except Exception:
            st = {}
        m.set("graph_cache_replays_total", st.get("graph_replays", 0))
        m.set("graph_cache_captures_total", st.get("graph_captures", 0))
        m.set("graph_cache_replayed_kernels_total", st.get("replayed_kernels", 0))
        m.set("backend_h2d_bytes_total", st.get("h2d_bytes", 0))
        m.set("backend_d2h_bytes_total", st.get("d2h_bytes", 0))
        pool = getattr(backend, "pool", None)
        if pool is not None and hasattr(pool, "free_blocks"):
            total = pool.total_blocks() if hasattr(pool, "total_blocks") else 0
            bt = getattr(pool, "block_tokens", 64)
            m.set("kv_pool_tokens", total * bt)
            m.set("kv_pool_tokens_used", max(0, total - pool.free_blocks()) * bt)
        m.set("tp_ranks", st.get("tp_ranks", 1))
        m.set("tp_group_up", 0 if self.state == "group_lost" else 1)
        m.set("tp_commands_sent_total", st.get("tp_commands", 0))
        m.set("tp_sent_bytes_total", st.get("ctrl_bytes", 0))
        m.set("commit_replays_total", st.get("commit_replays", 0))
        m.set("backend_tree_windows_total", st.get("tree_windows", 0))
        m.set("backend_tree_row_copies_total", st.get("tree_copies", 0) + st.get("tree_moves", 0))
        m.set("backend_image_rows_total", st.get("media_rows", 0))
        if "expert_slots" in st:            # routed experts paged from a record file
            m.set("expert_cache_slots", st["expert_slots"])
            m.set("expert_cache_resident", st.get("expert_resident", 0))
            for k in ("hits", "misses", "bytes_read", "evictions", "hint_fills", "hint_drops", "asked", "cold"):
                m.set(f"expert_cache_{k}_total", st.get("expert_" + k, 0))

    def _route(self, events) -> None:
        for ev in events:
            t = self.tickets.get(ev.id)
            if t is None:
                continue
            if ev.kind == "tokens":
                now = time.monotonic()
                if t.t_first is None:
                    t.t_first = now
                    self.metrics.observe("ttft_seconds", t.t_first - t.t_submit)
                else:
                    self.metrics.observe("token_batch_itl_seconds", now - getattr(t, "t_last", now))
                t.t_last = now
                self.metrics.inc("token_batches_total")
                self.metrics.inc("generated_tokens_total", len(ev.tokens))
                t.post(("tokens", ev.tokens))
            else:
                if ev.kind == "done":
                    t.post(("done", ev.reason, ev.usage))
                    self.metrics.observe("e2e_seconds", time.monotonic() - t.t_submit)
                    self.metrics.inc("finished_total", reason=ev.reason)
                else:
                    t.post(("error", ev.message or ev.reason))
                    self.metrics.inc("finished_total", reason="error")
                self.tickets.pop(ev.id, None)
                self._done_one()

    def stop(self) -> None:
        self.cmd.put(("stop", None, None))
        self.thread.join(timeout=10)
