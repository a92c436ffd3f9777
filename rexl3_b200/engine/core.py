"""The engine step loop: deferred submit -> prefill slices (serial / burst) -> decode / verify rounds -> commit or
rollback -> events.

One ``step()`` is one scheduling iteration: a decode round over every active sequence (one window whose rows are, per
sequence, its last token plus its drafts), then prefill work for sequences still reading their prompt.  Sampling is the
keyed sampler on the CPU over the backend's top candidates; a draft is accepted iff it equals the keyed sample at its
position, so drafted == serial by construction.  Behaviour parity: reference crates/engine/src/lib.rs:1715-2200
(step / step_inner / decode_round), :1169-1626 (submit, prefill slices, prefix planning), :548-637 (Request / Event /
FinishReason), :724-803 (BudgetPolicy, PrefillPolicy).
"""
from __future__ import annotations

import numpy as np  # noqa: F401  (type of score rows)

import math
import time
from collections import deque
from dataclasses import dataclass, field

from ..sampling import Sampling, SamplingError, choose, seed_for
from ..sched import AdmitError, Admission, CostModel, Demand, PrefixIndex, chain_hashes, choose_budget
from ..spec import AcceptStats, CopyDrafter, NgramDrafter, SpecMode, accept
from ..utils import trace
from .backend import Backend, BackendError, DraftAsk, RowRequest

PREFILL_STEP_ROWS = 4096
PREFILL_PASS_GUARD = 8       # steps after which a prompt that keeps being passed over for shorter ones is served first


@dataclass
class Request:
    id: str
    prompt: list
    max_new_tokens: int = 256
    sampling: Sampling = None
    stop_ids: tuple = ()
    draft: bool = True
    prefix_cache: bool = True
    deadline: float | None = None       # absolute time.monotonic() after which the request is cancelled
    # reasoning budget: at most `reasoning_budget` tokens inside the thinking block, then the closing tag's tokens are forced, one per round
    reasoning_budget: int | None = None
    think_close_ids: tuple = ()
    reasoning_open: bool = False        # the prompt ends inside the thinking block (the template opened it)
    think_open_ids: tuple = ()          # a generated opening tag also starts the block
    media: object = None                # backend.MediaInputs: image rows of the prompt (embeddings, positions, content digests)


@dataclass
class Event:
    kind: str                 # "tokens" | "done" | "error"
    id: str
    tokens: list = field(default_factory=list)
    reason: str = ""          # stop | length | cancelled | error | deadline
    usage: dict = field(default_factory=dict)
    message: str = ""


@dataclass
class _Seq:
    req: Request
    slot: int
    tokens: list
    prompt_len: int
    prefilled: int = 0
    cached: int = 0
    generated: int = 0
    drafter: CopyDrafter = None
    ngram: NgramDrafter = None     # created on first use
    stats: AcceptStats = None
    drafted: int = 0
    accepted: int = 0
    rounds: int = 0
    t_submit: float = 0.0
    t_first: float | None = None
    committed_blocks: int = 0
    hashes: list = None
    reasoning: dict = None     # reasoning-budget state (see Engine._reasoning_budget)
    passed: int = 0            # prefill steps in which shorter prompts were served instead of this one
    curve: object = None       # spec.arbiter.DepthCurve: this stream's conditional acceptance by draft position (budget policies past "legacy")


class StepError(Exception):
    def __init__(self, kind: str, message: str, fatal: bool, group_lost: bool = False):
        super().__init__(f"{kind}: {message}")
        self.kind, self.fatal, self.group_lost = kind, fatal, group_lost


BUDGET_POLICIES = ("legacy", "curve", "plan", "margin", "scored")


@dataclass
class TreeConfig:
    """Draft-tree rounds (reference crates/engine/src/lib.rs:724-832, TreeConfig): at most `max_nodes` draft nodes per stream and round
    (the window holds the anchor as well, and a tree window has at most 64 rows), searched with `policy`."""
    max_nodes: int = 16
    policy: object = None

    def __post_init__(self):
        from ..spec.tree import Policy
        if self.policy is None:
            self.policy = Policy()
        if not 1 <= self.max_nodes <= 63:
            raise ValueError("a tree holds 1..63 draft nodes")


class Engine:
    def __init__(self, backend: Backend, admission: Admission | None = None, *, window_rows: int = 64, prefill_chunk: int = PREFILL_STEP_ROWS,
                 spec: SpecMode | str = "auto", max_drafts: int = 4, cost: CostModel | None = None, prefix: PrefixIndex | None = None,
                 prefill_policy: str = "burst", burst_div: int = 2, burst_cap: int = 16, cache_namespace: bytes = b"", device_sampler: bool = False,
                 spill=None, arbiter=None, trees=None, budget_policy: str = "legacy", round_cost=None):
        self.backend = backend
        self.admission = admission
        self.window_rows = min(window_rows, backend.max_rows)
        self.prefill_chunk = prefill_chunk
        self.spec = spec if isinstance(spec, SpecMode) else SpecMode(spec)
        self.max_drafts = max_drafts
        self.can_rollback = getattr(backend, "supports_rollback", lambda: True)()
        self.cost = cost
        self.prefix = prefix if (prefix is not None and backend.prefix_block_tokens() > 0) else None
        # second tier (sched.spill.SpillStore): blocks leaving the index are exported to it, and a lookup that ends early continues there
        # optional spec.Arbiter: per round and stream it picks how many of the offered drafts to verify (or none) by expected committed tokens
        # per model-millisecond, learns each source's acceptance by depth from the outcomes, and probes idle sources now and then
        self.arbiter = arbiter
        # how many of a stream's drafts ride in the verify window (reference crates/engine/src/lib.rs:724-746, BudgetPolicy); no policy changes a
        # committed token.  legacy: one geometric acceptance rate per stream, trimmed after the draft by the verify step's cost.  curve: the
        # stream's measured conditional acceptance by draft position instead.  plan: curve, decided BEFORE the draft with the draft's cost in
        # the model (`round_cost`: sched.RoundCost), so a stream not worth drafting is not drafted and the drafter is asked only for the
        # positions that will be verified.  margin: plan, then trimmed again after the draft by the drafter's own confidence in each pick.
        # scored: the pre-draft plan only picks WHICH streams draft (they are asked for every pick), the confidences trim afterwards.
        if budget_policy not in BUDGET_POLICIES:
            raise ValueError(f"unknown budget policy {budget_policy!r}; one of {', '.join(BUDGET_POLICIES)}")
        self.budget_policy, self.round_cost = budget_policy, round_cost
        from ..spec.stats import MODES, MarginBins, PositionStats
        self.position_stats = {m: PositionStats() for m in MODES}     # per draft position: offered / verified / reached / accepted
        self.margin_bins = MarginBins()                               # acceptance by the drafter's margin (the confidence of margin / scored)
        # TreeConfig: verify windows are draft trees when the backend supports them (chain windows otherwise)
        self.trees = trees
        self.prefix_cuts = bool(self.prefix is not None and getattr(backend, "prefix_needs_cuts", lambda: False)())
        self.spill = spill if self.prefix is not None else None
        if self.spill is not None:
            self.prefix.on_evict = self._spill_out
        self.prefill_policy = prefill_policy
        # sample and accept on the device (the keyed sampler's device twin) when the backend offers it: only token ids come back
        self.device_sampler = bool(device_sampler and getattr(backend, "supports_device_sampler", lambda: False)())
        self.burst_div, self.burst_cap = max(1, burst_div), max(1, burst_cap)
        self.cache_namespace = cache_namespace
        self.waiting: deque = deque()
        self.seqs: dict = {}           # id -> _Seq (admitted)
        self.order: list = []          # admitted ids in arrival order
        self.free_slots = list(range(backend.max_slots - 1, -1, -1)) if admission is None else None
        self.events: list = []
        self.counters = dict(rounds=0, rows=0, prefill_tokens=0, decode_tokens=0, drafted=0, accepted=0, cached_tokens=0, requests=0,
                             finished=0, errors=0, spilled_blocks=0, unspilled_blocks=0)
        self.phase_ns = dict(draft=0, verify=0, commit=0, prefill=0)
        # speculation by draft position (0 = the first draft after the anchor): drafts offered to a window, drafts whose row was reached
        # (every earlier draft accepted), drafts accepted; the per-position acceptance curve is accepted / reached
        self.spec_pos = dict(offered=[0] * max(1, max_drafts), reached=[0] * max(1, max_drafts), accepted=[0] * max(1, max_drafts))
        self._window_start = 0         # rotation of the decode window over the active streams when they outnumber its rows
        self.pause_decode = False      # hold decode rounds (used while a benchmark fills the batch with prompts)

    # ------------------------------------------------------------------ submit / cancel
    def check(self, req: Request) -> None:
        """Refuse what can never run (fail closed), before queueing."""
        if not req.prompt:
            raise ValueError("empty prompt")
        if any((not isinstance(t, int)) or t < 0 or t >= self.backend.vocab_size for t in req.prompt):
            raise ValueError("prompt token outside the vocabulary")
        if req.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if req.media is not None:
            if not getattr(self.backend, "supports_media", lambda: False)():
                raise ValueError("this backend takes no image inputs")
            m = req.media
            if len(m.rows) != len(m.embeds) or (len(m.rows) and (int(m.rows[0]) < 0 or int(m.rows[-1]) >= len(req.prompt))) or \
                    (m.pos3 is not None and len(m.pos3) != len(req.prompt)):
                raise ValueError("image rows do not match the prompt")
        (req.sampling or Sampling()).validate()
        if self.admission is not None:
            self.admission.check(len(req.prompt) + req.max_new_tokens)

    def submit(self, req: Request) -> None:
        """Deferred submit: validated now, admitted in arrival order when memory and a slot allow."""
        self.check(req)
        if req.sampling is None:
            req.sampling = Sampling()
        if req.sampling.seed == 0 and req.sampling.temperature > 0:
            req.sampling = req.sampling.with_seed(seed_for(req.prompt, 0))
        self.waiting.append((req, time.monotonic()))
        self.counters["requests"] += 1

    def cancel(self, rid: str, reason: str = "cancelled") -> bool:
        for i, (r, _) in enumerate(self.waiting):
            if r.id == rid:
                del self.waiting[i]
                self.events.append(Event("done", rid, reason=reason, usage=self._usage(None, r)))
                return True
        s = self.seqs.get(rid)
        if s is None:
            return False
        self._finish(s, reason)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.seqs)

    def active_count(self) -> int:
        return len(self.seqs)

    def take_events(self) -> list:
        ev, self.events = self.events, []
        return ev

    # ------------------------------------------------------------------ prompt scoring (decisions, prompt log-probabilities)
    def score_prompt(self, tokens) -> "np.ndarray":
        """Full-vocabulary logits (float32) of the position after `tokens`, computed on a free slot between steps.  Nothing is
        generated and nothing stays in the KV cache.  Raises AdmitError("NoSlot") when every slot is busy."""
        tokens = [int(t) for t in tokens]
        if not tokens:
            raise ValueError("empty prompt")
        if self.admission is not None:
            slot = self.admission.admit(len(tokens) + 1)
        else:
            if not self.free_slots:
                raise AdmitError("NoSlot", reason="every slot is busy")
            slot = self.free_slots.pop()
        try:
            return self.backend.score_last(slot, tokens, self.prefill_chunk)
        finally:
            self.backend.release(slot)
            if self.admission is not None:
                self.admission.release(slot)
            else:
                self.free_slots.append(slot)

    # ------------------------------------------------------------------ admission
    def _admit(self) -> None:
        while self.waiting:
            req, t0 = self.waiting[0]
            need = len(req.prompt) + req.max_new_tokens
            try:
                if self.admission is not None:
                    slot = self.admission.admit(need)
                else:
                    if not self.free_slots:
                        return
                    slot = self.free_slots.pop()
            except AdmitError as e:
                if e.kind in ("NoMemory", "NoSlot"):
                    if self.prefix is not None and e.kind == "NoMemory" and len(self.prefix):
                        freed = self.prefix.evict_bytes(e.info.get("needed", 0) - e.info.get("available", 0))
                        if freed:
                            self.backend.prefix_release(freed)
                            continue
                    return  # strictly in arrival order: the head waits, nobody overtakes
                self.waiting.popleft()
                self.events.append(Event("error", req.id, reason="error", message=str(e)))
                continue
            self.waiting.popleft()
            s = _Seq(req, slot, list(req.prompt), len(req.prompt), drafter=CopyDrafter(), stats=AcceptStats(), t_submit=t0)
            self.seqs[req.id] = s
            self.order.append(req.id)
            if req.media is not None:
                self.backend.set_media(slot, req.media)
            self._plan_prefix(s)

    def _plan_prefix(self, s: _Seq) -> None:
        if self.prefix is None or not s.req.prefix_cache:
            return
        bt = self.backend.prefix_block_tokens()
        # image placeholders hash by their image's content, not by the placeholder id
        s.hashes = chain_hashes(s.tokens[:s.prompt_len] if s.req.media is None else s.req.media.hash_tokens(s.tokens[:s.prompt_len]), bt, self.cache_namespace)
        chain = self.prefix.lookup(s.hashes, s.prompt_len)
        if self.spill is not None:
            chain = self._spill_in(s, chain)
        if chain:
            n = self.backend.prefix_restore(s.slot, [e.handle for e in chain])
            s.prefilled = s.cached = n
            s.committed_blocks = n // bt
            self.counters["cached_tokens"] += n

    def _spill_out(self, entry) -> None:
        if entry.key in self.spill:
            return
        payload = self.backend.prefix_export(entry.handle)
        if payload is not None and self.spill.put(entry.key, payload):
            self.counters["spilled_blocks"] += 1

    def _spill_in(self, s: _Seq, chain: list) -> list:
        """Continue a device-cache chain with blocks held by the spill tier: import each into the backend and the index, in order."""
        max_blocks = (s.prompt_len - 1) // self.backend.prefix_block_tokens()
        k = len(chain)
        while k < max_blocks and s.hashes[k] in self.spill:
            payload = self.spill.get(s.hashes[k])
            handle = self.backend.prefix_import(payload) if payload is not None else None
            if handle is None:
                break
            dup, evicted = self.prefix.insert(s.hashes[:k + 1], [None] * k + [handle], self.backend.prefix_bytes_per_block())
            gone = [h for h in list(dup) + list(evicted) if h is not None]
            if gone:
                self.backend.prefix_release(gone)
            e = self.prefix.entries.get(s.hashes[k])
            if e is None or e.handle is not handle:       # the budget could not keep it: stop here
                break
            chain = chain + [e]
            k += 1
            self.counters["unspilled_blocks"] += 1
        return chain

    # ------------------------------------------------------------------ the step
    def step(self) -> list:
        """One scheduling iteration; returns the events it produced."""
        self._expire()
        self._admit()
        try:
            with trace.nvtx_range("decode_round"):
                self._decode_round()
            with trace.nvtx_range("prefill"):
                self._prefill()
        except BackendError as e:
            self.counters["errors"] += 1
            if e.fatal:
                raise StepError("Fatal", str(e), True, getattr(e, "group_lost", False))
            for rid in list(self.seqs):
                self._finish(self.seqs[rid], "error", message=str(e))
            raise StepError("Backend", str(e), False)
        return self.take_events()

    def run_until_idle(self, max_steps: int = 1 << 30) -> list:
        out = []
        for _ in range(max_steps):
            if not self.has_work():
                break
            out.extend(self.step())
        return out

    def _expire(self) -> None:
        now = time.monotonic()
        for req, _ in list(self.waiting):
            if req.deadline is not None and now > req.deadline:
                self.cancel(req.id, "deadline")
        for s in list(self.seqs.values()):
            if s.req.deadline is not None and now > s.req.deadline:
                self._finish(s, "deadline")

    def _check_backend(self) -> None:
        err = self.backend.take_error()
        if err is not None:
            raise err

    # ------------------------------------------------------------------ decode round
    def _decode_round(self) -> None:
        if self.pause_decode:
            return
        active = [self.seqs[i] for i in self.order if self.seqs[i].prefilled >= self.seqs[i].prompt_len and self.seqs[i].generated > 0]
        if not active:
            return
        if len(active) > self.window_rows:
            # more decodable streams than window rows: the window's start rotates, so every stream gets its turn (first come is not
            # first served forever) and none waits for an earlier one to finish
            start = self._window_start % len(active)
            active = (active[start:] + active[:start])[:self.window_rows]
            self._window_start = start + self.window_rows
        if self.trees is not None and self.can_rollback and getattr(self.backend, "supports_trees", lambda: False)():
            return self._decode_round_trees(active)
        t0 = time.perf_counter_ns()
        # 1. how many drafts each stream may use
        maxes = []
        for s in active:
            room = s.req.max_new_tokens - s.generated
            m = min(self.max_drafts, max(0, room - 1)) if (self.spec.enabled and s.req.draft and self.can_rollback) else 0
            maxes.append(m)
        pol = self.budget_policy
        if pol in ("plan", "margin", "scored") and any(maxes):
            # decided before the draft, with the draft's own cost: who drafts, and (plan, margin) how deep
            pre = [Demand.from_conditional(self._curve(s).conditional(m), m).with_kv_tokens(len(s.tokens)) for s, m in zip(active, maxes)]
            ahead = self._share(pre, self.window_rows, draft_sunk=False)
            maxes = [(m if a > 0 else 0) if pol == "scored" else min(m, a) for m, a in zip(maxes, ahead)]
            self.counters["planned_out"] = self.counters.get("planned_out", 0) + sum(1 for m in maxes if m == 0)
        # 2. proposals: native drafter first, copy drafter otherwise
        proposals = [[] for _ in active]
        confs = [None] * len(active)
        margins = [None] * len(active)
        offered = [0] * len(active)
        sources = ["none"] * len(active)        # which drafter each proposal came from: "native" (backend drafter) or "copy" (host drafters)
        if any(maxes):
            if self.spec.native and self.backend.supports_native_draft():
                asks = [DraftAsk(s.slot, s.tokens, m, s.req.sampling) for s, m in zip(active, maxes) if m > 0]
                offers = self.backend.propose_batch(asks)
                for i, s in enumerate(active):
                    off = offers.get(s.slot)
                    if off is not None and maxes[i] > 0:
                        proposals[i] = list(off.tokens[:maxes[i]])
                        confs[i] = list(off.conf[:len(proposals[i])]) if off.conf else None
                        margins[i] = list(off.margin[:len(proposals[i])]) if off.margin else None
                        if confs[i] is None and margins[i] and len(margins[i]) >= len(proposals[i]):
                            # conditional confidences from the margins: what picks with such a lead have done so far
                            confs[i] = self.margin_bins.confidences(margins[i])
                        sources[i] = "native" if proposals[i] else "none"
            if self.spec.copy:
                for i, s in enumerate(active):
                    if not proposals[i] and maxes[i] > 0:
                        proposals[i] = s.drafter.propose(s.tokens, maxes[i])
                        sources[i] = "copy" if proposals[i] else "none"
            if self.spec.ngram:
                for i, s in enumerate(active):
                    if not proposals[i] and maxes[i] > 0:
                        if s.ngram is None:
                            s.ngram = NgramDrafter()
                        proposals[i] = s.ngram.propose(s.tokens, maxes[i])
                        sources[i] = "copy" if proposals[i] else "none"
        choices = None
        if self.arbiter is not None:
            offers = {s.req.id: ({sources[i]: len(proposals[i])} if proposals[i] else {}) for i, s in enumerate(active)}
            picks = self.arbiter.choose(offers, self.window_rows)
            choices = []
            for i, s in enumerate(active):
                c = picks[s.req.id]
                proposals[i] = proposals[i][:c.drafts()] if c.kind == sources[i] else []
                choices.append(c if proposals[i] else None)
        offered = [len(p) for p in proposals]
        # 3. budget: share the window's rows by expected value
        budget = self.window_rows
        if pol == "legacy":
            demands = [Demand.geometric(s.stats.accept_rate(), len(p)) for s, p in zip(active, proposals)]
        elif pol in ("curve", "plan"):
            demands = [Demand.from_conditional(self._curve(s).conditional(len(p)), len(p)).with_kv_tokens(len(s.tokens)) for s, p in zip(active, proposals)]
        else:       # margin, scored: the drafter's own confidence in each pick where it gave one
            demands = [Demand.from_conditional(c if (c and len(c) >= len(p)) else self._curve(s).conditional(len(p)), len(p)).with_kv_tokens(len(s.tokens))
                       for s, p, c in zip(active, proposals, confs)]
        alloc = self._share(demands, budget, draft_sunk=True)
        for i in range(len(active)):
            proposals[i] = proposals[i][:alloc[i]]
        t1 = time.perf_counter_ns()
        # 4. the window
        reqs = [RowRequest(s.slot, [s.tokens[-1]] + p, len(s.tokens) - 1) for s, p in zip(active, proposals)]
        cand = max(s.req.sampling.candidate_count(self.backend.vocab_size) for s in active)
        cand = min(cand, 64)
        greedy = [s.req.sampling.temperature == 0.0 for s in active]
        sampled = None
        if self.device_sampler:
            sampled = self.backend.step_sampled(reqs, cand, [(s.req.sampling, len(s.tokens)) for s in active])
            rows = [[None] * len(q.tokens) for q in reqs]
        else:
            rows = self.backend.step_verified(reqs, cand, greedy)
        self._check_backend()
        t2 = time.perf_counter_ns()
        if len(rows) != len(reqs) or any(len(r) != len(q.tokens) for r, q in zip(rows, reqs)):
            raise BackendError("backend returned a window of the wrong shape", fatal=False)
        self.counters["rounds"] += 1
        self.counters["rows"] += sum(len(q.tokens) for q in reqs)
        self.counters["round_streams"] = self.counters.get("round_streams", 0) + len(reqs)
        self.counters["round_draft_streams"] = self.counters.get("round_draft_streams", 0) + sum(1 for p in proposals if p)
        # 5. sample every row at its own position, accept the matching prefix, commit or finish
        for si, (s, p, out) in enumerate(zip(active, proposals, rows)):
            base = len(s.tokens)
            try:
                if sampled is not None:
                    samples = sampled[si][0]
                    if samples is None:
                        raise SamplingError("NaN logit")
                elif s.req.sampling.temperature == 0.0 and all(len(o.ids) and o.values[0] == o.values[0] and
                                                              (len(o.ids) == 1 or o.values[0] > o.values[1] or
                                                               (o.values[0] == o.values[1] and o.ids[0] < o.ids[1])) for o in out):
                    # greedy over candidates that arrive ordered (value desc, id asc): the first one is the keyed sampler's choice
                    samples = [int(o.ids[0]) for o in out]
                else:
                    samples = [choose(o.values, o.ids, base + j, s.req.sampling) for j, o in enumerate(out)]
            except SamplingError as e:
                self._finish(s, "error", message=f"sampling failed: {e}")  # a NaN row fails only its sequence
                continue
            a = accept(p, samples)
            s.rounds += 1
            if choices is not None:
                from ..spec.arbiter import NONE, Choice
                self.arbiter.observe(s.req.id, Choice(choices[si].kind, len(p)) if (choices[si] is not None and p) else NONE, a)
            if p:
                sp = self.spec_pos
                for j in range(min(len(p), len(sp["offered"]))):
                    sp["offered"][j] += 1
                    sp["reached"][j] += 1 if j <= a else 0
                    sp["accepted"][j] += 1 if j < a else 0
                s.stats.update(len(p), a)
                self._curve(s).observe(len(p), a)
                from ..spec.stats import mode_of
                self.position_stats[mode_of(s.req.sampling)].record(max(offered[si], len(p)), len(p), a)
                if margins[si]:
                    self.margin_bins.record(margins[si], len(p), a)
                s.drafted += len(p)
                s.accepted += a
                self.counters["drafted"] += len(p)
                self.counters["accepted"] += a
            else:
                s.stats.relax()
            emitted, reason = self._emit(s, samples[:a + 1])
            if reason is not None:
                self._finish(s, reason)
            else:
                self.backend.commit(s.slot, len(emitted))
        self.phase_ns["draft"] += t1 - t0
        self.phase_ns["verify"] += t2 - t1
        self.phase_ns["commit"] += time.perf_counter_ns() - t2

    def _curve(self, s):
        if s.curve is None:
            from ..spec.arbiter import DepthCurve
            s.curve = DepthCurve([0.7])
        return s.curve

    def _share(self, demands, budget: int, draft_sunk: bool) -> list:
        """Drafts per stream for a window of `budget` rows: by the round cost model where there is one (with the draft's own cost when the
        draft has not run yet), else by the verify step's cost table, else by marginal value alone."""
        if self.round_cost is not None:
            from ..sched import plan_round
            return plan_round(self.round_cost, demands, budget, draft_sunk).drafts
        if self.cost is not None:
            return choose_budget(self.cost, demands, budget)[1]
        from ..sched import allocate
        return allocate(demands, budget)

    def _emit(self, s, new) -> tuple:
        """Commits the round's tokens `new` to the sequence one by one (reasoning budget, stop ids, length) and queues the event.
        -> (tokens emitted, finish reason or None)."""
        emitted, reason = [], None
        for t in new:
            forced = False
            if s.req.reasoning_budget is not None and s.req.think_close_ids:
                t, forced = self._reasoning_budget(s, t)
            emitted.append(t)
            s.tokens.append(t)
            s.generated += 1
            if t in s.req.stop_ids:
                reason = "stop"
                break
            if s.generated >= s.req.max_new_tokens:
                reason = "length"
                break
            if forced:
                break      # the samples after a forced token were made for another continuation: their rows are not kept
        self.counters["decode_tokens"] += len(emitted)
        self.events.append(Event("tokens", s.req.id, tokens=emitted))
        return emitted, reason

    def _decode_round_trees(self, active) -> None:
        """A decode round whose windows are draft trees (reference crates/engine/src/lib.rs:2215, decode_round_trees): every stream's native
        offer becomes a best-first tree over its candidate lattice (a chain when the drafter gave no lattice), the copy drafter's chain is
        grafted below the anchor, the window's rows are shared among the streams by the nodes' probabilities of lying on the accepted path,
        one forward verifies every node, the target's own samples walk down each tree, and the accepted path is committed.  The committed
        tokens are the target's samples at their positions, so the output equals the serial run's whatever the trees held."""
        from ..sched import allocate
        from ..spec.tree import DraftTree, best_first, with_copy, accept_tree
        from .backend import TreeRequest
        cfg = self.trees
        t0 = time.perf_counter_ns()
        maxes = []
        for s in active:
            room = s.req.max_new_tokens - s.generated
            maxes.append(min(self.max_drafts, max(0, room - 1)) if (self.spec.enabled and s.req.draft) else 0)
        trees = [DraftTree() for _ in active]
        if any(maxes) and self.spec.native and self.backend.supports_native_draft():
            asks = [DraftAsk(s.slot, s.tokens, m, s.req.sampling) for s, m in zip(active, maxes) if m > 0]
            offers = self.backend.propose_batch(asks)
            for i, s in enumerate(active):
                off = offers.get(s.slot)
                if off is None or maxes[i] <= 0:
                    continue
                if off.lattice is not None and len(off.lattice.ids) > 0:
                    lat = off.lattice
                    lat = type(lat)(lat.ids[:maxes[i]], lat.unary[:maxes[i]], None if lat.edge is None else lat.edge[:maxes[i]])
                    trees[i] = best_first(lat, cfg.max_nodes, cfg.policy)
                else:
                    toks = list(off.tokens[:maxes[i]])
                    conf = list(off.conf[:len(toks)]) + [0.7] * (len(toks) - len(off.conf))
                    lp, logp = 0.0, []
                    for c in conf:
                        lp += math.log(min(1.0, max(1e-6, c)))
                        logp.append(lp)
                    trees[i] = DraftTree(toks, list(range(-1, len(toks) - 1)), list(range(1, len(toks) + 1)), logp)
        if self.spec.copy:
            for i, s in enumerate(active):
                if maxes[i] > 0:
                    chain = s.drafter.propose(s.tokens, maxes[i])
                    if chain:
                        trees[i] = with_copy(trees[i], chain, cfg.max_nodes)
        # nodes are in pop order with non-increasing probabilities: a stream's share of the window is a prefix of its tree
        demands = [Demand(t.probabilities()) for t in trees]
        alloc = allocate(demands, self.window_rows)
        trees = [t.prefix(min(n, cfg.max_nodes, 63)) for t, n in zip(trees, alloc)]
        t1 = time.perf_counter_ns()
        reqs = [TreeRequest(s.slot, [s.tokens[-1]] + t.tokens, [-1] + [p + 1 for p in t.parents], len(s.tokens) - 1) for s, t in zip(active, trees)]
        cand = min(64, max(s.req.sampling.candidate_count(self.backend.vocab_size) for s in active))
        rows = self.backend.step_tree(reqs, cand)
        self._check_backend()
        t2 = time.perf_counter_ns()
        if len(rows) != len(reqs) or any(len(r) != len(q.tokens) for r, q in zip(rows, reqs)):
            raise BackendError("backend returned a tree window of the wrong shape", fatal=False)
        self.counters["rounds"] += 1
        self.counters["tree_rounds"] = self.counters.get("tree_rounds", 0) + 1
        self.counters["rows"] += sum(len(q.tokens) for q in reqs)
        self.counters["round_streams"] = self.counters.get("round_streams", 0) + len(reqs)
        self.counters["round_draft_streams"] = self.counters.get("round_draft_streams", 0) + sum(1 for t in trees if len(t))
        for s, t, q, out in zip(active, trees, reqs, rows):
            base = len(s.tokens)
            depth = q.depths()
            try:
                # row r's sample is the token at index base + depth(r): the keyed sampler draws it for that position
                samples = [choose(o.values, o.ids, base + depth[r], s.req.sampling) for r, o in enumerate(out)]
            except SamplingError as e:
                self._finish(s, "error", message=f"sampling failed: {e}")
                continue
            path, committed = accept_tree(t, samples)
            s.rounds += 1
            a = len(path)
            if len(t):
                deepest = max(t.depth)
                sp = self.spec_pos
                for j in range(min(deepest, len(sp["offered"]))):
                    sp["offered"][j] += 1
                    sp["reached"][j] += 1 if j <= a else 0
                    sp["accepted"][j] += 1 if j < a else 0
                s.stats.update(deepest, a)
                s.drafted += len(t)
                s.accepted += a
                self.counters["drafted"] += len(t)
                self.counters["accepted"] += a
                self.counters["tree_nodes"] = self.counters.get("tree_nodes", 0) + len(t)
                self.counters["tree_depth_kept"] = self.counters.get("tree_depth_kept", 0) + a
            else:
                s.stats.relax()
            emitted, reason = self._emit(s, committed)
            if reason is not None:
                self._finish(s, reason)
            else:
                # the rows kept are the anchor and the accepted nodes whose tokens were emitted (a forced token ends the list early)
                self.backend.commit_path(s.slot, [n + 1 for n in path[:len(emitted) - 1]])
        self.phase_ns["draft"] += t1 - t0
        self.phase_ns["verify"] += t2 - t1
        self.phase_ns["commit"] += time.perf_counter_ns() - t2

    def _reasoning_budget(self, s, t: int):
        """Reasoning budget (reference crates/engine/src/lib.rs:560-603): every generated token, the one sampled at the end of prefill
        included, passes through here before it is committed.  `used` counts the tokens committed inside the thinking block; the token
        that would be committed when `used == reasoning_budget` while the block is still open is replaced by the closing tag (index 0 for
        a budget of 0), whose remaining tokens follow one per call.  A closing tag the model commits itself ends the block and spends the
        budget.  The rule reads committed tokens only, so the serial and every drafted path commit the same token at every index.
        -> (token to commit, whether it replaced the sample)."""
        st = s.reasoning
        if st is None:
            st = s.reasoning = dict(open=s.req.reasoning_open, used=0, force=None, close_match=0, open_match=0)
        close, opn = s.req.think_close_ids, s.req.think_open_ids
        if not st["open"]:
            if opn:
                st["open_match"] = st["open_match"] + 1 if t == opn[st["open_match"]] else (1 if t == opn[0] else 0)
                if st["open_match"] == len(opn):
                    st.update(open=True, open_match=0, used=0, close_match=0)
            return t, False
        if st["force"] is None and st["used"] >= s.req.reasoning_budget and not (st["close_match"] > 0 and t == close[st["close_match"]]):
            st.update(force=0, close_match=0)     # out of budget and the model is not in the middle of closing the block itself
        if st["force"] is not None:
            forced = close[st["force"]]
            st["force"] += 1
            if st["force"] == len(close):
                st.update(open=False, force=None)
            return forced, forced != t
        st["close_match"] = st["close_match"] + 1 if t == close[st["close_match"]] else (1 if t == close[0] else 0)
        if st["close_match"] == len(close):
            st.update(open=False, close_match=0)
            return t, False
        st["used"] += 1
        return t, False

    # ------------------------------------------------------------------ prefill
    def _prefill(self) -> None:
        """The prompt rows of one step.  Policy "serial": one slice, the waiting prompts in arrival order.  Policy "burst" (the default):
        while prompts queue up, up to ceil(waiting / burst_div) slices (at most burst_cap; one while one prompt waits) share ONE backend call
        of at most `prefill_chunk` rows; each slice goes to the prompt with the fewest rows left, oldest among equals, and a prompt that was
        passed over PREFILL_PASS_GUARD steps goes first, so a long prompt among short ones is slowed, never starved (the reference's
        `PrefillPolicy::Burst`, crates/engine/src/lib.rs:766-803).  Every prefill kernel is row-invariant, so the policy moves first tokens in
        time and changes no bit of any reply."""
        pending = [self.seqs[i] for i in self.order if i in self.seqs and (self.seqs[i].prefilled < self.seqs[i].prompt_len or self.seqs[i].generated == 0)]
        if not pending:
            return
        t0 = time.perf_counter_ns()
        if self.prefill_policy == "burst" and not self.prefix_cuts and len(pending) > 1:
            guarded = [s for s in pending if s.passed >= PREFILL_PASS_GUARD]
            rest = [s for s in pending if s.passed < PREFILL_PASS_GUARD]
            rest.sort(key=lambda s: s.prompt_len - s.prefilled)        # stable: oldest among equals
            max_slices = min(self.burst_cap, -(-len(pending) // self.burst_div))
            chosen, rows_left = [], self.prefill_chunk
            for s in guarded + rest:
                if len(chosen) >= max_slices or rows_left <= 0:
                    break
                n = min(rows_left, s.prompt_len - s.prefilled)
                chosen.append((s, n))
                rows_left -= n
            took = {id(s) for s, _ in chosen}
            for s in pending:
                s.passed = 0 if id(s) in took else s.passed + 1
            items = [(s.slot, s.prefilled, s.tokens[s.prefilled:s.prefilled + n], s.prefilled + n >= s.prompt_len) for s, n in chosen]
            cand = min(64, max(s.req.sampling.candidate_count(self.backend.vocab_size) for s, _ in chosen))
            outs = self.backend.prefill_slices(items, cand)
            self._check_backend()
            for (s, n), o in zip(chosen, outs):
                s.prefilled += n
                self.counters["prefill_tokens"] += n
                if s.prefilled >= s.prompt_len:
                    self._complete_prefill(s, o)
                else:
                    self._commit_prefix(s)
            self.phase_ns["prefill"] += time.perf_counter_ns() - t0
            return
        s = pending[0]
        n = min(self.prefill_chunk, s.prompt_len - s.prefilled)
        if self.prefix_cuts and s.req.prefix_cache:
            # a recurrent backend snapshots its state where a slice ends: end one at the last block boundary a later prompt could reuse
            bt = self.backend.prefix_block_tokens()
            cut = (s.prompt_len - 1) // bt * bt
            if s.prefilled < cut < s.prefilled + n:
                n = cut - s.prefilled
        last = s.prefilled + n >= s.prompt_len
        cand = min(64, s.req.sampling.candidate_count(self.backend.vocab_size))
        out = self.backend.prefill_slice(s.slot, s.prefilled, s.tokens[s.prefilled:s.prefilled + n], cand, last)
        self._check_backend()
        s.prefilled += n
        self.counters["prefill_tokens"] += n
        self._commit_prefix(s)   # progressive checkpoints: a cancelled long prompt resumes from its last full block
        if last:
            self._complete_prefill(s, out)
        self.phase_ns["prefill"] += time.perf_counter_ns() - t0

    def _commit_prefix(self, s: _Seq) -> None:
        if self.prefix is None or not s.req.prefix_cache or s.hashes is None:
            return
        bt = self.backend.prefix_block_tokens()
        full = min(s.prefilled, s.prompt_len) // bt
        if full <= s.committed_blocks:
            return
        handles = self.backend.prefix_commit(s.slot, full)
        if not handles:
            return
        dup, evicted = self.prefix.insert(s.hashes[:full], handles, self.backend.prefix_bytes_per_block())
        drop = list(dup) + list(evicted)
        if drop:
            self.backend.prefix_release(drop)
        s.committed_blocks = full

    def _complete_prefill(self, s: _Seq, out) -> None:
        self._commit_prefix(s)
        if out is None:
            raise BackendError("backend returned no candidates for the last prompt row", fatal=False)
        try:
            t = choose(out.values, out.ids, s.prompt_len, s.req.sampling)
        except SamplingError as e:
            self._finish(s, "error", message=f"sampling failed: {e}")
            return
        if s.req.reasoning_budget is not None and s.req.think_close_ids:
            t, _ = self._reasoning_budget(s, t)     # index 0 of the reply obeys the budget like every later token
        s.tokens.append(t)
        s.generated = 1
        s.t_first = time.monotonic()
        self.counters["decode_tokens"] += 1
        self.events.append(Event("tokens", s.req.id, tokens=[t]))
        if t in s.req.stop_ids:
            self._finish(s, "stop")
        elif s.generated >= s.req.max_new_tokens:
            self._finish(s, "length")

    # ------------------------------------------------------------------ finish
    def _usage(self, s, req=None) -> dict:
        if s is None:
            return dict(prompt_tokens=len(req.prompt), completion_tokens=0, total_tokens=len(req.prompt), cached_tokens=0,
                        spec=dict(drafted=0, accepted=0, rounds=0))
        u = dict(prompt_tokens=s.prompt_len, completion_tokens=s.generated, total_tokens=s.prompt_len + s.generated, cached_tokens=s.cached,
                 spec=dict(drafted=s.drafted, accepted=s.accepted, rounds=s.rounds))
        if s.t_first is not None:
            u["ttft_s"] = s.t_first - s.t_submit
        return u

    def _finish(self, s: _Seq, reason: str, message: str = "") -> None:
        self.backend.release(s.slot)
        if self.arbiter is not None:
            self.arbiter.forget(s.req.id)
        if self.admission is not None:
            self.admission.release(s.slot)
        else:
            self.free_slots.append(s.slot)
        del self.seqs[s.req.id]
        self.order.remove(s.req.id)
        self.counters["finished"] += 1
        kind = "error" if reason == "error" else "done"
        self.events.append(Event(kind, s.req.id, reason=reason, usage=self._usage(s), message=message))


def generate(engine: Engine, prompts: list, max_new_tokens: int = 32, sampling: Sampling | None = None, stop_ids=()) -> list:
    """Offline generation: run `prompts` (token-id lists) to completion and return the generated ids of each."""
    out = {}
    for i, p in enumerate(prompts):
        engine.submit(Request(str(i), list(p), max_new_tokens, sampling, tuple(stop_ids)))
        out[str(i)] = []
    while engine.has_work():
        for ev in engine.step():
            if ev.kind == "tokens":
                out[ev.id].extend(ev.tokens)
            elif ev.kind == "error":
                raise RuntimeError(f"request {ev.id}: {ev.message}")
    return [out[str(i)] for i in range(len(prompts))]
