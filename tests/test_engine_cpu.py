"""Engine step loop on the CPU mock: exactness harness (and that it catches each injected fault), admission, errors,
deadlines, stop tokens, prefix cache."""
import time

import numpy as np
import pytest

from rexl3_b200 import sched
from rexl3_b200.engine import BackendError, Engine, MockBackend, MockOptions, Request, StepError, TreeConfig, TreeRequest, generate, harness
from rexl3_b200.sampling import GREEDY, Sampling


def mk(**kw):
    return lambda: MockBackend(MockOptions(**kw))


@pytest.mark.parametrize("check", [f.__name__ for f in harness.ALL])
def test_exactness_checks_pass_on_the_honest_mock(check):
    assert getattr(harness, check)(mk(), 512) is None


@pytest.mark.parametrize("fault,caught_by", [("window_dependent", "row_invariance"), ("chunk_dependent", "chunked_prefill_equals_whole"),
                                             ("rollback_leak", "rollback_equals_replay"), ("prefix_stale", "cached_equals_cold")])
def test_each_fault_is_caught_by_its_check(fault, caught_by):
    assert getattr(harness, caught_by)(mk(fault=fault), 512) is not None


def test_native_draft_speeds_up_without_changing_output():
    p = harness.default_prompts(512)
    base = Engine(MockBackend(MockOptions()), spec="none")
    a = generate(base, p, 64, harness.SAMPLING)
    fast = Engine(MockBackend(MockOptions(native_draft=True)), spec="auto", max_drafts=4)
    b = generate(fast, p, 64, harness.SAMPLING)
    assert a == b and fast.counters["rounds"] < base.counters["rounds"] and fast.counters["accepted"] > 0


def test_admission_queues_in_arrival_order_and_refuses_what_never_fits():
    model = sched.ModelMemory(0, 10)
    adm = sched.Admission(10 * 300, 0, model, 2)
    eng = Engine(MockBackend(MockOptions(slots=2)), adm, spec="none")
    with pytest.raises(sched.AdmitError):
        eng.submit(Request("big", [1] * 400, 10, GREEDY))
    for i in range(3):
        eng.submit(Request(f"r{i}", [1 + i] * 100, 20, GREEDY))
    eng.step()
    assert eng.active_count() == 2 and len(eng.waiting) == 1
    done = [e.id for e in eng.run_until_idle() if e.kind == "done"]
    assert done.index("r0") < done.index("r2") and set(done) == {"r0", "r1", "r2"}
    assert adm.available() == adm.capacity


def test_stop_token_length_and_usage():
    be = MockBackend(MockOptions(eos=7, eos_after=5))
    eng = Engine(be, spec="none")
    eng.submit(Request("a", [1, 2, 3], 50, GREEDY, stop_ids=(7,)))
    eng.submit(Request("b", [4, 5], 4, GREEDY))
    ev = eng.run_until_idle()
    fin = {e.id: e for e in ev if e.kind == "done"}
    assert fin["a"].reason == "stop" and fin["b"].reason == "length"
    assert fin["b"].usage["completion_tokens"] == 4 and fin["b"].usage["prompt_tokens"] == 2 and "ttft_s" in fin["b"].usage
    toks = [t for e in ev if e.kind == "tokens" and e.id == "a" for t in e.tokens]
    assert toks[-1] == 7 and len(toks) == fin["a"].usage["completion_tokens"]


def test_validation_cancel_and_deadline():
    eng = Engine(MockBackend(MockOptions()), spec="none")
    with pytest.raises(ValueError):
        eng.submit(Request("x", [], 5, GREEDY))
    with pytest.raises(ValueError):
        eng.submit(Request("x", [99999], 5, GREEDY))
    with pytest.raises(ValueError):
        eng.submit(Request("x", [1], 5, Sampling(top_p=2.0)))
    eng.submit(Request("c", [1, 2], 100, GREEDY))
    eng.step()
    assert eng.cancel("c") and not eng.has_work()
    assert [e.reason for e in eng.take_events() if e.kind == "done"] == ["cancelled"]
    eng.submit(Request("d", [1, 2], 10 ** 6, GREEDY, deadline=time.monotonic() + 0.05))
    t0 = time.monotonic()
    reasons = []
    while eng.has_work() and time.monotonic() - t0 < 5:
        reasons += [e.reason for e in eng.step() if e.kind == "done"]
    assert reasons == ["deadline"]


def test_backend_errors_retryable_fail_the_batch_fatal_raise():
    eng = Engine(MockBackend(MockOptions(retryable_from_step=3)), spec="none")
    eng.submit(Request("a", [1, 2, 3], 50, GREEDY))
    with pytest.raises(StepError) as e:
        eng.run_until_idle()
    assert not e.value.fatal and not eng.has_work()
    assert any(ev.kind == "error" for ev in eng.take_events())
    eng = Engine(MockBackend(MockOptions(fatal_at_step=2)), spec="none")
    eng.submit(Request("a", [1, 2, 3], 50, GREEDY))
    with pytest.raises(StepError) as e:
        eng.run_until_idle()
    assert e.value.fatal


def test_nan_row_fails_only_its_sequence():
    be = MockBackend(MockOptions(nan_at_step=3))
    eng = Engine(be, spec="none", prefill_policy="serial")
    eng.submit(Request("a", [1, 2, 3], 6, Sampling(temperature=0.7)))
    ev = eng.run_until_idle()
    assert any(e.kind == "error" and "NaN" in e.message for e in ev)
    eng.submit(Request("b", [1, 2, 3], 3, GREEDY))
    assert any(e.kind == "done" and e.reason == "length" for e in eng.run_until_idle())


def test_prefix_cache_hits_share_blocks_and_evict():
    be = MockBackend(MockOptions(blocks=64))
    idx = sched.PrefixIndex(sched.CacheBudget(max_bytes=3 * be.prefix_bytes_per_block()), block_tokens=64)
    eng = Engine(be, spec="none", prefix=idx)
    shared = np.random.default_rng(0).integers(0, 512, size=200).tolist()
    generate(eng, [shared + [1]], 4, GREEDY)
    assert len(idx) == 3 and be.pool.free_blocks() == 64 - 3          # the cache holds the three full blocks
    generate(eng, [shared + [2, 3]], 4, GREEDY)
    assert eng.counters["cached_tokens"] == 192
    other = np.random.default_rng(1).integers(0, 512, size=200).tolist()
    generate(eng, [other], 4, GREEDY)
    assert len(idx) == 3 and idx.stats["evictions"] == 3 and be.pool.free_blocks() == 64 - 3
    assert MockOptions.parse("vocab=100,native_draft=true,fault=rollback_leak").native_draft
    with pytest.raises(ValueError):
        MockOptions.parse("nope=1")


def test_reasoning_budget_forces_the_closing_tag():
    """After `reasoning_budget` tokens inside the thinking block the closing tag's tokens replace the samples, one per round; drafts
    accepted beyond a forced token are not kept; without a budget nothing changes."""
    close = (7001, 7002)
    opts = MockOptions(slots=2, vocab=8000)
    base = generate(Engine(MockBackend(opts), None, spec="copy"), [list(range(10, 40))], 24, GREEDY)[0]
    assert not any(t in close for t in base)
    eng = Engine(MockBackend(opts), None, spec="copy")
    req = Request("r", list(range(10, 40)), 24, GREEDY, reasoning_budget=5, think_close_ids=close, reasoning_open=True)
    eng.submit(req)
    out = []
    while eng.has_work():
        for ev in eng.step():
            if ev.kind == "tokens":
                out.extend(ev.tokens)
    assert len(out) == 24
    i = out.index(close[0])
    assert i == 5 and out[i + 1] == close[1]               # the reply's token at index `budget` is the forced close (index 0 is counted)
    assert out[:i] == base[:i]                               # identical up to the forced close
    assert out.count(close[0]) == 1
    # a closing tag produced by the model itself ends the block: no forcing afterwards
    eng2 = Engine(MockBackend(opts), None, spec="none")
    nat = (base[2], base[3])
    eng2.submit(Request("n", list(range(10, 40)), 24, GREEDY, reasoning_budget=8, think_close_ids=nat, reasoning_open=True))
    out2 = []
    while eng2.has_work():
        for ev in eng2.step():
            if ev.kind == "tokens":
                out2.extend(ev.tokens)
    assert out2 == base


def _run_budget(budget, close, spec="copy", prompt=None, n=12):
    eng = Engine(MockBackend(MockOptions(slots=2, vocab=8000)), None, spec=spec)
    eng.submit(Request("r", prompt or list(range(10, 40)), n, GREEDY, reasoning_budget=budget, think_close_ids=close, reasoning_open=True))
    out = []
    while eng.has_work():
        for ev in eng.step():
            if ev.kind == "tokens":
                out.extend(ev.tokens)
    return out


def test_reasoning_budget_zero_one_and_a_close_sampled_first():
    """The close is forced at the reply's index `budget` (0 -> the very first token, which is sampled at the end of prefill); a close the
    model commits itself, even as its first token, spends the budget and is never forced again.  Serial and drafted paths agree."""
    base = generate(Engine(MockBackend(MockOptions(slots=2, vocab=8000)), None, spec="none"), [list(range(10, 40))], 12, GREEDY)[0]
    for spec in ("none", "copy"):
        out0 = _run_budget(0, (7001,), spec)
        assert out0[0] == 7001 and out0.count(7001) == 1
        out1 = _run_budget(1, (7001,), spec)
        assert out1[0] == base[0] and out1[1] == 7001 and out1.count(7001) == 1
        # the model's own first token is the close tag: the block ends there and nothing is forced later
        first = _run_budget(4, (base[0],), spec)
        assert first == base
        # a two-token close with budget 0 occupies indices 0 and 1
        two = _run_budget(0, (7001, 7002), spec)
        assert two[:2] == [7001, 7002] and two.count(7001) == 1


def test_burst_prefill_serves_short_prompts_first_and_never_starves_a_long_one():
    rng = np.random.default_rng(5)
    lens = [3000, 40, 700, 41, 2500, 90, 39, 1200, 64, 8]
    prompts = [rng.integers(0, 512, size=n).tolist() for n in lens]

    def run(policy, **kw):
        eng = Engine(MockBackend(MockOptions(slots=16, max_rows=512)), spec="none", prefill_policy=policy, prefill_chunk=256, **kw)
        for i, p in enumerate(prompts):
            eng.submit(Request(str(i), p, 6, GREEDY))
        first, out, step = {}, {str(i): [] for i in range(len(prompts))}, 0
        while eng.has_work():
            step += 1
            for ev in eng.step():
                if ev.kind == "tokens":
                    first.setdefault(ev.id, step)
                    out[ev.id].extend(ev.tokens)
        return first, out, step

    f_serial, o_serial, n_serial = run("serial")
    f_burst, o_burst, n_burst = run("burst")
    assert o_serial == o_burst                                     # the policy changes no token
    # serial: arrival order, so the 8-token prompt waits for all the long ones; burst: the short ones share the first steps
    short = [str(i) for i, n in enumerate(lens) if n <= 90]
    assert max(f_burst[i] for i in short) <= 2 and f_serial["9"] > 30
    assert sorted(f_burst.values())[len(lens) // 2] < sorted(f_serial.values())[len(lens) // 2]
    # a stream of new short prompts cannot starve the long one: it is served at least every PREFILL_PASS_GUARD + 1 steps
    eng = Engine(MockBackend(MockOptions(slots=64, max_rows=512)), spec="none", prefill_chunk=256, burst_cap=1)
    eng.submit(Request("long", prompts[0], 2, GREEDY))
    k, done_at = 0, None
    for step in range(1, 400):
        eng.submit(Request(f"s{k}", prompts[9], 1, GREEDY))
        eng.submit(Request(f"t{k}", prompts[9], 1, GREEDY))
        k += 1
        if any(ev.id == "long" and ev.kind == "tokens" for ev in eng.step()):
            done_at = step
            break
    assert done_at is not None and done_at <= (3000 // 256 + 1) * 10


def test_tree_rounds_commit_the_serial_tokens_and_keep_more_than_chains():
    """Tree windows on the mock: same tokens as the serial run at every tree size, greedy and sampled; with a drafter whose first candidate
    is wrong a quarter of the time but whose second is then right, trees keep more drafts per round than chains over the same offers."""
    p = harness.default_prompts(512)
    for sampling in (GREEDY, harness.SAMPLING):
        serial = generate(Engine(MockBackend(MockOptions()), spec="none"), p, 64, sampling)
        chain = Engine(MockBackend(MockOptions(native_draft=True, lattice=True)), spec="auto", max_drafts=4)
        assert generate(chain, p, 64, sampling) == serial
        tree = Engine(MockBackend(MockOptions(native_draft=True, lattice=True, trees=True)), spec="auto", max_drafts=4, trees=TreeConfig(max_nodes=12))
        assert generate(tree, p, 64, sampling) == serial
        assert tree.counters["tree_rounds"] == tree.counters["rounds"] > 0
        assert tree.counters["rounds"] < chain.counters["rounds"], (tree.counters, chain.counters)
    # the harness check catches a backend whose rejected tree rows leak into the state
    assert harness.trees_equal_serial(mk(native_draft=True, lattice=True, trees=True), 512) is None
    assert harness.trees_equal_serial(mk(native_draft=True, lattice=True, trees=True, fault="rollback_leak"), 512) is not None


def test_tree_rounds_with_stop_ids_budgets_and_many_streams():
    """Stop tokens and length limits inside an accepted path end the request at the same token as the serial run; more streams than the
    window has rows still get their anchors."""
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 512, size=int(n)).tolist() for n in rng.integers(3, 40, size=12)]
    for kw in (dict(), dict(eos=7, eos_after=9)):
        serial = generate(Engine(MockBackend(MockOptions(slots=16, **kw)), spec="none"), prompts, 23, GREEDY, stop_ids=(7,))
        eng = Engine(MockBackend(MockOptions(slots=16, native_draft=True, lattice=True, trees=True, **kw)), spec="auto", max_drafts=4, window_rows=16,
                     trees=TreeConfig(max_nodes=8))
        assert generate(eng, prompts, 23, GREEDY, stop_ids=(7,)) == serial


def test_mock_tree_window_rows_equal_one_row_steps():
    """Each row of a tree window returns what a one-row step returns after the tokens on its path; commit_path refuses rows that are no path."""
    be = MockBackend(MockOptions(trees=True))
    ctx = [5, 6, 7]
    be.prefill_slice(0, 0, ctx[:-1], 8, False)
    q = TreeRequest(0, [7, 11, 12, 13, 14], [-1, 0, 0, 1, 2], 2)
    assert q.depths() == [0, 1, 1, 2, 2]
    rows = be.step_tree([q], 8)[0]
    for r, path in enumerate(([7], [7, 11], [7, 12], [7, 11, 13], [7, 12, 14])):
        ref = MockBackend(MockOptions())
        ref.prefill_slice(0, 0, ctx[:-1] + path[:-1], 8, False) if len(ctx[:-1] + path[:-1]) else None
        from rexl3_b200.engine import RowRequest
        one = ref.step([RowRequest(0, [path[-1]], len(ctx) - 1 + len(path) - 1)], 8)[0][0]
        assert (one.ids == rows[r].ids).all() and (one.values == rows[r].values).all()
    with pytest.raises(BackendError):
        be.commit_path(0, [1, 4])
    be.step_tree([q], 8)
    be.commit_path(0, [2, 4])
    assert be.ctx[0] == [5, 6, 7, 12, 14]


@pytest.mark.parametrize("policy", ["legacy", "curve", "plan", "margin", "scored"])
def test_budget_policies_never_change_a_token(policy):
    from rexl3_b200.sched import DraftCost, RoundCost, StepCost
    p = harness.default_prompts(512) + [harness.default_prompts(512)[1][:20] * 5]
    serial = generate(Engine(MockBackend(MockOptions()), spec="none"), p, 40, harness.SAMPLING)
    from rexl3_b200.sched import CostModel
    rc = RoundCost(StepCost({1: CostModel([(1, 10.0), (64, 14.0)]), 8: CostModel([(8, 11.0), (64, 16.0)])}),
                   DraftCost(CostModel([(1, 1.0), (8, 2.0)]), CostModel([(1, 0.2), (32, 0.8)]), 0.5))
    for kw in (dict(), dict(round_cost=rc)):
        eng = Engine(MockBackend(MockOptions(native_draft=True)), spec="auto", max_drafts=4, window_rows=10, budget_policy=policy, **kw)
        assert generate(eng, p, 40, harness.SAMPLING) == serial
        assert eng.counters["accepted"] > 0
    with pytest.raises(ValueError):
        Engine(MockBackend(MockOptions()), budget_policy="greedy")


def test_scored_policy_gives_scarce_rows_to_the_confident_stream():
    """Two streams, a window with room for four drafts in all.  The drafter is sure of one stream's picks and unsure of the other's:
    `scored` (every pick asked for, the confidences share the rows) verifies the sure stream's whole chain, `legacy` (one measured rate per
    stream) leaves the other stream a real share; `plan` with a costly draft stops drafting a stream whose measured acceptance has collapsed."""
    from rexl3_b200.engine import DraftOffer
    from rexl3_b200.sched import CostModel, DraftCost, RoundCost, StepCost

    class Sure(MockBackend):
        rows_by_slot = None

        def propose_batch(self, asks):
            out = super().propose_batch(asks)
            for a in asks:
                out[a.slot] = DraftOffer(out[a.slot].tokens, [0.95 if a.slot == sure_slot[0] else 0.15] * len(out[a.slot].tokens))
            return out

        def step(self, reqs, candidates):
            if len(reqs) == 2:                      # only the rounds in which the two streams compete for the rows
                for r in reqs:
                    self.rows_by_slot.setdefault(r.slot, []).append(len(r.tokens) - 1)
            return super().step(reqs, candidates)

    p = harness.default_prompts(512, (9, 11))
    got = {}
    for policy in ("legacy", "scored"):
        be = Sure(MockOptions(native_draft=True, draft_error=0.0))
        be.rows_by_slot = {}
        eng = Engine(be, spec="auto", max_drafts=4, window_rows=6, budget_policy=policy)
        sure_slot = [None]
        for i, q in enumerate(p):
            eng.submit(Request(str(i), q, 40, GREEDY))
        eng.step()
        sure_slot[0] = eng.seqs["0"].slot
        other = eng.seqs["1"].slot
        while eng.has_work():
            eng.step()
        got[policy] = (sum(be.rows_by_slot[sure_slot[0]]), sum(be.rows_by_slot[other]))
    assert got["scored"][0] > got["scored"][1] * 2        # the confident stream rode with (almost) all the drafts
    assert got["legacy"][1] * 4 > sum(got["legacy"])        # one measured rate each, both accept everything: the other stream keeps a real share
    assert got["scored"][1] * 10 < sum(got["scored"])
    # plan: a drafter that is always wrong drives the stream's curve down until the plan, which counts the draft's cost, stops asking
    rc = RoundCost(StepCost.rows_only(CostModel([(1, 10.0), (64, 12.0)])), DraftCost(CostModel([(1, 6.0), (8, 8.0)]), CostModel([(1, 0.5), (32, 2.0)]), 1.0))
    eng = Engine(MockBackend(MockOptions(native_draft=True, draft_error=1.0)), spec="auto", max_drafts=4, budget_policy="plan", round_cost=rc)
    generate(eng, [p[0]], 40, GREEDY)
    assert eng.counters.get("planned_out", 0) > 10 and eng.counters["drafted"] < 40
