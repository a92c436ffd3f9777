"""Scheduling primitives and speculation logic (CPU)."""
import numpy as np
import pytest

from rexl3_b200 import sched, spec
from rexl3_b200.sampling import Sampling


def _adm(capacity_tokens=1000, slots=4):
    model = sched.ModelMemory(weights_bytes=100, kv_bytes_per_token=10, state_bytes_per_slot=5)
    return sched.Admission(100 + capacity_tokens * 10 + 5 * slots, 0, model, slots)


def test_admission_fails_closed_and_releases():
    a = _adm(1000, 2)
    with pytest.raises(sched.AdmitError) as e:
        a.check(2000)
    assert e.value.kind == "NeverFits"
    s0 = a.admit(600)
    with pytest.raises(sched.AdmitError) as e:
        a.admit(600)
    assert e.value.kind == "NoMemory"
    s1 = a.admit(300)
    with pytest.raises(sched.AdmitError) as e:
        a.admit(1)
    assert e.value.kind == "NoSlot"
    a.release(s0)
    assert a.admit(600) == s0 and s1 != s0
    a.with_max_context(500)
    with pytest.raises(sched.AdmitError) as e:
        a.check(501)
    assert e.value.kind == "ContextTooLong"


def test_admission_refuses_zero_byte_kv_and_pins():
    with pytest.raises(sched.MemoryError_):
        sched.Admission(1000, 0, sched.ModelMemory(10, 0), 1)
    a = _adm(100, 2)
    a.pin(500)
    with pytest.raises(sched.AdmitError):
        a.admit(60)
    a.unpin(500)
    a.admit(60)
    a.with_kv_tokens(80)
    with pytest.raises(sched.AdmitError):
        a.admit(30)


def test_block_pool_refcounts():
    p = sched.BlockPool(4, 64)
    assert p.blocks_for(65) == 2
    a = p.alloc(3)
    assert p.alloc(2) is None
    p.retain(a[:1])
    p.release(a)
    assert p.free_blocks() == 3 and p.refcount(a[0]) == 1
    p.release(a[:1])
    assert p.free_blocks() == 4
    with pytest.raises(AssertionError):
        p.release(a[:1])
    with pytest.raises(AssertionError):
        p.retain(a[:1])


def test_kv_layout_bytes():
    l = sched.KvLayout.gqa(64, 8, 128, "bf16", 64)
    assert l.bytes_per_token() == 2 * 8 * 128 * 2 * 64 and l.bytes_per_page() == l.bytes_per_token() * 64
    assert sched.KvLayout.gqa(64, 8, 128, "fp8").bytes_per_token() == 64 * 2 * (8 * 128 + 32)
    assert sched.KvLayout.mla(61, 512, 64).bytes_per_token() == 61 * 576 * 2


def test_prefix_index_strict_prefix_lru_and_ghosts():
    idx = sched.PrefixIndex(sched.CacheBudget(max_bytes=3 * 100), "lru", block_tokens=4)
    toks = list(range(20))
    h = sched.chain_hashes(toks, 4)
    assert len(h) == 5 and sched.chain_hashes(toks[:8], 4) == h[:2]
    assert sched.chain_hashes(toks, 4, b"other-model") != h
    dup, ev = idx.insert(h[:3], ["a", "b", "c"], 100)
    assert not dup and not ev
    assert [e.handle for e in idx.lookup(h, 20)] == ["a", "b", "c"]
    assert [e.handle for e in idx.lookup(h, 12)] == ["a", "b"]       # strict: 12 tokens = 3 blocks, one must still run
    assert idx.lookup(h, 4) == []
    h2 = sched.chain_hashes([99] * 8, 4)
    dup, ev = idx.insert(h2, ["x", "y"], 100)
    assert ev == ["c", "b"]                                             # leaves first, least recently used
    assert idx.lookup(h, 20)[0].handle == "a" and idx.stats["ghost_hits"] >= 1
    dup, _ = idx.insert(h[:1], ["again"], 100)
    assert dup == ["again"]                                            # an existing block keeps its handle
    assert idx.reach_tokens() == 8


def test_prefix_size_aware_prefers_cheap_victims():
    idx = sched.PrefixIndex(sched.CacheBudget(max_bytes=250), "size_aware", block_tokens=4)
    ha, hb, hc = (sched.chain_hashes([i] * 4, 4) for i in (1, 2, 3))
    idx.insert(ha, ["big-cheap"], 100, cost_each=1.0)
    idx.insert(hb, ["costly"], 100, cost_each=1000.0)
    _, ev = idx.insert(hc, ["new"], 100, cost_each=10.0)
    assert ev == ["big-cheap"]


def test_plan_cuts():
    cuts = sched.plan_cuts(0, 10000, sched.CutPolicy(every_tokens=4096, align=64))
    assert cuts[0] == 4096 and cuts[1] == 8192 and cuts[-1] == 9984 and all(c % 64 == 0 for c in cuts)
    assert sched.plan_cuts(100, 100, sched.CutPolicy()) == []


def test_budget_planner_greedy_and_cost_model():
    d = [sched.Demand.geometric(0.9, 4), sched.Demand.geometric(0.3, 4)]
    assert sched.allocate(d, 2 + 3) == [3, 0]
    assert sched.allocate(d, 1) == [0, 0]
    assert sched.Demand.from_conditional([0.5, 0.5], 3).values == [0.5, 0.25, 0.125]
    assert abs(sched.expected_tokens(0.5, 2) - 1.75) < 1e-12
    flat = sched.CostModel([(1, 10.0), (64, 10.5)])
    rows, drafts = sched.choose_budget(flat, d, 64)
    assert rows == 2 + 8 and drafts == [4, 4]                         # rows are nearly free: take every draft
    steep = sched.CostModel([(1, 1.0), (2, 2.0), (64, 64.0)])
    rows, drafts = sched.choose_budget(steep, d, 64)
    assert rows == 2 and drafts == [0, 0]                             # a row costs a full step: no drafts
    with pytest.raises(ValueError):
        sched.CostModel([])
    with pytest.raises(ValueError):
        sched.CostModel([(1, -1.0)])
    assert abs(flat.ms(128) - (10.5 + 0.5 * 64 / 63)) < 1e-9           # extended past the table by its last slope
    rc = sched.RoundCost(sched.StepCost.from_grid([(1, 1, 10), (64, 1, 11), (1, 8, 12), (64, 8, 13)]),
                         sched.DraftCost(sched.CostModel([(1, 100.0)]), sched.CostModel([(1, 1.0)])), kv_ms_per_token=0.0)
    assert sched.plan_round(rc, d, 64, draft_sunk=False).drafts == [0, 0]   # the draft itself is too dear to pay for
    assert sum(sched.plan_round(rc, d, 64, draft_sunk=True).drafts) > 0
    assert sched.adaptive_block(3, False, 2) == 8 and sched.adaptive_block(12, True, 2) == 16 and sched.adaptive_block(12, True, 9) == 8


def test_accept_and_stats():
    assert spec.accept([1, 2, 3], [1, 2, 9, 4]) == 2 and spec.accept([], [5]) == 0 and spec.accept([7], [8]) == 0
    st = spec.AcceptStats(0.5, 4.0, 0.9)
    for _ in range(50):
        st.update(4, 4)
    assert st.accept_rate() > 0.9
    for _ in range(50):
        st.update(4, 0)
    low = st.accept_rate()
    assert low < 0.2
    for _ in range(50):
        st.relax()
    assert st.accept_rate() > low                                       # drifts back to the prior so drafting is retried


def test_copy_drafter_continues_longest_match():
    d = spec.CopyDrafter(min_match=3, max_draft=5)
    t = [1, 2, 3, 4, 5, 6, 7, 8, 9, 1, 2, 3]
    assert d.propose(t, 4) == [4, 5, 6, 7]
    assert d.propose(t, 9) == [4, 5, 6, 7, 8]                           # capped by max_draft
    assert d.propose([1, 2], 4) == [] and spec.CopyDrafter(3, 5).propose([5, 6, 7, 8], 4) == []
    m, cont = d.propose_after(t, [4, 5], 3)
    assert m >= 3 and cont == [6, 7, 8]
    assert d.propose([9, 9, 9, 1], 3) == []                             # shorter sequence: the index is rebuilt


def test_spec_mode_and_keyed_draft_pick():
    assert spec.SpecMode("auto").native and spec.SpecMode("copy").copy and not spec.SpecMode("none").enabled
    with pytest.raises(ValueError):
        spec.SpecMode("fast")
    vals, ids = [0.1, 2.0, 2.0], [7, 9, 3]
    assert spec.draft_pick(vals, ids, 5, None) == 3
    s = Sampling(seed=11, temperature=1.0, top_k=3, top_p=1.0)
    from rexl3_b200.sampling import choose
    assert spec.draft_pick(vals, ids, 5, s) == choose(vals, ids, 5, s)


def test_depth_curve_and_arbiter_choose_and_probe():
    c = spec.DepthCurve([0.8, 0.5], weight=2.0, decay=0.9, chain=0.9)
    assert abs(c.alpha(1) - 0.8) < 1e-9 and abs(c.alpha(2) - 0.72) < 1e-9
    for _ in range(30):
        c.observe(2, 0)
    assert c.alpha(1) < 0.2 and c.expected_tokens(2) < 1.3
    arb = spec.Arbiter(verify_ms=lambda s, r: 10.0 + 4.0 * r, native_ms=lambda s, r: 0.5, probe_every=4)
    picks = arb.choose({"a": dict(copy=3, native=4)}, 64)
    assert picks["a"].kind in ("copy", "native") and picks["a"].n >= 1
    for _ in range(40):                                                 # everything proposed is rejected
        ch = arb.choose({"a": dict(copy=3, native=4)}, 64)["a"]
        arb.observe("a", ch, 0)
    kinds = []
    for _ in range(12):
        ch = arb.choose({"a": dict(copy=3, native=4)}, 64)["a"]
        kinds.append((ch.kind, ch.n))
        arb.observe("a", ch, 0)
    assert ("none", 0) in kinds and any(k != "none" and n == 1 for k, n in kinds)   # mostly serial, with one-deep probes
    dear = spec.Arbiter(verify_ms=lambda s, r: 10.0 * r)
    assert dear.choose({"a": dict(copy=3, native=0)}, 64)["a"].kind == "none"


def test_draft_tree_best_first_and_accept():
    lat = spec.Lattice(ids=[[10, 11, 12], [20, 21, 22]], unary=[[3.0, 2.0, 0.1], [2.5, 2.4, 0.0]], edge=None)
    t = spec.best_first(lat, 5, spec.Policy(branch=2))
    assert t.tokens[0] == 10 and t.parents[0] == -1 and len(t) == 5
    assert spec.best_first(lat, 3, spec.Policy(branch=2)).tokens == t.tokens[:3]          # nested budgets
    p = t.probabilities()
    assert all(p[i] >= p[i + 1] for i in range(len(p) - 1))
    child = next(i for i in range(len(t)) if t.parents[i] == 0)
    samples = [0] * (len(t) + 1)
    samples[0] = 10
    samples[1] = t.tokens[child]
    samples[child + 1] = 777
    path, committed = spec.accept_tree(t, samples)
    assert path == [0, child] and committed == [10, t.tokens[child], 777]
    path, committed = spec.accept_tree(t, [999] + [0] * len(t))
    assert path == [] and committed == [999]
    g = spec.with_copy(t, [10, 55], 8)
    assert 55 in g.tokens and g.parents[g.tokens.index(55)] == 0


def test_ngram_drafter_learns_short_patterns_and_stays_silent_without_evidence():
    from rexl3_b200.spec import NgramDrafter
    d = NgramDrafter(order=3, max_draft=5, min_count=2)
    seq = [1, 2, 3, 9, 1, 2, 3, 8, 1, 2]
    assert d.propose(seq, 4)[:1] == [3]                    # "1 2" was followed by 3 twice
    assert d.propose(seq, 4) == [3]                        # ... and after "2 3" came 9 once and 8 once: no evidence, the chain stops
    assert d.propose(seq + [3], 4) == []
    assert NgramDrafter().propose([5, 6, 7, 8], 4) == []   # nothing repeated: nothing offered
    # incremental indexing gives the same tables as indexing at once, and a shorter sequence resets them
    a, b = NgramDrafter(order=3), NgramDrafter(order=3)
    for n in range(2, len(seq) + 1):
        a.propose(seq[:n], 3)
    b.propose(seq, 3)
    assert a.tables == b.tables
    a.propose([4, 4], 3)
    assert a.indexed == 2 and all(len(t) <= 1 for t in a.tables)
    assert d.propose(seq, 0) == []


def test_engine_uses_the_ngram_drafter_and_stays_exact():
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.mock import MockBackend, MockOptions
    from rexl3_b200.sampling import GREEDY
    prompt = [3, 4, 5, 6] * 6

    def run(spec):
        # order=2: the mock's next token depends on the last two tokens only, so its text falls into a cycle an n-gram table can learn
        eng = Engine(MockBackend(MockOptions(order=2, vocab=16)), None, window_rows=16, spec=spec)
        eng.submit(Request("a", prompt, 96, GREEDY))
        out = []
        for _ in range(600):
            if not eng.has_work():
                break
            for ev in eng.step():
                assert ev.kind != "error", ev.message
                if ev.kind == "tokens":
                    out.extend(ev.tokens)
        return out, eng.counters
    plain, _ = run("none")
    drafted, c = run("ngram")
    assert drafted == plain and c["drafted"] > 0 and c["accepted"] > 0


def test_engine_with_the_arbiter_stays_exact_and_learns_to_draft():
    """The arbiter decides per round how many offered drafts are worth verifying; whatever it decides, the tokens equal plain decoding.  On a
    model whose text cycles the copy / n-gram drafts are almost always right, so after its probes the arbiter keeps drafting."""
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.mock import MockBackend, MockOptions
    from rexl3_b200.sampling import GREEDY
    from rexl3_b200.spec import Arbiter
    prompts = [[3, 4, 5, 6] * 6, [7, 8, 9] * 9]

    def run(arbiter):
        eng = Engine(MockBackend(MockOptions(order=2, vocab=16)), None, window_rows=16, spec="auto" if arbiter else "none", arbiter=arbiter)
        for i, p in enumerate(prompts):
            eng.submit(Request(f"r{i}", p, 120, GREEDY))
        out = {f"r{i}": [] for i in range(len(prompts))}
        for _ in range(800):
            if not eng.has_work():
                break
            for ev in eng.step():
                assert ev.kind != "error", ev.message
                if ev.kind == "tokens":
                    out[ev.id].extend(ev.tokens)
        return out, eng.counters
    plain, c0 = run(None)
    arb = Arbiter(verify_ms=lambda streams, rows: 10.0 + 0.05 * rows, probe_every=4)
    got, c1 = run(arb)
    assert got == plain
    assert c1["drafted"] > 0 and c1["accepted"] > 0.8 * c1["drafted"] and c1["rounds"] < c0["rounds"]
    assert arb.streams == {}                                  # forgotten when the requests finished
