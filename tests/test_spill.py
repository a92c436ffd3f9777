"""The prefix cache's spill tier: the store itself, and the engine continuing a lookup from it."""
import os

from rexl3_b200.engine import Engine, Request
from rexl3_b200.engine.mock import MockBackend, MockOptions
from rexl3_b200.sampling import GREEDY
from rexl3_b200.sched.prefix import CacheBudget, PrefixIndex
from rexl3_b200.sched.spill import HEADER, SpillStore


def test_store_roundtrip_budget_adoption_and_corruption(tmp_path):
    d = str(tmp_path / "spill")
    st = SpillStore(d, max_bytes=3 * (HEADER.size + 100))
    keys = [bytes([i]) * 8 for i in range(5)]
    for k in keys[:3]:
        assert st.put(k, k * 12 + b"abcd")
    assert st.get(keys[0]) == keys[0] * 12 + b"abcd"          # touch 0: 1 is now the oldest
    assert st.put(keys[3], b"x" * 100)
    assert keys[1] not in st and keys[0] in st and len(st) == 3 and st.stats["evictions"] == 1
    assert not os.path.exists(os.path.join(d, keys[1].hex() + ".blk"))
    assert not st.put(keys[4], b"y" * 10_000)                  # larger than the whole budget
    assert st.get(keys[4]) is None and st.stats["misses"] == 1
    # a restart adopts what is on disk
    st2 = SpillStore(d, max_bytes=1 << 20)
    assert sorted(st2.index) == sorted([keys[0], keys[2], keys[3]]) and st2.get(keys[3]) == b"x" * 100
    # a damaged file is dropped, not served
    path = os.path.join(d, keys[2].hex() + ".blk")
    raw = bytearray(open(path, "rb").read())
    raw[-1] ^= 0xFF
    open(path, "wb").write(raw)
    assert st2.get(keys[2]) is None and keys[2] not in st2 and st2.stats["corrupt"] == 1 and not os.path.exists(path)


def _run(eng, rid, prompt, n=6):
    eng.submit(Request(rid, prompt, n, GREEDY))
    out = []
    for _ in range(500):
        if not eng.has_work():
            break
        for ev in eng.step():
            assert ev.kind != "error", ev.message
            if ev.kind == "tokens" and ev.id == rid:
                out.extend(ev.tokens)
    return out


def test_engine_refills_an_evicted_prefix_from_the_spill_tier(tmp_path):
    opts = MockOptions()
    bt = opts.block_tokens
    be = MockBackend(opts)
    per_block = be.prefix_bytes_per_block()
    prefix = PrefixIndex(CacheBudget(max_bytes=3 * per_block), block_tokens=bt)          # room for three blocks only
    spill = SpillStore(str(tmp_path / "spill"), max_bytes=1 << 20)
    eng = Engine(be, None, window_rows=8, prefill_chunk=4 * bt, spec="none", prefix=prefix, spill=spill)
    a = [(7 * i + 3) % opts.vocab for i in range(5 * bt + 2)]
    b = [(11 * i + 5) % opts.vocab for i in range(5 * bt + 2)]
    cold = _run(eng, "a1", a)
    _run(eng, "b1", b)                                            # pushes a's blocks out of the three-block device cache
    assert eng.counters.get("spilled_blocks", 0) >= 3 and len(spill) >= 3
    before = eng.counters["cached_tokens"]
    warm = _run(eng, "a2", a)
    assert warm == cold
    assert eng.counters.get("unspilled_blocks", 0) >= 1
    assert eng.counters["cached_tokens"] - before >= bt          # part of the prompt came back without being recomputed
    # no page leaks: everything the index still holds is accounted for
    assert be.pool.total_blocks() - be.pool.free_blocks() == len(prefix.entries)


def test_server_flag_wires_the_spill_tier(tmp_path):
    from starlette.testclient import TestClient

    from rexl3_b200.server import main
    d = str(tmp_path / "spill")
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512", "--slots", "2", "--max-model-len", "2048", "--prefix-cache-mib", "1",
                                     "--prefix-spill-dir", d, "--prefix-spill-mib", "64"])
    app, handle = main.make_app(args)
    try:
        assert handle.wait_ready(10)
        with TestClient(app) as c:
            a, b = "a" * 1500, "b" * 1500                         # 23 blocks each against a 16-block device cache
            for p in (a, b, a):
                r = c.post("/v1/completions", json={"prompt": p, "max_tokens": 4, "temperature": 0})
                assert r.status_code == 200
            t = c.get("/metrics").text
        vals = {ln.split(" ")[0]: float(ln.split(" ")[1]) for ln in t.splitlines() if ln.startswith("rexl3_") and "{" not in ln}
        assert vals["rexl3_engine_spilled_blocks_total"] > 0 and vals["rexl3_engine_unspilled_blocks_total"] > 0
        assert vals["rexl3_prefix_spill_entries"] > 0 and vals["rexl3_prefix_cache_entries"] > 0
        assert any(n.endswith(".blk") for n in os.listdir(d))
    finally:
        handle.stop()


def test_cache_namespace_separates_packs_kv_dtypes_and_scales():
    """The prefix-cache / spill namespace changes with the pack fingerprint, the KV dtype and the FP8 scale tensor, not only the name."""
    import types
    import torch
    from rexl3_b200.models import dense
    from rexl3_b200.server.main import cache_namespace
    cfg = dense.CONFIGS["test-hd128"]
    a16 = types.SimpleNamespace(kv_dtype="bf16")
    a8 = types.SimpleNamespace(kv_dtype="fp8")
    base = cache_namespace("m", cfg, {"pack_fingerprint": "aa"}, a16)
    assert base == cache_namespace("m", cfg, {"pack_fingerprint": "aa"}, a16)
    assert base != cache_namespace("m", cfg, {"pack_fingerprint": "bb"}, a16)       # re-quantised pack, same served name
    assert base != cache_namespace("m", cfg, {}, a16)                               # random-init is its own namespace
    assert base != cache_namespace("m", cfg, {"pack_fingerprint": "aa"}, a8)
    m1 = types.SimpleNamespace(kv_scale=torch.ones(2, 2, 2))
    m2 = types.SimpleNamespace(kv_scale=torch.ones(2, 2, 2) * 1.5)
    assert cache_namespace("m", cfg, {"pack_fingerprint": "aa"}, a8, m1) != cache_namespace("m", cfg, {"pack_fingerprint": "aa"}, a8, m2)
