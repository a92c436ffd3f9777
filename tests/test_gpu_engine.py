"""The engine's exactness harness on the CUDA backend (real kernels, CUDA-graph replay)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def make_backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["test-hd128"]
    w = dense.random_weights(cfg, seed=3)
    model = dense.DenseGPU(w, num_pages=96, max_rows=64, max_seqs=8, max_blocks_per_seq=8, max_prefill_rows=512)
    state = {}

    def make():
        # one model, fresh bookkeeping (the KV pages are simply overwritten)
        state["b"] = DenseGpuBackend(model, max_slots=8)
        return state["b"]
    make.vocab = cfg.vocab
    return make


@pytest.mark.parametrize("check", ["row_invariance", "serial_batched_equals_solo", "drafted_equals_serial", "chunked_prefill_equals_whole",
                                   "rollback_equals_replay", "cached_equals_cold", "trees_equal_serial"])
def test_exactness_on_device(make_backend, check):
    from rexl3_b200.engine import harness
    assert getattr(harness, check)(make_backend, make_backend.vocab) is None


def test_smoke_entry():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import __graft_entry__ as g
    g.smoke()


def test_device_sampler_equals_host_sampler():
    """The verify kernel (keyed sampler + accept rule on the device) gives the engine the same tokens as the host sampler."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    from rexl3_b200.sampling import GREEDY, Sampling
    cfg = dense.CONFIGS["test-hd128"]
    w = dense.random_weights(cfg, seed=2)
    rng = np.random.default_rng(5)
    base = rng.integers(0, cfg.vocab, size=24).tolist()
    prompts = [base * 3, rng.integers(0, cfg.vocab, size=40).tolist()]          # a repetitive prompt gives the copy drafter something to offer
    samplings = [GREEDY, Sampling(seed=11, temperature=0.8, top_k=20, top_p=0.9)]
    outs = {}
    for dev in (False, True):
        m = dense.DenseGPU(w, num_pages=32, max_rows=64, max_seqs=4, max_blocks_per_seq=6, max_prefill_rows=256)
        eng = Engine(DenseGpuBackend(m, max_slots=4), None, window_rows=32, prefill_chunk=256, spec="copy", device_sampler=dev)
        assert eng.device_sampler == dev
        for i, (p, s) in enumerate(zip(prompts, samplings)):
            eng.submit(Request(f"r{i}", p, 14, s))
        got = {f"r{i}": [] for i in range(len(prompts))}
        for _ in range(200):
            if not eng.has_work():
                break
            for ev in eng.step():
                if ev.kind == "tokens":
                    got[ev.id].extend(ev.tokens)
                assert ev.kind != "error", ev.message
        outs[dev] = got
    assert outs[False] == outs[True]


def test_prefix_spill_tier_restores_pages_bit_for_bit(tmp_path):
    """Blocks evicted from a two-block device prefix cache go to the spill directory; the same prompt later gets them back (page bytes
    imported into fresh pages) and decodes exactly what the cold run decoded."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    from rexl3_b200.sampling import GREEDY
    from rexl3_b200.sched.prefix import CacheBudget, PrefixIndex
    from rexl3_b200.sched.spill import SpillStore
    cfg = dense.CONFIGS["test-hd128"]
    m = dense.DenseGPU(dense.random_weights(cfg, seed=6), num_pages=48, max_rows=64, max_seqs=4, max_blocks_per_seq=8, max_prefill_rows=512)
    be = DenseGpuBackend(m, max_slots=4)
    prefix = PrefixIndex(CacheBudget(max_bytes=2 * be.prefix_bytes_per_block()), block_tokens=64)
    spill = SpillStore(str(tmp_path / "spill"), max_bytes=1 << 30)
    eng = Engine(be, None, window_rows=16, prefill_chunk=256, spec="none", prefix=prefix, spill=spill)
    rng = np.random.default_rng(9)
    a, b = rng.integers(0, cfg.vocab, size=4 * 64 + 9).tolist(), rng.integers(0, cfg.vocab, size=4 * 64 + 9).tolist()

    def run(rid, prompt):
        eng.submit(Request(rid, prompt, 10, GREEDY))
        out = []
        for _ in range(200):
            if not eng.has_work():
                break
            for ev in eng.step():
                assert ev.kind != "error", ev.message
                if ev.kind == "tokens":
                    out.extend(ev.tokens)
        return out

    cold = run("a1", a)
    run("b1", b)
    assert len(spill) >= 2 and eng.counters.get("spilled_blocks", 0) >= 2
    before = eng.counters["cached_tokens"]
    warm = run("a2", a)
    assert warm == cold
    assert eng.counters.get("unspilled_blocks", 0) >= 1 and eng.counters["cached_tokens"] > before
    assert be.pool.total_blocks() - be.pool.free_blocks() == len(prefix.entries)
