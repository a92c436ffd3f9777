"""Tree windows on the CUDA backend: every row of a window of draft trees returns the bits of one-row steps along its path, an accepted
path that is not the tree's first chain is moved to its positions, and an engine that verifies trees emits the serial run's tokens."""
import hashlib

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["test-hd128"]
    return dense.DenseGPU(dense.random_weights(cfg, seed=3), num_pages=160, max_rows=64, max_seqs=8, max_blocks_per_seq=8, max_prefill_rows=512)


@pytest.fixture(scope="module", params=["fp8", "int8"])
def qmodel(request):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["test-hd128"]
    return dense.DenseGPU(dense.random_weights(cfg, seed=3), num_pages=160, max_rows=64, max_seqs=8, max_blocks_per_seq=8, max_prefill_rows=512,
                          kv_dtype=request.param)


def _serial_row(model, ctx, path, count):
    """The output of the last one-row step of a serial run: prompt ctx[:-1], then ctx[-1] and the path's tokens one by one."""
    from rexl3_b200.engine import RowRequest
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    be = DenseGpuBackend(model, max_slots=8, use_graphs=False)
    be.pool.alloc(96)          # the backend under test holds the model's first pages: this run keeps to pages 96..
    be.prefill_slice(3, 0, ctx[:-1], count, False)
    out = None
    for j, t in enumerate([ctx[-1]] + path):
        out = be.step([RowRequest(3, [t], len(ctx) - 1 + j)], count)[0][0]
        be.commit(3, 1)
    be.release(3)
    return out


@pytest.mark.parametrize("ctx_len", [6, 64, 65, 256, 257, 300])
def test_tree_window_rows_equal_serial_steps_bit_for_bit(model, ctx_len):
    """Anchors before, at and after a page boundary (64) and an attention chunk boundary (256); a second sequence shares the window."""
    from rexl3_b200.engine import RowRequest, TreeRequest
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    rng = np.random.default_rng(ctx_len)
    V = model.cfg.vocab
    ctx = rng.integers(0, V, size=ctx_len).tolist()
    other = rng.integers(0, V, size=40).tolist()
    toks = [ctx[-1]] + rng.integers(0, V, size=8).tolist()
    parents = [-1, 0, 1, 0, 3, 3, 1, 5, 2]          # first chain 0-1-2 (and 8 below it), a second branch 0-3-{4, 5-7}, 6 under 1
    be = DenseGpuBackend(model, max_slots=8)
    assert be.supports_trees()
    be.prefill_slice(1, 0, ctx[:-1], 8, False)
    be.prefill_slice(2, 0, other[:-1], 8, False)
    q1 = TreeRequest(1, toks, parents, len(ctx) - 1)
    q2 = TreeRequest(2, [other[-1], 17, 18], [-1, 0, 0], len(other) - 1)
    out1, out2 = be.step_tree([q1, q2], 8)
    assert be.take_error() is None
    for r in range(len(toks)):
        path, a = [], r
        while a > 0:
            path.append(toks[a])
            a = parents[a]
        ref = _serial_row(model, ctx, path[::-1], 8)
        assert np.array_equal(ref.ids, out1[r].ids) and np.array_equal(ref.values, out1[r].values), f"row {r} (depth {len(path)})"
    ref = _serial_row(model, other, [18], 8)
    assert np.array_equal(ref.ids, out2[2].ids) and np.array_equal(ref.values, out2[2].values)
    # keep 0-3-5-7 (no node of it sits where the first chain would put it) and the anchor alone in the other slot, then go on serially
    be.commit_path(1, [3, 5, 7])
    be.commit_path(2, [])
    nxt = be.step([RowRequest(1, [99], len(ctx) + 3), RowRequest(2, [55], len(other))], 8)
    assert be.take_error() is None
    ref = _serial_row(model, ctx, [toks[3], toks[5], toks[7], 99], 8)
    assert np.array_equal(ref.ids, nxt[0][0].ids) and np.array_equal(ref.values, nxt[0][0].values)
    ref = _serial_row(model, other, [55], 8)
    assert np.array_equal(ref.ids, nxt[1][0].ids) and np.array_equal(ref.values, nxt[1][0].values)
    st = be.stats()
    assert st["tree_windows"] == 1 and st["tree_moves"] == 3 and st["tree_copies"] > 0
    assert be.pool.free_blocks() + len(be.pages[1]) + len(be.pages[2]) == be.pool.total_blocks()      # private pages went back at commit_path
    be.release(1)
    be.release(2)
    assert be.pool.free_blocks() == be.pool.total_blocks()


def test_engine_tree_rounds_emit_the_serial_tokens(model):
    """The engine with tree rounds against the serial engine on the same backend class.  The drafter is an oracle with noise: it knows the
    serial continuation and puts the right token at a hashed rank of each level (or leaves it out), so accepted paths run through second
    and third candidates: private pages, ancestor copies and path moves all carry tokens that are then emitted."""
    from rexl3_b200.engine import DraftOffer, Engine, TreeConfig, generate, harness
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.spec.tree import Lattice
    V = model.cfg.vocab
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, V, size=n).tolist() for n in (3, 60, 150, 250)]
    n = 40
    for sampling in (harness.SAMPLING,):
        serial = generate(Engine(DenseGpuBackend(model, max_slots=8), spec="none"), prompts, n, sampling)

        class Oracle(DenseGpuBackend):
            def supports_native_draft(self):
                return True

            def propose_batch(self, asks):
                out = {}
                for a in asks:
                    i = next(k for k, p in enumerate(prompts) if a.context[:len(p)] == p and len(a.context) - len(p) <= n)
                    g = len(a.context) - len(prompts[i])
                    ids, un = [], []
                    for j in range(a.max_drafts):
                        hsh = int.from_bytes(hashlib.blake2b(f"{i}.{g}.{j}".encode(), digest_size=8).digest(), "little")
                        cand = [(hsh >> (8 * k)) % V for k in range(1, 5)]
                        if g + j < len(serial[i]) and hsh % 5 < 4:
                            cand[hsh % 5] = serial[i][g + j]
                        ids.append(cand)
                        un.append([3.0, 2.0, 1.0, 0.0])
                    out[a.slot] = DraftOffer([c[0] for c in ids], [], Lattice(ids, un))
                return out

        be = Oracle(model, max_slots=8)
        assert be.supports_trees()
        eng = Engine(be, spec="auto", max_drafts=4, trees=TreeConfig(max_nodes=12))
        treed = generate(eng, prompts, n, sampling)
        assert harness._diff("trees", serial, treed) is None
        st = be.stats()
        assert eng.counters["tree_rounds"] > 0 and eng.counters["accepted"] > 20 and st["tree_moves"] > 0 and st["tree_copies"] > 0, (eng.counters, st)
        assert eng.counters["rounds"] < n        # fewer rounds than tokens: paths were kept
        assert be.pool.free_blocks() == be.pool.total_blocks()


@pytest.mark.parametrize("ctx_len", [65, 257])
def test_tree_window_over_quantized_caches(qmodel, ctx_len):
    """The same property over an fp8 cache (static per-head scales) and an int8 cache (one scale per token and head, which moves with its row)."""
    from rexl3_b200.engine import RowRequest, TreeRequest
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    rng = np.random.default_rng(ctx_len + 1000)
    V = qmodel.cfg.vocab
    ctx = rng.integers(0, V, size=ctx_len).tolist()
    toks = [ctx[-1]] + rng.integers(0, V, size=5).tolist()
    parents = [-1, 0, 0, 2, 1, 3]
    be = DenseGpuBackend(qmodel, max_slots=8)
    assert be.supports_trees()
    be.prefill_slice(1, 0, ctx[:-1], 8, False)
    out = be.step_tree([TreeRequest(1, toks, parents, len(ctx) - 1)], 8)[0]
    assert be.take_error() is None
    for r in range(len(toks)):
        path, a = [], r
        while a > 0:
            path.append(toks[a])
            a = parents[a]
        ref = _serial_row(qmodel, ctx, path[::-1], 8)
        assert np.array_equal(ref.ids, out[r].ids) and np.array_equal(ref.values, out[r].values), f"row {r}"
    be.commit_path(1, [2, 3, 5])
    nxt = be.step([RowRequest(1, [77], len(ctx) + 3)], 8)[0][0]
    ref = _serial_row(qmodel, ctx, [toks[2], toks[3], toks[5], 77], 8)
    assert np.array_equal(ref.ids, nxt.ids) and np.array_equal(ref.values, nxt.values)
    be.release(1)
    assert be.pool.free_blocks() == be.pool.total_blocks()
