"""Hybrid (Mamba2 + attention) executor on the sm_100a kernels vs the fp32 reference, and through the engine."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


def _setup(seed=1, name="test-hybrid"):
    from rexl3_b200.models import hybrid
    cfg = hybrid.CONFIGS[name]
    w = hybrid.random_weights(cfg, seed=seed)
    return cfg, w, hybrid


@pytest.mark.parametrize("name", ["test-hybrid", "test-hybrid-gdn", "test-hybrid-kda"])
def test_chunked_prefill_and_mixed_decode_match_reference(name):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    cfg, w, hybrid = _setup(name=name)
    ref = hybrid.ReferenceHybrid(w, device="cuda")
    m = hybrid.HybridGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    assert m.k_cache[0] is None and m.k_cache[1] is not None
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=100).tolist()
    other = rng.integers(0, cfg.vocab, size=2).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[2, :2] = _i32([5, 9])
    bt[1, :1] = _i32([2])
    slot = lambda s, p: int(bt[s, p // 64]) * 64 + p % 64  # noqa: E731
    want = ref.forward_seq(2, prompt, 0)
    scale = want.abs().max().item()
    # chunk 1: sequence 2 rows 0..69 together with sequence 1's two-token prompt (two segments in one launch)
    c1 = 70
    ids = prompt[:c1] + other
    pos = list(range(c1)) + [0, 1]
    seqs = [2] * c1 + [1] * 2
    pf = dict(seq_ids=_i32([2, 1]), q_start=_i32([0, c1]), q_len=_i32([c1, 2]), pos0=_i32([0, 0]), nseq=2, max_qlen=c1)
    lg = m.forward_rows(_i32(ids), _i32(pos), _i32([slot(s, p) for s, p in zip(seqs, pos)]), _i32(seqs), _i32([p + 1 for p in pos]), bt, prefill=pf,
                        logit_rows=torch.tensor([c1 - 1, c1 + 1], device="cuda"))
    torch.cuda.synchronize()
    m.check()
    w_other = ref.forward_seq(1, other, 0)
    assert (lg[0, :cfg.vocab] - want[c1 - 1]).abs().max().item() < 0.05 * scale
    assert (lg[1, :cfg.vocab] - w_other[1]).abs().max().item() < 0.05 * scale
    # chunk 2: the rest of sequence 2 continues from the pools (conv history and state cross the chunk boundary)
    T = len(prompt)
    pos = list(range(c1, T))
    pf = dict(seq_ids=_i32([2]), q_start=_i32([0]), q_len=_i32([T - c1]), pos0=_i32([c1]), nseq=1, max_qlen=T - c1)
    lg = m.forward_rows(_i32(prompt[c1:]), _i32(pos), _i32([slot(2, p) for p in pos]), _i32([2] * len(pos)), _i32([p + 1 for p in pos]), bt, prefill=pf,
                        logit_rows=torch.tensor([len(pos) - 1, 0], device="cuda"))
    torch.cuda.synchronize()
    m.check()
    assert (lg[0, :cfg.vocab] - want[T - 1]).abs().max().item() < 0.05 * scale
    assert (lg[1, :cfg.vocab] - want[c1]).abs().max().item() < 0.05 * scale
    # decode window: sequence 1 feeds two rows (positions 2, 3), sequence 2 one row, sequence 0 starts at position 0
    t2 = int(want[T - 1].argmax())
    ids, pos, seqs = [11, 12, t2, 7], [2, 3, T, 0], [1, 1, 2, 0]
    bt[0, :1] = _i32([3])
    lg = m.forward_rows(_i32(ids), _i32(pos), _i32([slot(s, p) for s, p in zip(seqs, pos)]), _i32(seqs), _i32([p + 1 for p in pos]), bt, max_ctx=256)
    torch.cuda.synchronize()
    m.check()
    w1 = ref.forward_seq(1, [11, 12], 2)
    w2 = ref.forward_seq(2, [t2], T)
    w0 = ref.forward_seq(0, [7], 0)
    for row, wv in ((0, w1[0]), (1, w1[1]), (2, w2[0]), (3, w0[0])):
        assert (lg[row, :cfg.vocab] - wv).abs().max().item() < 0.05 * scale, row
    # the state pools hold what the reference holds
    conv_ref, s_ref = ref.ssm[(2, 0)]
    assert (m.state_view(0)[2] - s_ref).abs().max().item() < 0.03 * s_ref.abs().max().item()
    assert (m.conv_pool[0][2] - conv_ref).abs().max().item() < 0.03 * conv_ref.abs().max().item()


@pytest.mark.parametrize("name", ["test-hybrid", "test-hybrid-gdn", "test-hybrid-kda"])
def test_engine_greedy_stream_matches_reference_with_graphs(name):
    """Engine over the hybrid backend (graph replay, chunked prefill, two streams): every greedy token is the fp32 reference's best token
    (within the kernels' tolerance) when the reference is fed the engine's own stream."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import HybridGpuBackend
    from rexl3_b200.sampling import GREEDY
    cfg, w, hybrid = _setup(seed=4, name=name)
    ref = hybrid.ReferenceHybrid(w, device="cuda")
    m = hybrid.HybridGPU(w, num_pages=32, max_rows=64, max_seqs=4, max_blocks_per_seq=6, max_prefill_rows=256)
    be = HybridGpuBackend(m, max_slots=4)
    eng = Engine(be, None, window_rows=16, prefill_chunk=48, spec="copy")
    assert eng.can_rollback and eng.prefix is None
    rng = np.random.default_rng(3)
    prompts = {"a": rng.integers(0, cfg.vocab, size=100).tolist(), "b": rng.integers(0, cfg.vocab, size=5).tolist()}
    n_new, exact = 12, 0
    for k, p in prompts.items():
        eng.submit(Request(k, p, n_new, GREEDY))
    got = {k: [] for k in prompts}
    for _ in range(300):
        if not eng.has_work():
            break
        for ev in eng.step():
            assert ev.kind != "error", ev.message
            if ev.kind == "tokens":
                got[ev.id].extend(ev.tokens)
    assert be.graph_replays > 0
    for si, (k, p) in enumerate(prompts.items()):
        assert len(got[k]) == n_new
        lg = ref.forward_seq(si, p, 0)[-1]
        pos = len(p)
        for t in got[k]:
            # teacher-forced on the engine's own token: it must be the reference's best token up to the kernels' numeric tolerance
            assert lg[t].item() >= lg.max().item() - 0.05 * lg.abs().max().item(), (k, pos, t, int(lg.argmax()))
            exact += int(t == int(lg.argmax()))
            lg = ref.forward_seq(si, [t], pos)[0]
            pos += 1
    assert exact >= n_new, "most steps have a clear winner and must agree exactly"


@pytest.fixture(scope="module", params=["test-hybrid", "test-hybrid-gdn", "test-hybrid-kda"])
def make_hybrid_backend(request):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine.gpu_backend import HybridGpuBackend
    cfg, w, hybrid = _setup(seed=6, name=request.param)
    model = hybrid.HybridGPU(w, num_pages=96, max_rows=64, max_seqs=8, max_blocks_per_seq=8, max_prefill_rows=512)

    def make():
        # one model, fresh bookkeeping: KV pages are overwritten and a row at position 0 starts from a zero state whatever the pools hold
        return HybridGpuBackend(model, max_slots=8, state_snapshots=True, verify_snapshots=True)
    make.vocab = cfg.vocab
    return make


@pytest.mark.parametrize("check", ["row_invariance", "serial_batched_equals_solo", "drafted_equals_serial", "chunked_prefill_equals_whole",
                                   "rollback_equals_replay", "cached_equals_cold"])
def test_exactness_on_device_with_record_and_commit(make_hybrid_backend, check):
    """The five exactness checks and cached == cold over the recurrent families: draft rows run in record mode, rejected rows leave no trace
    in the pools, and a prefix hit restores the state snapshot taken where a prefill slice ended."""
    from rexl3_b200.engine import harness
    assert getattr(harness, check)(make_hybrid_backend, make_hybrid_backend.vocab) is None


def test_record_then_commit_leaves_the_pools_as_a_direct_run_does():
    """Model level: a 2-sequence window of 4 rows each in record mode writes nothing; committing (2, 4) rows gives the pools, bit for bit,
    that feeding exactly those rows as final rows gives."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    for name in ("test-hybrid", "test-hybrid-gdn", "test-hybrid-kda"):
        cfg, w, hybrid = _setup(seed=9, name=name)
        m = hybrid.HybridGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
        K = m.K
        m.enable_record(16)
        rng = np.random.default_rng(1)
        bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
        bt[0, 0], bt[1, 0] = 3, 7
        # positions 0..4 of both sequences as final rows, so the pools hold a real state
        def rows(seq_pos):     # noqa: E306
            return (_i32(rng.integers(0, cfg.vocab, size=len(seq_pos)).tolist()), _i32([p for _, p in seq_pos]),
                    _i32([int(bt[s, 0]) * 64 + p for s, p in seq_pos]), _i32([s for s, _ in seq_pos]), _i32([p + 1 for _, p in seq_pos]))
        warm = [(0, p) for p in range(5)] + [(1, p) for p in range(5)]
        m.forward_rows(*rows(warm), bt, want_logits=False)
        before = {li: (m.conv_pool[li].clone(), m.ssm_pool[li].clone()) for li in m.ssm_pool}
        win = [(0, p) for p in range(5, 9)] + [(1, p) for p in range(5, 9)]
        a = rows(win)
        m.ssm_mode = K.SCAN_RECORD
        lg_rec = m.forward_rows(*a, bt).clone()
        m.ssm_mode = K.SCAN_FINAL
        for li in m.ssm_pool:
            assert torch.equal(m.conv_pool[li], before[li][0]) and torch.equal(m.ssm_pool[li], before[li][1]), (name, li)
        m.commit_rows(8, a[3], a[1], _i32([0, 4]), _i32([2, 4]), 2)
        torch.cuda.synchronize()
        m.check()
        got = {li: (m.conv_pool[li].clone(), m.ssm_pool[li].clone()) for li in m.ssm_pool}
        # the same kept rows as final rows from the same starting pools
        for li in m.ssm_pool:
            m.conv_pool[li].copy_(before[li][0])
            m.ssm_pool[li].copy_(before[li][1])
        keep = [0, 1, 4, 5, 6, 7]
        idx = torch.tensor(keep, device="cuda")
        lg_dir = m.forward_rows(*[t[idx].contiguous() for t in a], bt)
        torch.cuda.synchronize()
        m.check()
        assert torch.equal(lg_dir, lg_rec[idx]), name
        for li in m.ssm_pool:
            assert torch.equal(m.conv_pool[li][:2], got[li][0][:2]) and torch.equal(m.ssm_pool[li][:2], got[li][1][:2]), (name, li)
