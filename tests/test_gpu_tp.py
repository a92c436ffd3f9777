"""Tensor-parallel dense decoder: R shards stepped phase by phase on ONE GPU (loopback group) against the single-GPU
executor and the fp32 reference.  Every peer wait is already satisfied when its kernel runs, so nothing spins."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("ranks", [2, 4])
def test_tp_loopback_matches_single_gpu_and_reference(ranks):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dataclasses
    from rexl3_b200.models import dense, dense_tp
    from rexl3_b200.parallel.symm import LoopbackGroup
    cfg = dataclasses.replace(dense.CONFIGS["test-hd128"], n_kv=4, name="tp-test")     # 8 q / 4 kv heads: splits over 2 and 4 ranks
    w = dense.random_weights(cfg, seed=5)
    ref = dense.ReferenceDense(w, device="cuda")
    single = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    layout = dense_tp.DenseTPShard.layout(cfg, ranks, 256)
    g = LoopbackGroup(layout)
    shards = [dense_tp.DenseTPShard(cfg, g, r, 16, 256, 4, 4, dense_tp.shard_weights(w, r, ranks)) for r in range(ranks)]
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=100).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = _i32([5, 9])
    T = len(prompt)
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([T]), pos0=_i32([0]), nseq=1, max_qlen=T)
    args = (_i32(prompt), _i32(pos), _i32(slots), _i32([0] * T), _i32([p + 1 for p in pos]), bt)
    lr = torch.tensor([T - 1], device="cuda")

    def run_tp(a, **kw):
        gens = [s.phases(*a, **kw) for s in shards]
        outs = [None] * ranks
        for fns in zip(*gens):
            for r, fn in enumerate(fns):
                outs[r] = fn()
        torch.cuda.synchronize()
        for s in shards:
            K = s.status.tolist()
            assert K[0] == 0, K
        if "cand_count" in kw:        # the last phase returned the merged candidates on the leader; logits are kept per shard
            full = torch.cat([s.last_logits for s in shards], dim=1)[:, :cfg.vocab]
            ids, vals = outs[0]
            tv, ti = torch.sort(full, dim=1, descending=True, stable=True)
            n = kw["cand_count"]
            assert torch.equal(vals, tv[:, :n]) and torch.equal(ids.long(), ti[:, :n])
            return full
        return torch.cat([o[:, :] for o in outs], dim=1)[:, :cfg.vocab]

    got = run_tp(args, prefill=pf, logit_rows=lr)
    want1 = single.forward_rows(*args, prefill=pf, logit_rows=lr)[:, :cfg.vocab].clone()
    want = ref.forward_seq(0, prompt, 0)[T - 1]
    scale = want.abs().max().item()
    assert (got[0] - want).abs().max().item() < 0.05 * scale
    assert (got[0] - want1[0]).abs().max().item() < 0.03 * scale
    # decode step (one row), twice: tickets advance with the epoch
    t0 = int(want.argmax())
    for step in range(2):
        p = T + step
        a2 = (_i32([t0]), _i32([p]), _i32([int(bt[0, p // 64]) * 64 + p % 64]), _i32([0]), _i32([p + 1]), bt)
        got = run_tp(a2, max_ctx=256, cand_count=8 if step == 0 else 64)
        w0 = ref.forward_seq(0, [t0], p)[0]
        assert (got[0] - w0).abs().max().item() < 0.05 * scale
        t0 = int(w0.argmax())


def test_a_peer_wait_that_runs_out_returns_a_status_and_the_context_stays_usable():
    """The wait for a flag nobody publishes, with a 5 ms limit set by the host: the kernel returns by itself, the status words name the
    site and say ST_PEER_TIMEOUT, the next kernel on the same context runs normally, and the backend turns the words into a fatal
    `group_lost` error.  Then the same with the abort word instead of a short limit.  Nothing traps, nothing hangs, no rank dies."""
    import ctypes
    import time
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.ops import kernels as K
    from rexl3_b200.ops import lib as _lib
    L = _lib.load()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")          # the peers' flag words: never written
    epoch = torch.ones(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    status = K.new_status()
    K.set_wait_limit(status, 5000)
    t0 = time.time()
    _lib.check(L.rx_tp_wait_flags(flags.data_ptr(), 2, epoch.data_ptr(), 1, status.data_ptr(), st), "rx_tp_wait_flags")
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.5
    s = status.tolist()
    assert s[0] == K.ST_PEER_TIMEOUT and s[1] == 180
    with pytest.raises(_lib.KernelError, match="peer timed out"):
        K.check_status(status)
    assert int((torch.arange(10, device="cuda") * 2).sum()) == 90       # the context is alive
    # abort word: a wait with the default (2 s) limit gives up at once
    status = K.new_status()
    K.set_abort(status)
    t0 = time.time()
    _lib.check(L.rx_tp_wait_flags(flags.data_ptr(), 2, epoch.data_ptr(), 1, status.data_ptr(), st), "rx_tp_wait_flags")
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0 and status.tolist()[0] == K.ST_ABORTED
    # the backend's view of the same words
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend

    class _M:          # the two attributes _check touches
        pass
    be = DenseGpuBackend.__new__(DenseGpuBackend)
    be.m = _M()
    be.m.status = K.new_status()
    be.h_status = torch.tensor([K.ST_PEER_TIMEOUT, 180, 0, 1, 0, 0, 0, 0], dtype=torch.int32)
    be._err = None
    be._check()
    err = be.take_error()
    assert err is not None and err.fatal and err.group_lost
