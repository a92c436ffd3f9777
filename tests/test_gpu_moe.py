"""Mixture-of-experts executor on the GPU against the fp32 reference: router picks, grouped EXL3 GEMM, combine, the whole model."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


def _setup(seed=3, **over):
    import dataclasses
    from rexl3_b200.models import moe
    cfg = dataclasses.replace(moe.CONFIGS["test-moe"], **over)
    w = moe.random_moe_weights(cfg, seed=seed)
    return cfg, w, moe


@pytest.mark.parametrize("mode", ["softmax", "sigmoid_bias"])
def test_router_matches_reference(mode):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import moe
    from rexl3_b200.ops import lib as L
    import dataclasses
    cfg = dataclasses.replace(moe.CONFIGS["test-moe"], n_experts=64, top_k=6, router_mode=mode, routed_scale=2.5 if mode != "softmax" else 1.0)
    g = torch.Generator(device="cuda").manual_seed(0)
    M, d = 37, 256
    x = torch.randn(M, d, device="cuda", generator=g).to(torch.bfloat16)
    gate = (torch.randn(cfg.n_experts, d, device="cuda", generator=g) / 16).to(torch.bfloat16)
    bias = 0.1 * torch.randn(cfg.n_experts, device="cuda", generator=g) if mode != "softmax" else None
    ids = torch.zeros(M, cfg.top_k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(M, cfg.top_k, dtype=torch.float32, device="cuda")
    lib = L.load()
    L.check(lib.rx_moe_router(x.data_ptr(), gate.data_ptr(), L.ptr(bias), M, d, cfg.n_experts, cfg.top_k, 0 if mode == "softmax" else 1,
                              cfg.routed_scale, ids.data_ptr(), wts.data_ptr(), L.stream_ptr()), "router")
    torch.cuda.synchronize()
    ri, rw = moe.route_reference(x.float() @ gate.float().T, cfg, bias)
    assert torch.equal(ids.long(), ri)
    torch.testing.assert_close(wts, rw, rtol=2e-3, atol=1e-5)


@pytest.mark.parametrize("act", ["swiglu", "relu2", "grouped"])
def test_moe_model_matches_reference_prefill_and_decode(act):
    """`relu2`: experts without a gate, down(relu(up)^2), sixteen of them with six picks per token under the sigmoid router."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if act == "swiglu":
        cfg, w, moe = _setup()
    elif act == "grouped":          # group-limited routing in the executor: 16 experts in 4 groups, a token keeps its 2 best groups
        cfg, w, moe = _setup(n_experts=16, top_k=4, router_mode="sigmoid_bias", routed_scale=2.5, n_group=4, topk_group=2)
    else:
        from rexl3_b200.models import moe
        cfg = moe.CONFIGS["test-moe-relu2"]
        w = moe.random_moe_weights(cfg, seed=3)
        assert w.layers[0].experts_gu[0].svh.shape[0] == cfg.expert_ffn
    ref = moe.ReferenceMoE(w, device="cuda")
    # prefill scratch larger than the decode class: the two classes address the sorted-pair buffers with different strides
    m = moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=1024)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=90).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = _i32([3, 7])
    T = len(prompt)
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([T]), pos0=_i32([0]), nseq=1, max_qlen=T)
    args = (_i32(prompt), _i32(pos), _i32(slots), _i32([0] * T), _i32([p + 1 for p in pos]), bt)
    got = m.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
    m.check()
    want = ref.forward_seq(0, prompt, 0)
    scale = want.abs().max().item()
    # a token whose router scores are nearly tied may pick another expert than the fp32 reference: allow a few rows to differ
    err = (got - want).abs().amax(dim=1) / scale
    assert (err < 0.05).float().mean().item() > 0.9, err
    assert err[-1].item() < 0.05
    t0 = int(want[-1].argmax())
    for step in range(3):
        p = T + step
        a2 = (_i32([t0]), _i32([p]), _i32([int(bt[0, p // 64]) * 64 + p % 64]), _i32([0]), _i32([p + 1]), bt)
        g1 = m.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
        m.check()
        w0 = ref.forward_seq(0, [t0], p)[0]
        assert (g1[0] - w0).abs().max().item() < 0.05 * scale
        t0 = int(w0.argmax())


def test_moe_draft_layers_match_reference():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    cfg, w, moe = _setup(seed=5)
    ref = moe.ReferenceMoE(w, device="cuda")
    m = moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    prompt = np.random.default_rng(1).integers(0, cfg.vocab, size=40).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :1] = _i32([2])
    T = len(prompt)
    pos = list(range(T))
    pf = dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([T]), pos0=_i32([0]), nseq=1, max_qlen=T)
    args = (_i32(prompt), _i32(pos), _i32([2 * 64 + p for p in pos]), _i32([0] * T), _i32([p + 1 for p in pos]), bt)
    got = m.forward_rows(*args, prefill=pf, n_layers=cfg.draft_layers, logit_rows=torch.tensor([T - 1], device="cuda"))[:, :cfg.vocab].clone()
    m.check()
    want = ref.forward_seq(0, prompt, 0, n_layers=cfg.draft_layers)[-1]
    assert (got[0] - want).abs().max().item() < 0.05 * want.abs().max().item()


def test_self_speculative_draft_is_exact():
    """Engine over the MoE backend: drafts from the first layers change the schedule, never the tokens."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.sampling import GREEDY
    cfg, w, moe = _setup(seed=9)
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (50, 21)]
    outs = {}
    for mode in ("none", "self"):
        m = moe.MoEGPU(w, num_pages=24, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
        be = DenseGpuBackend(m, max_slots=4, self_draft=(mode == "self"))
        eng = Engine(be, None, window_rows=32, prefill_chunk=256, spec=mode, max_drafts=3)
        for i, p in enumerate(prompts):
            eng.submit(Request(f"r{i}", p, 10, GREEDY))
        got = {f"r{i}": [] for i in range(len(prompts))}
        for _ in range(200):
            if not eng.has_work():
                break
            for ev in eng.step():
                if ev.kind == "tokens":
                    got[ev.id].extend(ev.tokens)
                assert ev.kind != "error", ev.message
        outs[mode] = got
        if mode == "self":
            assert eng.counters["drafted"] > 0 and be.draft_steps > 0
    assert outs["none"] == outs["self"]


@pytest.mark.parametrize("ranks", [2, 4])
def test_expert_parallel_loopback_matches_single(ranks):
    """R expert-parallel ranks stepped phase by phase on one GPU: bit-identical logits on every rank, equal to the one-GPU
    executor up to the order of the expert sum."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.parallel import ep
    cfg, w, moe = _setup(seed=4)
    single = moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    comms = ep.make_loopback(cfg, ranks, 256)
    shards = [moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256,
                         experts=ep.expert_range(cfg.n_experts, r, ranks), ep=comms[r]) for r in range(ranks)]
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, size=70).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = _i32([3, 7])
    T = len(prompt)
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([T]), pos0=_i32([0]), nseq=1, max_qlen=T)
    args = (_i32(prompt), _i32(pos), _i32(slots), _i32([0] * T), _i32([p + 1 for p in pos]), bt)

    def run(a, **kw):
        gens = [s.forward_phases(*a, **kw) for s in shards]
        outs = [None] * ranks
        live = True
        while live:
            for r, g in enumerate(gens):
                try:
                    next(g)
                except StopIteration as e:
                    outs[r] = e.value[:, :cfg.vocab].clone()
                    live = False
        torch.cuda.synchronize()
        for s in shards:
            s.check()
        return outs

    outs = run(args, prefill=pf)
    want = single.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    scale = want.abs().max().item()
    assert (outs[0] - want).abs().max().item() < 0.02 * scale
    p = T
    a2 = (_i32([5]), _i32([p]), _i32([int(bt[0, p // 64]) * 64 + p % 64]), _i32([0]), _i32([p + 1]), bt)
    o2 = run(a2, max_ctx=256)
    w2 = single.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
    assert torch.equal(o2[0], o2[-1]) and (o2[0] - w2).abs().max().item() < 0.02 * scale


@pytest.mark.parametrize("ranks", [2, 4])
def test_token_all_to_all_expert_parallel_equals_single_gpu(ranks):
    """Data-parallel rows with a token all-to-all: every rank feeds its OWN sequence, (row, slot) pairs travel to the rank that owns their expert
    and the results travel home; stepped phase by phase on one GPU.  Each rank's logits equal the one-GPU executor's on that sequence bit for
    bit (same finish, same slot-ordered fma chain), in prefill and in a decode step."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.parallel import ep
    cfg, w, moe = _setup(seed=4)
    single = moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    comms = ep.make_a2a_loopback(cfg, ranks, 256)
    shards = [moe.MoEGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256,
                         experts=ep.expert_range(cfg.n_experts, r, ranks), a2a=comms[r]) for r in range(ranks)]
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (70, 45, 9, 130)[:ranks]]
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :3] = _i32([3, 7, 5])

    def rows_of(tokens, p0):
        pos = list(range(p0, p0 + len(tokens)))
        return (_i32(tokens), _i32(pos), _i32([int(bt[0, p // 64]) * 64 + p % 64 for p in pos]), _i32([0] * len(pos)), _i32([p + 1 for p in pos]), bt)

    def run(per_rank):
        gens = [s.forward_phases(*a, **kw) for s, (a, kw) in zip(shards, per_rank)]
        outs, live = [None] * ranks, ranks
        while live:
            for r, g in enumerate(gens):
                if outs[r] is not None:
                    continue
                try:
                    next(g)
                except StopIteration as e:
                    outs[r] = e.value[:, :cfg.vocab].clone()
                    live -= 1
        torch.cuda.synchronize()
        for s in shards:
            s.check()
        return outs

    pf = lambda n: dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([n]), pos0=_i32([0]), nseq=1, max_qlen=n)  # noqa: E731
    outs = run([(rows_of(p, 0), dict(prefill=pf(len(p)))) for p in prompts])
    for r, p in enumerate(prompts):
        want = single.forward_rows(*rows_of(p, 0), prefill=pf(len(p)))[:, :cfg.vocab].clone()
        assert torch.equal(outs[r], want), r
    outs = run([(rows_of([5 + r], len(p)), dict(max_ctx=256)) for r, p in enumerate(prompts)])
    for r, p in enumerate(prompts):
        single.forward_rows(*rows_of(p, 0), prefill=pf(len(p)))
        want = single.forward_rows(*rows_of([5 + r], len(p)), max_ctx=256)[:, :cfg.vocab].clone()
        assert torch.equal(outs[r], want), r


@pytest.mark.parametrize("rows,tile_rows", [(5, 16), (70, 32)])
def test_mxfp4_grouped_gemm_matches_dequantized_reference(rows, tile_rows):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.format import mxfp4
    from rexl3_b200.ops import kernels as K
    from rexl3_b200.ops import lib as L
    lib = L.load()
    rng = np.random.default_rng(1)
    E, N, Kd, topk = 6, 256, 384, 2
    wq, sc, wf = [], [], []
    for e in range(E):
        w = rng.normal(0, 0.05 * (1 + e), size=(N, Kd)).astype(np.float32)
        q, s = mxfp4.quantize(w)
        wq.append(q.view(np.uint8)); sc.append(s); wf.append(mxfp4.dequant(q, s))
    d_w = torch.from_numpy(np.stack(wq)).cuda()
    d_s = torch.from_numpy(np.stack(sc)).cuda()
    ids = torch.from_numpy(rng.integers(0, E, size=(rows, topk)).astype(np.int32)).cuda()
    pairs = rows * topk
    i32 = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")  # noqa: E731
    offs, pos_of_pair, pair_of_pos, expert_of_pos, total = i32(E + 1), i32(pairs), i32(pairs), i32(pairs), i32(1)
    max_tiles = E + (pairs + tile_rows - 1) // tile_rows
    tile_tab = i32(3 * max_tiles)
    L.check(lib.rx_moe_plan(ids.data_ptr(), pairs, E, 0, E, tile_rows, max_tiles, offs.data_ptr(), pos_of_pair.data_ptr(), pair_of_pos.data_ptr(),
                            expert_of_pos.data_ptr(), tile_tab.data_ptr(), total.data_ptr(), L.stream_ptr()), "plan")
    x = torch.from_numpy(rng.normal(0, 1, size=(rows, Kd)).astype(np.float32)).cuda().to(torch.bfloat16)
    xs = torch.zeros(pairs, Kd, dtype=torch.float16, device="cuda")
    L.check(lib.rx_moe_gather_rot(x.data_ptr(), ids.data_ptr(), pos_of_pair.data_ptr(), pairs, topk, Kd, None, xs.data_ptr(), L.stream_ptr()), "gather")
    splits = 2
    part = torch.zeros(splits, pairs, N, dtype=torch.float32, device="cuda")
    status = K.new_status()
    L.check(lib.rx_mxfp4_gemm_grouped(xs.data_ptr(), pairs, Kd, d_w.data_ptr(), d_s.data_ptr(), E, N, part.data_ptr(), splits, tile_tab.data_ptr(),
                                      max_tiles, tile_rows, status.data_ptr(), L.stream_ptr()), "mxfp4")
    torch.cuda.synchronize()
    K.check_status(status, "mxfp4")
    got = part.sum(0).cpu().numpy()
    pos = pos_of_pair.cpu().numpy()
    xh = xs.float().cpu().numpy()
    idn = ids.cpu().numpy().reshape(-1)
    for p in range(pairs):
        want = xh[pos[p]] @ wf[idn[p]].T
        np.testing.assert_allclose(got[pos[p]], want, rtol=2e-2, atol=2e-2 * np.abs(want).max())


@pytest.mark.parametrize("n_group,topk_group", [(8, 3), (4, 1), (16, 16)])
def test_group_limited_router_matches_reference(n_group, topk_group):
    """Sigmoid + bias scores, the `topk_group` best of `n_group` expert groups (group score = its two best keys), then top-k inside them."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dataclasses
    from rexl3_b200.models import moe
    from rexl3_b200.ops import lib as L
    lib = L.load()
    cfg = dataclasses.replace(moe.CONFIGS["test-moe"], n_experts=64, top_k=6, router_mode="sigmoid_bias", routed_scale=2.5)
    M, d, E, k = 37, cfg.d_model, cfg.n_experts, cfg.top_k
    g = torch.Generator(device="cuda").manual_seed(n_group)
    x = torch.randn(M, d, device="cuda", generator=g).to(torch.bfloat16)
    gate = (torch.randn(E, d, device="cuda", generator=g) / 16).to(torch.bfloat16)
    bias = 0.1 * torch.randn(E, device="cuda", generator=g)
    ids = torch.zeros(M, k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(M, k, dtype=torch.float32, device="cuda")
    logits = torch.empty(M, E, dtype=torch.float32, device="cuda")
    L.check(lib.rx_moe_router_grouped(x.data_ptr(), gate.data_ptr(), bias.data_ptr(), M, d, E, k, 1, cfg.routed_scale, n_group, topk_group, logits.data_ptr(),
                                      ids.data_ptr(), wts.data_ptr(), L.stream_ptr()), "router")
    torch.cuda.synchronize()
    want_ids, want_w = moe.route_reference(logits, cfg, bias, n_group, topk_group)      # the device's own logits: the selection is then exact
    assert torch.equal(ids.long(), want_ids)
    assert torch.allclose(wts, want_w, rtol=1e-4, atol=1e-6)
    per = E // n_group
    assert all(len({int(e) // per for e in row}) <= topk_group for row in ids.tolist())
