"""End-to-end dense decoder on the sm_100a kernels vs the fp32 PyTorch reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("name", ["test-hd128", "tiny-llama"])
def test_prefill_and_decode_logits_match_reference(name):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS[name]
    w = dense.random_weights(cfg, seed=1)
    ref = dense.ReferenceDense(w, device="cuda")
    m = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=100).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = _i32([5, 9])
    bt[1, :1] = _i32([2])
    T = len(prompt)
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([T]), pos0=_i32([0]), nseq=1, max_qlen=T)
    logits = m.forward_rows(_i32(prompt), _i32(pos), _i32(slots), _i32([0] * T), _i32([p + 1 for p in pos]), bt, prefill=pf,
                            logit_rows=torch.tensor([T - 1, 10], device="cuda"))
    torch.cuda.synchronize()
    m.check()
    want = ref.forward_seq(0, prompt, 0)
    scale = want.abs().max().item()
    got = logits[:, :cfg.vocab]
    assert (got[0] - want[T - 1]).abs().max().item() < 0.05 * scale
    assert (got[1] - want[10]).abs().max().item() < 0.05 * scale
    assert got[0].argmax().item() == want[T - 1].argmax().item() or (want[T - 1].topk(2).values.diff().abs().item() < 0.02 * scale)
    # decode: two sequences in one window (seq 0 continues, seq 1 starts with a single token at position 0)
    t0, t1 = int(want[T - 1].argmax()), 7
    ids, pos2, seqs = [t0, t1], [T, 0], [0, 1]
    slots2 = [int(bt[0, T // 64]) * 64 + T % 64, int(bt[1, 0]) * 64]
    logits = m.forward_rows(_i32(ids), _i32(pos2), _i32(slots2), _i32(seqs), _i32([T + 1, 1]), bt, max_ctx=256)
    torch.cuda.synchronize()
    m.check()
    w0 = ref.forward_seq(0, [t0], T)[0]
    w1 = ref.forward_seq(1, [t1], 0)[0]
    assert (logits[0, :cfg.vocab] - w0).abs().max().item() < 0.05 * scale
    assert (logits[1, :cfg.vocab] - w1).abs().max().item() < 0.05 * scale
    # candidates: exact order of the device top-k
    ids_c, vals_c = m.candidates(logits, 8)
    v, i = torch.sort(logits[:, :cfg.vocab], dim=1, descending=True, stable=True)
    assert torch.equal(ids_c.long(), i[:, :8]) and torch.equal(vals_c, v[:, :8])


def test_fp8_kv_cache_close_to_bf16_cache():
    """E4M3 KV with calibrated per-head scales: prefill + decode logits stay close to the bf16-cache executor."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.models import dense
    for name in ("test-hd128", "tiny-llama"):
        cfg = dense.CONFIGS[name]
        w = dense.random_weights(cfg, seed=3)
        a = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
        b = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256, kv_dtype="fp8")
        rng = np.random.default_rng(0)
        b.calibrate_kv(rng.integers(0, cfg.vocab, size=128).tolist())
        assert float(b.kv_scale.min()) > 0 and not torch.equal(b.kv_scale, torch.ones_like(b.kv_scale))
        prompt = rng.integers(0, cfg.vocab, size=150).tolist()
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
        bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
        bt[1, :3] = i32([5, 9, 2])
        T = len(prompt)
        pos = list(range(T))
        slots = [int(bt[1, p // 64]) * 64 + p % 64 for p in pos]
        pf = dict(seq_ids=i32([1]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
        args = (i32(prompt), i32(pos), i32(slots), i32([1] * T), i32([p + 1 for p in pos]), bt)
        la = a.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
        lb = b.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
        a.check(); b.check()
        scale = la.abs().max().item()
        assert (la - lb).abs().max().item() < 0.06 * scale
        p = T
        a2 = (i32([7]), i32([p]), i32([int(bt[1, p // 64]) * 64 + p % 64]), i32([1]), i32([p + 1]), bt)
        da = a.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
        db = b.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
        a.check(); b.check()
        assert (da - db).abs().max().item() < 0.06 * scale


def test_int8_kv_cache_with_token_scales_close_to_bf16_cache_and_through_the_engine():
    """int8 KV with one power-of-two scale per (token, KV head): the stored bytes and scales reproduce the bf16 cache within the quantisation step,
    prefill (mma.sync byte-page kernel) and decode windows stay close to the bf16-cache executor, and the engine's exactness checks that touch the
    cache (drafted == serial, cached == cold with the spill payload) hold on it."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.engine import harness
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    for name in ("test-hd128", "tiny-llama"):
        cfg = dense.CONFIGS[name]
        w = dense.random_weights(cfg, seed=3)
        a = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
        b = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256, kv_dtype="int8")
        rng = np.random.default_rng(0)
        prompt = rng.integers(0, cfg.vocab, size=150).tolist()
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
        bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
        bt[1, :3] = i32([5, 9, 2])
        T = len(prompt)
        pos = list(range(T))
        slots = [int(bt[1, p // 64]) * 64 + p % 64 for p in pos]
        pf = dict(seq_ids=i32([1]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
        args = (i32(prompt), i32(pos), i32(slots), i32([1] * T), i32([p + 1 for p in pos]), bt)
        la = a.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
        lb = b.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
        a.check(); b.check()
        # layer 0 sees the same inputs in both executors: its int8 page times its scales is the bf16 page up to half a step
        k16 = a.k_cache[0][5].float()
        k8 = b.k_cache[0][5].float() * b.k_tscale[0][5][..., None]
        step = b.k_tscale[0][5][..., None]
        assert ((k16 - k8).abs() <= 0.5 * step + 0.01 * k16.abs() + 1e-6).all()
        sc = b.k_tscale[0][5]
        assert torch.equal(sc, torch.exp2(torch.round(torch.log2(sc)))) and float(b.k_cache[0][5].abs().max()) <= 127
        scale = la.abs().max().item()
        assert (la - lb).abs().max().item() < 0.05 * scale
        p = T
        a2 = (i32([7]), i32([p]), i32([int(bt[1, p // 64]) * 64 + p % 64]), i32([1]), i32([p + 1]), bt)
        da = a.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
        db = b.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
        a.check(); b.check()
        assert (da - db).abs().max().item() < 0.05 * scale
    cfg = dense.CONFIGS["test-hd128"]
    model = dense.DenseGPU(dense.random_weights(cfg, seed=3), num_pages=96, max_rows=64, max_seqs=8, max_blocks_per_seq=8, max_prefill_rows=512, kv_dtype="int8")
    make = lambda: DenseGpuBackend(model, max_slots=8)  # noqa: E731
    for check in ("drafted_equals_serial", "rollback_equals_replay", "cached_equals_cold", "row_invariance"):
        assert getattr(harness, check)(make, cfg.vocab) is None, check
    be = make()
    from rexl3_b200.engine import Engine, generate
    from rexl3_b200.sampling import GREEDY
    generate(Engine(be, spec="none"), [list(range(1, 130))], 2, GREEDY)
    handle = ("page", 3)
    blob = be.prefix_export(handle)
    assert len(blob) == 2 * cfg.n_layers * (cfg.n_kv * 64 * cfg.head_dim + cfg.n_kv * 64 * 4)
    got = be.prefix_import(blob)
    assert got is not None


def test_per_linear_rotations_serve_and_match_the_reference(tmp_path):
    """A pack quantised one linear at a time (q / k / v and gate / up each with its own input rotation) is written, loaded and served
    through one GEMM per part; prefill and decode logits match the fp32 reference of the same weights, and the engine generates."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine import Engine, generate
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.models import dense
    from rexl3_b200.quant import quantize
    from rexl3_b200.sampling import GREEDY
    cfg = dense.CONFIGS["test-hd128"]
    quantize.write_pack(str(tmp_path / "p"), dense.random_weights(cfg, seed=4, per_linear=True))
    w = quantize.load_pack(str(tmp_path / "p"))
    assert isinstance(w.layers[0].qkv, dense.HostSplitLinear)
    ref = dense.ReferenceDense(w, device="cuda")
    m = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=90).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = _i32([3, 7])
    T = len(prompt)
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=_i32([0]), q_start=_i32([0]), q_len=_i32([T]), pos0=_i32([0]), nseq=1, max_qlen=T)
    logits = m.forward_rows(_i32(prompt), _i32(pos), _i32(slots), _i32([0] * T), _i32([p + 1 for p in pos]), bt, prefill=pf,
                            logit_rows=torch.tensor([T - 1], device="cuda"))
    m.check()
    want = ref.forward_seq(0, prompt, 0)
    scale = want.abs().max().item()
    assert (logits[0, :cfg.vocab] - want[T - 1]).abs().max().item() < 0.05 * scale
    t0 = int(want[T - 1].argmax())
    logits = m.forward_rows(_i32([t0]), _i32([T]), _i32([int(bt[0, T // 64]) * 64 + T % 64]), _i32([0]), _i32([T + 1]), bt, max_ctx=256)
    m.check()
    assert (logits[0, :cfg.vocab] - ref.forward_seq(0, [t0], T)[0]).abs().max().item() < 0.05 * scale
    # through the engine, with CUDA graphs (the per-part launches and the placement copies are captured like any other window)
    m2 = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    out = generate(Engine(DenseGpuBackend(m2, max_slots=4), None, spec="none"), [prompt[:20], prompt[20:50]], 8, GREEDY)
    assert all(len(o) == 8 for o in out)


def test_moe_and_mla_models_load_from_their_packs(tmp_path):
    """The MoE GQA decoder (EXL3 experts) and the MLA + MoE decoder (MXFP4 routed experts) written as packs, probed by the registry,
    loaded and run on the device: the same logits as the executor built from the in-memory weights."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import mla, moe, registry
    from rexl3_b200.quant import packs
    i32 = _i32
    bt = torch.zeros(2, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = i32([1, 2])
    T = 40
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
    for kind, cfg, mk, write, cls in (("moe", moe.CONFIGS["test-moe"], moe.random_moe_weights, packs.write_moe_pack, moe.MoEGPU),
                                      ("mla_moe", mla.CONFIGS["test-mla"], mla.random_mla_weights, packs.write_mla_pack, mla.MlaMoEGPU)):
        w = mk(cfg, seed=6)
        write(str(tmp_path / kind), w)
        fam, plan = registry.probe(str(tmp_path / kind))
        assert fam.id == kind
        w2 = packs.load_any(str(tmp_path / kind))
        toks = np.random.default_rng(1).integers(0, cfg.vocab, size=T).tolist()
        outs = []
        for ww in (w, w2):
            m = cls(ww, num_pages=8, max_rows=64, max_seqs=2, max_blocks_per_seq=4, max_prefill_rows=128)
            lg = m.forward_rows(i32(toks), i32(pos), i32(slots), i32([0] * T), i32([p + 1 for p in pos]), bt, prefill=pf,
                                logit_rows=torch.tensor([T - 1], device="cuda"))
            torch.cuda.synchronize()
            outs.append(lg[0, :cfg.vocab].clone())
        assert torch.equal(outs[0], outs[1]), kind


def _mtp_setup(seed=5):
    import dataclasses
    from rexl3_b200.models import dense
    cfg = dataclasses.replace(dense.CONFIGS["test-hd128"], mtp=True, name="test-hd128-mtp")
    return cfg, dense.random_weights(cfg, seed=seed), dense


def test_mtp_block_matches_reference():
    """The multi-token-prediction block (hidden of position i + token i + 1 -> logits of token i + 2) against the fp32 oracle: a prefill slice
    of lagged rows, then chained draft rows on the block's own output."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    cfg, w, dense = _mtp_setup()
    ref = dense.ReferenceDense(w, device="cuda")
    m = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    rng = np.random.default_rng(3)
    prompt = rng.integers(0, cfg.vocab, size=90).tolist()
    T = len(prompt)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :3] = i32([3, 7, 5])
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
    m.forward_rows(i32(prompt), i32(pos), i32(slots), i32([0] * T), i32([p + 1 for p in pos]), bt, prefill=pf)
    hid = m.h[:T].clone()
    ref.forward_seq(0, prompt, 0)
    assert (hid.float() - ref.last_hidden).abs().max().item() < 0.05 * ref.last_hidden.abs().max().item()
    # lagged rows 0 .. T-2 (token i + 1 known), as a prefill slice of the block
    n = T - 1
    pf2 = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([n]), pos0=i32([0]), nseq=1, max_qlen=n)
    logits, hm = m.mtp_forward(i32(prompt[1:]), hid[:n].contiguous(), i32(pos[:n]), i32(slots[:n]), i32([0] * n), i32([p + 1 for p in pos[:n]]), bt, prefill=pf2,
                               logit_rows=torch.tensor([n - 1], device="cuda"))
    got, hm = logits[0, :cfg.vocab].clone(), hm.clone()
    m.check()
    want, want_h = ref.mtp_seq(0, prompt[1:], ref.last_hidden[:n], 0)
    scale = want.abs().max().item()
    assert (got - want[-1]).abs().max().item() < 0.05 * scale
    assert (hm.float() - want_h).abs().max().item() < 0.05 * want_h.abs().max().item()
    # row T-1 with a sampled token, then two chained rows on the block's own hidden (decode class, one row each)
    tok, h_in, h_ref = 17, hid[T - 1:T].contiguous(), ref.last_hidden[T - 1:T]
    for j in range(3):
        p = T - 1 + j
        lg, ho = m.mtp_forward(i32([tok]), h_in, i32([p]), i32([int(bt[0, p // 64]) * 64 + p % 64]), i32([0]), i32([p + 1]), bt, max_ctx=256)
        lg, h_in = lg[0, :cfg.vocab].clone(), ho.clone()
        m.check()
        wl, h_ref = ref.mtp_seq(0, [tok], h_ref, p)
        assert (lg - wl[0]).abs().max().item() < 0.06 * scale, j
        tok = int(wl[0].argmax())


def test_mtp_drafts_change_the_schedule_never_the_tokens():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.sampling import GREEDY
    cfg, w, dense = _mtp_setup(seed=6)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (70, 21, 130)]
    outs = {}
    for mode in ("none", "mtp"):
        m = dense.DenseGPU(w, num_pages=32, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=64)
        be = DenseGpuBackend(m, max_slots=4, mtp_draft=(mode == "mtp"))
        eng = Engine(be, None, window_rows=32, prefill_chunk=64, spec=mode, max_drafts=3)
        for i, p in enumerate(prompts):
            eng.submit(Request(f"r{i}", p, 12, GREEDY))
        got = {f"r{i}": [] for i in range(len(prompts))}
        for _ in range(300):
            if not eng.has_work():
                break
            for ev in eng.step():
                if ev.kind == "tokens":
                    got[ev.id].extend(ev.tokens)
                assert ev.kind != "error", ev.message
        outs[mode] = got
        if mode == "mtp":
            st = be.stats()
            assert eng.counters["drafted"] > 0 and st["draft_steps"] > 0 and st["mtp_rows"] > 0
    assert outs["none"] == outs["mtp"]


def test_guard_bands_stay_intact_through_prefill_and_decode(monkeypatch):
    """REXL3_CANARY=1: every scratch buffer of the executor sits between guard bands; a prefill slice and decode windows leave them untouched."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    monkeypatch.setenv("REXL3_CANARY", "1")
    from rexl3_b200.models import dense
    from rexl3_b200.utils import canary
    canary.forget()
    cfg = dense.CONFIGS["test-hd128"]
    m = dense.DenseGPU(dense.random_weights(cfg, seed=1), num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=128)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :3] = i32([3, 7, 5])
    T = 128
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
    m.forward_rows(i32([5] * T), i32(pos), i32(slots), i32([0] * T), i32([p + 1 for p in pos]), bt, prefill=pf, logit_rows=torch.tensor([T - 1], device="cuda"))
    for p in range(T, T + 3):
        m.forward_rows(i32([9]), i32([p]), i32([int(bt[0, p // 64]) * 64 + p % 64]), i32([0]), i32([p + 1]), bt, max_ctx=256)
    torch.cuda.synchronize()
    m.check()
    assert canary.check_all() >= 7
    canary.forget()


def test_q4_kv_cache_rows_and_attention():
    """q4 KV (E2M1 nibbles, one E8M0 scale per 32 values): the stored rows dequantise to the bf16 cache within half a code step, and prefill and
    decode windows over them stay close to the bf16-cache executor (a 4-bit cache is lossy: the bound is loose, the row check is tight)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import numpy as np
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["test-hd128"]
    w = dense.random_weights(cfg, seed=3)
    a = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256)
    b = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256, kv_dtype="q4")
    assert b.k_cache[0].shape[-1] == 64 and b.k_tscale[0].shape[-1] == 4
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=150).tolist()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[1, :3] = i32([5, 9, 2])
    T = len(prompt)
    pos = list(range(T))
    slots = [int(bt[1, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=i32([1]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
    args = (i32(prompt), i32(pos), i32(slots), i32([1] * T), i32([p + 1 for p in pos]), bt)
    la = a.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
    lb = b.forward_rows(*args, prefill=pf)[:, :cfg.vocab].clone()
    a.check()
    b.check()
    # layer 0 sees the same inputs in both executors: dequantise its q4 page on the host
    mags = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], device="cuda")
    for cache16, cache4, sc4 in ((a.k_cache[0][5], b.k_cache[0][5], b.k_tscale[0][5]), (a.v_cache[0][5], b.v_cache[0][5], b.v_tscale[0][5])):
        by = cache4.long()                                              # [n_kv, 64, 64] bytes
        nib = torch.stack([by & 15, by >> 4], dim=-1).reshape(*by.shape[:-1], 128)
        val = mags[nib & 7] * torch.where((nib & 8) != 0, -1.0, 1.0)
        scale = torch.exp2(sc4.float() - 127.0).repeat_interleave(32, dim=-1)
        deq = val * scale
        x = cache16.float()
        amax = x.view(*x.shape[:-1], 4, 32).abs().amax(-1)
        want_scale = torch.exp2(torch.ceil(torch.log2(amax.clamp_min(1e-4) / 6.0)).clamp(-14, 12))
        got_scale = torch.exp2(sc4.float() - 127.0)          # (the device takes the group maximum before the bf16 rounding of the other executor's cache)
        assert (got_scale == want_scale).float().mean().item() > 0.97 and ((got_scale / want_scale - 1).abs() <= 1.0).all()
        # nearest E2M1 code: the error is at most half the local code spacing (2 at the top of the range) times the scale
        assert ((x - deq).abs() <= 0.5 * scale * torch.where(x.abs() / scale >= 4, 2.0, torch.where(x.abs() / scale >= 2, 1.0, 0.5)) + 0.01 * x.abs() + 1e-6).all()
    scale_l = la.abs().max().item()
    assert (la - lb).abs().max().item() < 0.25 * scale_l and (la - lb).abs().mean().item() < 0.05 * scale_l
    p = T
    a2 = (i32([7]), i32([p]), i32([int(bt[1, p // 64]) * 64 + p % 64]), i32([1]), i32([p + 1]), bt)
    da = a.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
    db = b.forward_rows(*a2, max_ctx=256)[:, :cfg.vocab].clone()
    b.check()
    assert (da - db).abs().max().item() < 0.25 * scale_l
    # decode over the q4 cache == prefill over the q4 cache for the same row (both expand the same bytes)
    c = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=256, kv_dtype="q4")
    pf1 = dict(seq_ids=i32([1]), q_start=i32([0]), q_len=i32([T + 1]), pos0=i32([0]), nseq=1, max_qlen=T + 1)
    pos1 = list(range(T + 1))
    slots1 = [int(bt[1, q // 64]) * 64 + q % 64 for q in pos1]
    lc = c.forward_rows(i32(prompt + [7]), i32(pos1), i32(slots1), i32([1] * (T + 1)), i32([q + 1 for q in pos1]), bt, prefill=pf1)[:, :cfg.vocab].clone()
    assert (lc[-1] - db[0]).abs().max().item() < 0.02 * scale_l
