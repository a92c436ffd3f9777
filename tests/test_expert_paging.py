"""Routed experts paged from a record file: the file's layout on the CPU, and on the device a paged executor that returns the resident
executor's bits while its slab holds fewer experts than the model has."""
import numpy as np
import pytest
import torch

from rexl3_b200.models import expert_paging as xp
from rexl3_b200.models import moe
from rexl3_b200.sched import expert_cache as ec


def test_record_file_holds_every_expert_part_aligned(tmp_path):
    cfg = moe.CONFIGS["test-moe"]
    w = moe.random_moe_weights(cfg, seed=1)
    lay = xp.write_records(w, str(tmp_path / "experts.bin"))
    assert lay.n_layers == cfg.n_layers and lay.n_experts == cfg.n_experts and len(lay.index) == cfg.n_layers * cfg.n_experts
    assert all(off % ec.PART_ALIGN == 0 for _, off, _, _, _ in lay.parts) and [p[0] for p in lay.parts] == list(xp.PARTS)
    raw = open(lay.path, "rb").read()
    rec = (lay.expert_bytes + ec.PAGE - 1) // ec.PAGE * ec.PAGE
    assert len(raw) == rec * len(lay.index)
    off, n = lay.index[(2, 5)]
    assert off % ec.PAGE == 0 and n == lay.expert_bytes
    gu, dn = w.layers[2].experts_gu[5], w.layers[2].experts_down[5]
    for (name, o, nb, shape, dt), want in zip(lay.parts, xp._parts_of(gu, dn)):
        got = np.frombuffer(raw[off + o:off + o + nb], dtype=dt).reshape(shape)
        assert np.array_equal(got, want), name
    # an existing file of the right size is kept (same index), a wrong one is rewritten
    again = xp.write_records(w, lay.path)
    assert again.index == lay.index
    open(lay.path, "ab").write(b"x")
    assert xp.write_records(w, lay.path).index == lay.index and len(open(lay.path, "rb").read()) == len(raw)


@pytest.mark.gpu
def test_paged_executor_returns_the_resident_bits_and_evicts(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine import Engine, generate
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.sampling import GREEDY
    cfg = moe.CONFIGS["test-moe"]
    w = moe.random_moe_weights(cfg, seed=1)
    kw = dict(num_pages=32, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=128)
    resident = moe.MoEGPU(w, **kw)
    lay = xp.write_records(w, str(tmp_path / "experts.bin"))
    rec = (lay.expert_bytes + ec.PAGE - 1) // ec.PAGE * ec.PAGE
    # the slab holds 10 records: more than one layer's 8 experts, fewer than the model's 24
    paged = moe.MoEGPU(w, expert_paging=dict(path=lay.path, budget_bytes=10 * rec + 100), **kw)
    assert paged.paged.slots == 10 and paged.weight_bytes() < resident.weight_bytes()
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, cfg.vocab, size=n).tolist() for n in (5, 40, 70)]
    a = generate(Engine(DenseGpuBackend(resident, max_slots=4), spec="none"), prompts, 12, GREEDY)
    be = DenseGpuBackend(paged, max_slots=4)
    assert not be.use_graphs
    b = generate(Engine(be, spec="none"), prompts, 12, GREEDY)
    assert a == b
    # logits of one window, bit for bit
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    toks = prompts[1]
    n = len(toks)
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, 0] = 3
    args = (i32(toks), i32(list(range(n))), i32([3 * 64 + p for p in range(n)]), i32([0] * n), i32([p + 1 for p in range(n)]), bt)
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([n]), pos0=i32([0]), nseq=1, max_qlen=n)
    la = resident.forward_rows(*args, prefill=pf).clone()
    lb = paged.forward_rows(*args, prefill=pf).clone()
    assert torch.equal(la, lb)
    st = be.stats()
    assert st["expert_slots"] == 10 and st["expert_evictions"] > 0 and st["expert_cold"] > 0 and st["expert_bytes_read"] >= st["expert_cold"] * lay.expert_bytes * 0
    assert 0 < st["expert_cold_rate"] < 1
    paged.paged.close()


@pytest.mark.gpu
def test_paged_mxfp4_experts_under_the_latent_attention_executor(tmp_path):
    """The MXFP4 experts of the MLA + MoE executor from a record file: a slab of 9 records for 2 routed layers x 8 experts, bits equal to
    the resident executor's over a prefill and three decode steps."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import mla
    cfg = mla.CONFIGS["test-mla"]
    w = mla.random_mla_weights(cfg, seed=2)
    lay = xp.write_mx_records(w, str(tmp_path / "mx.bin"))
    assert lay.n_layers == cfg.n_layers - cfg.n_dense and [p[0] for p in lay.parts] == list(xp.MX_PARTS) and (0, 0) not in lay.index and (1, 7) in lay.index
    rec = (lay.expert_bytes + ec.PAGE - 1) // ec.PAGE * ec.PAGE
    kw = dict(num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=512)
    resident = mla.MlaMoEGPU(w, **kw)
    paged = mla.MlaMoEGPU(w, expert_paging=dict(path=lay.path, budget_bytes=9 * rec + 5), **kw)
    assert paged.paged.slots == 9 and paged.weight_bytes() < resident.weight_bytes()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=100).tolist()
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = i32([3, 7])
    T = len(prompt)
    pos = list(range(T))
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
    args = (i32(prompt), i32(pos), i32([int(bt[0, p // 64]) * 64 + p % 64 for p in pos]), i32([0] * T), i32([p + 1 for p in pos]), bt)
    a = resident.forward_rows(*args, prefill=pf).clone()
    b = paged.forward_rows(*args, prefill=pf).clone()
    assert torch.equal(a, b)
    t0 = int(a[-1, :cfg.vocab].argmax())
    for step in range(3):
        p = T + step
        a2 = (i32([t0]), i32([p]), i32([int(bt[0, p // 64]) * 64 + p % 64]), i32([0]), i32([p + 1]), bt)
        ga = resident.forward_rows(*a2, max_ctx=256).clone()
        gb = paged.forward_rows(*a2, max_ctx=256).clone()
        assert torch.equal(ga, gb)
        t0 = int(ga[0, :cfg.vocab].argmax())
    paged.check()
    st = paged.paged.stats()
    assert st["evictions"] > 0 and st["cold"] > 0 and st["asked"] > st["cold"]
    paged.paged.close()


@pytest.mark.gpu
def test_server_pages_the_experts_of_a_pack(tmp_path):
    """`--expert-cache-mib` on a MoE pack: the record file appears inside the pack, replies equal the all-resident server's, and /metrics
    carries the cache's counters."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from starlette.testclient import TestClient
    from rexl3_b200.quant import packs
    from rexl3_b200.server.main import make_app, parser
    cfg = moe.CONFIGS["test-moe"]
    folder = str(tmp_path / "pack")
    packs.write_moe_pack(folder, moe.random_moe_weights(cfg, seed=1))
    base = ["--backend", "cuda", "--model", folder, "--slots", "3", "--max-model-len", "512", "--prefill-chunk", "128", "--kv-tokens", "2048",
            "--window-rows", "16", "--spec", "none"]
    texts = []
    for extra in ([], ["--expert-cache-mib", "1"]):
        app, handle = make_app(parser().parse_args(base + extra))
        try:
            assert handle.wait_ready(120), handle.error
            with TestClient(app) as c:
                r = c.post("/v1/completions", json={"prompt": "the experts of this model live on disk", "max_tokens": 8, "temperature": 0})
                assert r.status_code == 200, r.text
                texts.append(r.json()["choices"][0]["text"])
                if extra:
                    m = c.get("/metrics").text
                    assert "rexl3_expert_cache_slots" in m and "rexl3_expert_cache_cold_total" in m
        finally:
            handle.stop()
    assert texts[0] == texts[1]
    import os
    assert os.path.exists(os.path.join(folder, "experts.records"))


def test_a_record_file_of_another_pack_is_rewritten(tmp_path):
    cfg = moe.CONFIGS["test-moe"]
    path = str(tmp_path / "e.bin")
    xp.write_records(moe.random_moe_weights(cfg, seed=1), path, tag="pack-a")
    a = open(path, "rb").read()
    xp.write_records(moe.random_moe_weights(cfg, seed=2), path, tag="pack-a")          # same tag: trusted, kept
    assert open(path, "rb").read() == a
    xp.write_records(moe.random_moe_weights(cfg, seed=2), path, tag="pack-b")          # same shape, another pack: rewritten
    b = open(path, "rb").read()
    assert len(b) == len(a) and b != a and open(path + ".tag").read() == "pack-b"
    xp.write_records(moe.random_moe_weights(cfg, seed=1), path)                        # untagged caller: does not trust a tagged file
    assert open(path, "rb").read() == a and not __import__("os").path.exists(path + ".tag")


@pytest.mark.gpu
def test_a_window_that_needs_more_experts_than_slots_fails_its_batch_only(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.engine import BackendError, RowRequest
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    cfg = moe.CONFIGS["test-moe"]
    w = moe.random_moe_weights(cfg, seed=1)
    lay = xp.write_records(w, str(tmp_path / "e.bin"))
    rec = (lay.expert_bytes + ec.PAGE - 1) // ec.PAGE * ec.PAGE
    m = moe.MoEGPU(w, expert_paging=dict(path=lay.path, budget_bytes=3 * rec + 1), num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4,
                   max_prefill_rows=128)
    be = DenseGpuBackend(m, max_slots=4)
    rng = np.random.default_rng(0)
    with pytest.raises(BackendError) as e:
        be.prefill_slice(0, 0, rng.integers(0, cfg.vocab, size=100).tolist(), 4, True)        # 200 picks: all 8 experts of a layer, 3 slots
    assert not e.value.fatal and "the slab holds 3" in str(e.value)
    be.release(0)
    out = be.prefill_slice(1, 0, [5], 4, True)             # one row picks 2 experts per layer: fits
    assert out is not None and np.isfinite(out.values).all()
    assert be.step([RowRequest(1, [7], 1)], 4)[0][0].ids.shape == (4,)
    m.paged.close()
