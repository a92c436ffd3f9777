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
