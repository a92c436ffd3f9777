"""Runtime interventions: manifest validation (fail closed, both sides named), orthonormalisation, the oracle, and the device path."""
import json
import os

import numpy as np
import pytest
import torch

from rexl3_b200.models import intervention as iv


def _write(tmp, d=64, layers=(1, 2), n_layers=4, **kw):
    rng = np.random.default_rng(0)
    a, b = rng.normal(size=d), rng.normal(size=(2, d))
    iv.write(str(tmp), n_layers=n_layers, d_model=d, directions=[("a.npy", a, list(layers)), ("b.npy", b, [layers[-1]])], alpha=kw.get("alpha", 1.0),
             model_name="m")
    return a, b


def test_load_orthonormalises_in_manifest_order(tmp_path):
    a, b = _write(tmp_path)
    ov = iv.load(str(tmp_path), n_layers=4, d_model=64, model_name="m")
    assert sorted(ov) == [1, 2] and ov[1].basis.shape == (1, 64) and ov[2].basis.shape == (3, 64)
    B = ov[2].basis.astype(np.float64)
    assert np.allclose(B @ B.T, np.eye(3), atol=1e-6)
    assert np.allclose(B[0], a / np.linalg.norm(a), atol=1e-6)            # the first direction is only normalised
    y = torch.randn(5, 64, dtype=torch.float64)
    z = iv.apply_reference(y, iv.LayerOverlay(2, 1.0, ov[2].basis)).double()
    assert float((z @ torch.from_numpy(B).T).abs().max()) < 1e-5            # nothing of the ablated span is left


@pytest.mark.parametrize("case", ["layers", "width", "sha", "schema", "layer_range", "dependent", "name", "path"])
def test_mismatches_refuse_naming_both_sides(tmp_path, case):
    _write(tmp_path)
    mp = os.path.join(tmp_path, "intervention.json")
    man = json.load(open(mp))
    kw = dict(n_layers=4, d_model=64, model_name="m")
    if case == "layers":
        kw["n_layers"] = 6
        want = ("n_layers 4", "n_layers 6")
    elif case == "width":
        kw["d_model"] = 128
        want = ("d_model 64", "d_model 128")
    elif case == "sha":
        with open(os.path.join(tmp_path, "a.npy"), "ab") as f:
            f.write(b"x")
        want = ("sha256", "pinned")
    elif case == "schema":
        man["schema"] = "other.v9"
        want = ("other.v9", iv.SCHEMA)
    elif case == "layer_range":
        man["directions"][0]["layers"] = [1, 9]
        want = ("layer 9", "0..3")
    elif case == "dependent":
        a = np.load(os.path.join(tmp_path, "a.npy"))
        np.save(os.path.join(tmp_path, "b.npy"), np.stack([a * 2.0, a * -1.0]))
        import hashlib
        man["directions"][1]["sha256"] = hashlib.sha256(open(os.path.join(tmp_path, "b.npy"), "rb").read()).hexdigest()
        want = ("span",)
    elif case == "name":
        kw["model_name"] = "other"
        want = ("'m'", "'other'")
    else:
        man["directions"][0]["file"] = "../a.npy"
        want = ("plain file name",)
    json.dump(man, open(mp, "w"))
    with pytest.raises(iv.InterventionError) as e:
        iv.load(str(tmp_path), **kw)
    for w in want:
        assert w in str(e.value), str(e.value)


def test_oracle_applies_the_overlay_at_the_block_output(tmp_path):
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["tiny-llama"]
    w = dense.random_weights(cfg, seed=2)
    rng = np.random.default_rng(1)
    iv.write(str(tmp_path), n_layers=cfg.n_layers, d_model=cfg.d_model, directions=[("d.npy", rng.normal(size=cfg.d_model), [0])], alpha=1.0)
    ov = iv.load(str(tmp_path), n_layers=cfg.n_layers, d_model=cfg.d_model)
    plain, steered = dense.ReferenceDense(w), dense.ReferenceDense(w)
    steered.interventions = ov
    toks = [3, 9, 27, 81]
    a, b = plain.forward_seq(0, toks, 0), steered.forward_seq(0, toks, 0)
    assert float((a - b).abs().max()) > 1e-4


@pytest.mark.gpu
def test_device_path_matches_the_oracle(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import dense
    cfg = dense.CONFIGS["test-hd128"]
    w = dense.random_weights(cfg, seed=4)
    rng = np.random.default_rng(2)
    iv.write(str(tmp_path), n_layers=cfg.n_layers, d_model=cfg.d_model,
             directions=[("d.npy", rng.normal(size=(2, cfg.d_model)), [0, 1])], alpha=1.0)
    ov = iv.load(str(tmp_path), n_layers=cfg.n_layers, d_model=cfg.d_model)
    ref = dense.ReferenceDense(w, device="cuda")
    ref.interventions = ov
    m = dense.DenseGPU(w, num_pages=16, max_rows=64, max_seqs=4, max_blocks_per_seq=4, max_prefill_rows=128)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    bt = torch.zeros(4, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = i32([3, 7])
    toks = rng.integers(0, cfg.vocab, size=60).tolist()
    T = len(toks)
    pos = list(range(T))
    slots = [int(bt[0, p // 64]) * 64 + p % 64 for p in pos]
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
    args = (i32(toks), i32(pos), i32(slots), i32([0] * T), i32([p + 1 for p in pos]), bt)
    plain = m.forward_rows(*args, prefill=pf, logit_rows=torch.tensor([T - 1], device="cuda"))[0, :cfg.vocab].clone()
    m.set_interventions(ov)
    got = m.forward_rows(*args, prefill=pf, logit_rows=torch.tensor([T - 1], device="cuda"))[0, :cfg.vocab].clone()
    m.check()
    want = ref.forward_seq(0, toks, 0)[-1]
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() < 0.05 * scale
    assert (got - plain).abs().max().item() > 0.02 * scale         # the overlay moved the logits
