"""Vision tower against its own fp32 form on the CPU, bilinear table sampling, and the prompt splice with M-RoPE positions."""
import numpy as np
import pytest
import torch

from rexl3_b200.vision import preprocess, tower


def test_interpolation_table_spans_the_learned_grid():
    idx, w = tower.interpolation_table(3, 5, 8)
    assert idx.shape == (15, 4) and np.allclose(w.sum(1), 1.0)
    assert idx[0, 0] == 0 and w[0, 0] == 1.0                         # the first patch sits on the table's first corner
    assert idx[-1].max() == 63 and np.isclose(w[-1][np.argmax(idx[-1] == 63)] + w[-1][idx[-1] == 63].sum() - w[-1][np.argmax(idx[-1] == 63)], 1.0)
    same, w1 = tower.interpolation_table(8, 8, 8)
    assert np.array_equal(same[:, 0], np.arange(64)) and np.allclose(w1[:, 0], 1.0)      # the table's own resolution: no blending


def test_tower_matches_its_fp32_form_and_merges_windows():
    cfg = tower.CONFIGS["test-vit"]
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, size=(70, 100, 3), dtype=np.uint8)
    inp = preprocess.preprocess_image(img, min_pixels=28 * 28, max_pixels=28 * 28 * 16)
    t32 = tower.VisionTower(cfg, seed=1, device="cpu", dtype=torch.float32)
    out = t32.encode(inp.pixel_values, inp.grid_thw, inp.position_ids)
    assert out.shape == (inp.image_tokens, cfg.out_dim) and torch.isfinite(out).all()
    # bf16 weights, fp32 math (the oracle of the device run) stays close to the all-fp32 network
    ref = tower.VisionTower(cfg, seed=1, device="cpu", dtype=torch.bfloat16).reference("cpu")
    o2 = ref.encode(inp.pixel_values, inp.grid_thw, inp.position_ids)
    assert (o2 - out).abs().max() < 0.05 * out.abs().max()
    # the rotary embedding is axial: shifting every patch by one column changes the encoding, shuffling nothing keeps it
    moved = inp.position_ids.copy()
    moved[:, 1] = (moved[:, 1] + 1) % inp.grid_thw[2]
    assert not torch.allclose(t32.encode(inp.pixel_values, inp.grid_thw, moved), out)
    outside = inp.position_ids.copy()
    outside[:, 1] += 1
    with pytest.raises(ValueError):
        t32.encode(inp.pixel_values, inp.grid_thw, outside)
    clip = preprocess.preprocess_video([img, img, img], min_pixels=28 * 28, max_pixels=28 * 28 * 16)
    oc = t32.encode(clip.pixel_values, clip.grid_thw, clip.position_ids)
    assert oc.shape[0] == clip.image_tokens == 2 * inp.image_tokens
    assert torch.allclose(oc[:inp.image_tokens], oc[inp.image_tokens:], atol=1e-5)     # two identical frame pairs encode alike (attention stays inside one)


def test_splice_positions_follow_the_mrope_rule():
    IMG = 9
    grid = (1, 4, 6)                                                  # merged 2 x 3 -> 6 tokens
    toks = [1, 2] + [IMG] * 6 + [3, 4]
    rows, pos3 = tower.splice(toks, IMG, [grid])
    assert rows.tolist() == list(range(2, 8))
    assert pos3[:2].tolist() == [[0, 0, 0], [1, 1, 1]]
    assert pos3[2:8, 0].tolist() == [2] * 6 and pos3[2:8, 1].tolist() == [2, 2, 2, 3, 3, 3] and pos3[2:8, 2].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos3[8].tolist() == [5, 5, 5] and pos3[9].tolist() == [6, 6, 6]       # text resumes after the largest position the image used
    with pytest.raises(ValueError):
        tower.splice([1, IMG, IMG, 2], IMG, [grid])
    with pytest.raises(ValueError):
        tower.splice([1, 2], IMG, [grid])


@pytest.mark.gpu
def test_tower_on_the_device_and_image_rows_reach_the_decoder():
    """bf16 tower on the GPU against the fp32 oracle; the encoded rows replace the placeholder embeddings of a decoder with M-RoPE sections and
    the logits follow the image (and equal the text-only path when the rows are the table's own embeddings and all axes agree)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import dataclasses
    from rexl3_b200.models import dense
    vcfg = tower.CONFIGS["test-vit"]
    rng = np.random.default_rng(1)
    img = rng.integers(0, 256, size=(60, 90, 3), dtype=np.uint8)
    inp = preprocess.preprocess_image(img, min_pixels=28 * 28, max_pixels=28 * 28 * 16)
    tw = tower.VisionTower(vcfg, seed=2, device="cuda")
    got = tw.encode(inp.pixel_values, inp.grid_thw, inp.position_ids).float().cpu()
    want = tw.reference("cpu").encode(inp.pixel_values, inp.grid_thw, inp.position_ids)
    assert (got - want).abs().max() < 0.06 * want.abs().max()
    cfg = dataclasses.replace(dense.CONFIGS["test-hd128"], mrope_sections=(24, 20, 20))
    assert cfg.d_model == vcfg.out_dim
    m = dense.DenseGPU(dense.random_weights(cfg, seed=3), num_pages=8, max_rows=64, max_seqs=2, max_blocks_per_seq=4, max_prefill_rows=128)
    IMG = 7
    toks = [5, 6] + [IMG] * inp.image_tokens + [8, 9, 10]
    rows, pos3 = tower.splice(toks, IMG, [inp.grid_thw])
    n = len(toks)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    bt = torch.zeros(2, 4, dtype=torch.int32, device="cuda")
    bt[0, :2] = i32([1, 2])
    pos = list(range(n))
    args = (i32(toks), i32(pos), i32([int(bt[0, p // 64]) * 64 + p % 64 for p in pos]), i32([0] * n), i32([p + 1 for p in pos]), bt)
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([n]), pos0=i32([0]), nseq=1, max_qlen=n)
    last = torch.tensor([n - 1], device="cuda")
    text_only = m.forward_rows(*args, prefill=pf, logit_rows=last).clone()
    ridx = torch.as_tensor(rows, device="cuda")
    same_rows = (ridx, m.embed[torch.tensor([IMG] * len(rows), device="cuda")])
    t3 = torch.tensor(pos, dtype=torch.int32, device="cuda")[:, None].repeat(1, 3).contiguous()
    assert torch.equal(m.forward_rows(*args, prefill=pf, logit_rows=last, embed_rows=same_rows, pos3=t3), text_only)
    with_image = m.forward_rows(*args, prefill=pf, logit_rows=last, embed_rows=(ridx, tw.encode(inp.pixel_values, inp.grid_thw, inp.position_ids)),
                                pos3=torch.as_tensor(pos3, device="cuda").contiguous()).clone()
    torch.cuda.synchronize()
    m.check()
    assert torch.isfinite(with_image).all() and (with_image - text_only).abs().max() > 1e-3


def test_tower_round_trips_through_a_pack_folder(tmp_path):
    """save_tower / load_tower: same rows bit for bit (both compute in fp32 from the stored bf16 tensors), config in config.json, refusals by name."""
    import json
    cfg = tower.CONFIGS["test-vit"]
    tw = tower.VisionTower(cfg, seed=5, device="cpu", dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["X"], "hidden_size": 512}))
    tower.save_tower(str(tmp_path), tw)
    doc = json.loads((tmp_path / "config.json").read_text())
    assert doc["hidden_size"] == 512 and doc["vision_config"]["hidden"] == cfg.hidden and doc["vision_config"]["out_dim"] == cfg.out_dim
    assert tower.config_from_pack(str(tmp_path)) == cfg
    back = tower.load_tower(str(tmp_path), "cpu", torch.float32)
    assert back.from_pack
    rng = np.random.default_rng(0)
    inp = preprocess.preprocess_image(rng.integers(0, 256, size=(50, 70, 3), dtype=np.uint8), min_pixels=28 * 28, max_pixels=28 * 28 * 9)
    a = tw.reference("cpu").encode(inp.pixel_values, inp.grid_thw, inp.position_ids)
    b = back.encode(inp.pixel_values, inp.grid_thw, inp.position_ids)
    assert torch.equal(a, b)
    # a folder without the file has no tower; a surplus or a missing tensor, or an unknown config key, is refused by name
    assert tower.config_from_pack(str(tmp_path / "nowhere")) is None
    doc["vision_config"]["colour"] = 1
    (tmp_path / "config.json").write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="unknown keys \\['colour'\\]"):
        tower.config_from_pack(str(tmp_path))
    del doc["vision_config"]["colour"]
    doc["vision_config"]["depth"] = 3
    (tmp_path / "config.json").write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="missing \\['vision.blocks.2"):
        tower.load_tower(str(tmp_path), "cpu", torch.float32)
