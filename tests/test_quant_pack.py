"""Quantizer (trellis encoder), pack writer / loader / scanner, and the CPU plumbing path on a quantized micro model."""
import json
import os
import struct

import numpy as np
import pytest

from rexl3_b200 import quant
from rexl3_b200.engine import Engine, generate
from rexl3_b200.engine.cpu_backend import CpuDenseBackend
from rexl3_b200.format import checkpoint, exl3, safetensors_io
from rexl3_b200.models import dense
from rexl3_b200.sampling import GREEDY

MICRO = dense.DenseConfig(n_layers=1, d_model=128, n_q=2, n_kv=1, head_dim=64, ffn=200, vocab=256, bits=4.0, name="micro")


@pytest.fixture(scope="module")
def micro():
    fp = quant.random_fp_weights(MICRO, 0)
    return fp, quant.quantize_dense(MICRO, fp)


@pytest.mark.parametrize("bits,cb,bound", [(4, "3inst", 0.008), (3, "mcg", 0.03), (2.5, "mul1", 0.06), (2, "3inst", 0.11)])
def test_trellis_encoder_emits_valid_rings_with_expected_distortion(bits, cb, bound):
    b = exl3.Bits.of(bits)
    tiles = np.random.default_rng(1).normal(size=(8, 256)).astype(np.float32)
    packed, err = quant.encode_tiles(tiles, b, cb)
    dec = exl3.codebook_f32(cb)[exl3.states(packed, b)]
    assert np.allclose(((dec - tiles) ** 2).sum(1), err, rtol=1e-3)
    assert float(((dec - tiles) ** 2).mean()) < bound
    # the ring is tail-biting: re-packing the decoded states gives the same words
    assert np.array_equal(exl3.pack_tiles(exl3.states(packed, b), b), packed)


def test_quantized_linear_reproduces_the_weight(micro):
    fp, w = micro
    got, want = w.layers[0].o.dense(), fp["layers"][0]["o"]
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 0.09
    x = np.random.default_rng(2).normal(size=(3, 128))
    l = w.layers[0].o
    y = exl3.forward(x, l.trellis, l.codebook, l.suh.astype(np.float64), l.svh.astype(np.float64))
    assert np.allclose(y, x @ l.dense().astype(np.float64), atol=1e-5)
    # padded FFN columns are exactly zero
    gu = w.layers[0].gate_up.dense()
    assert np.abs(gu[:, 200:256]).max() < 3e-2 and w.layers[0].gate_up.trellis.shape[1] * 16 == 512


def test_pack_round_trip_scan_and_refusals(micro, tmp_path):
    _, w = micro
    d = str(tmp_path / "pack")
    quant.write_pack(d, w)
    ck = checkpoint.scan(d)
    assert not ck.bad and not ck.issues and len(ck.groups) == 5
    g = ck.groups["model.layers.0.self_attn.qkv_proj"]
    assert (g.k, g.n, g.bits.value, g.codebook) == (128, 256, 4.0, "3inst")
    w2 = quant.load_pack(d)
    assert np.array_equal(w2.layers[0].gate_up.trellis, w.layers[0].gate_up.trellis)
    assert np.allclose(w2.embed, w.embed, atol=1e-2)
    # hostile header: data_offsets past the file
    raw = open(os.path.join(d, "model.safetensors"), "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hlen])
    hdr["lm_head.trellis"]["data_offsets"][1] += 10 ** 9
    bad = json.dumps(hdr).encode()
    evil = str(tmp_path / "evil")
    os.makedirs(evil)
    open(os.path.join(evil, "model.safetensors"), "wb").write(struct.pack("<Q", len(bad)) + bad + raw[8 + hlen:])
    hs = safetensors_io.read_header(os.path.join(evil, "model.safetensors"))
    assert any("runs past" in i for i in hs.issues) and "lm_head.trellis" not in hs.entries
    # a group that must not load: half width without the mul1 marker
    tr = exl3.random_trellis(8, 8, exl3.Bits.of(2.5))
    bad_dir = str(tmp_path / "bad")
    os.makedirs(bad_dir)
    safetensors_io.write_file(os.path.join(bad_dir, "m.safetensors"), {"x.trellis": tr, "x.suh": np.ones(128, np.float16), "x.svh": np.ones(128, np.float16)})
    assert "mul1" in checkpoint.scan(bad_dir).bad["x"]
    for junk in (b"", b"\x01\x00", struct.pack("<Q", 10 ** 12), struct.pack("<Q", 4) + b"nope"):
        p = str(tmp_path / "junk.safetensors")
        open(p, "wb").write(junk)
        assert safetensors_io.read_header(p).issues


def test_cpu_plumbing_prefill_and_greedy_decode_on_a_quantized_model(micro):
    """The shape of the CPU configuration: prefill a random prompt, greedy-decode, logits checked against the fp32 dequantized model."""
    _, w = micro
    be = CpuDenseBackend(w)
    prompt = np.random.default_rng(3).integers(0, MICRO.vocab, size=64).tolist()
    out = generate(Engine(be, spec="none"), [prompt], 32, GREEDY)[0]
    assert len(out) == 32
    ref = dense.ReferenceDense(w)
    logits = ref.forward_seq(0, prompt, 0)
    assert out[0] == int(logits[-1].argmax())
    seq = prompt + out
    full = dense.ReferenceDense(w).forward_seq(0, seq[:-1], 0)
    assert [int(full[i].argmax()) for i in range(63, len(seq) - 1)] == out


def test_pack_round_trips_the_multi_token_prediction_block(tmp_path):
    import dataclasses
    from rexl3_b200.models import dense, registry
    from rexl3_b200.quant import quantize
    cfg = dataclasses.replace(dense.CONFIGS["tiny-llama"], mtp=True)
    w = dense.random_weights(cfg, seed=3)
    quantize.write_pack(str(tmp_path), w)
    w2 = quantize.load_pack(str(tmp_path))
    assert w2.cfg.mtp and np.array_equal(w2.mtp.e_proj.trellis, w.mtp.e_proj.trellis) and np.array_equal(w2.mtp.layer.down.trellis, w.mtp.layer.down.trellis)
    a, b = dense.ReferenceDense(w), dense.ReferenceDense(w2)
    a.forward_seq(0, [1, 2, 3, 4], 0)
    b.forward_seq(0, [1, 2, 3, 4], 0)
    ma, _ = a.mtp_seq(0, [2, 3, 4], a.last_hidden[:3], 0)
    mb, _ = b.mtp_seq(0, [2, 3, 4], b.last_hidden[:3], 0)
    assert float((ma - mb).abs().max()) == 0.0
    fam, plan = registry.probe(str(tmp_path))
    assert fam.id == "dense" and "mtp_head" in plan.components and plan.drafters[0] == "mtp" and plan.tp_max == 1


def test_moe_pack_keeps_the_expert_activation(tmp_path):
    from rexl3_b200.models import moe
    from rexl3_b200.quant import packs
    cfg = moe.CONFIGS["test-moe-relu2"]
    w = moe.random_moe_weights(cfg, seed=2)
    packs.write_moe_pack(str(tmp_path), w)
    back = packs.load_any(str(tmp_path))
    assert back.cfg.expert_act == "relu2" and back.cfg.router_mode == "sigmoid_bias" and back.cfg.expert_up_width == cfg.expert_ffn
    assert back.layers[1].experts_gu[3].trellis.shape == w.layers[1].experts_gu[3].trellis.shape
    import numpy as np
    assert np.array_equal(back.layers[1].experts_gu[3].trellis, w.layers[1].experts_gu[3].trellis)


def test_group_limited_routing_keys_round_trip(tmp_path):
    import dataclasses
    from rexl3_b200.models import mla, moe
    from rexl3_b200.quant import packs
    cfg = dataclasses.replace(moe.CONFIGS["test-moe"], n_experts=16, top_k=4, router_mode="sigmoid_bias", n_group=4, topk_group=2)
    packs.write_moe_pack(str(tmp_path / "a"), moe.random_moe_weights(cfg, seed=2))
    back = packs.load_any(str(tmp_path / "a")).cfg
    assert (back.n_group, back.topk_group) == (4, 2)
    mc = dataclasses.replace(mla.CONFIGS["test-mla"], n_group=4, topk_group=2)
    packs.write_mla_pack(str(tmp_path / "b"), mla.random_mla_weights(mc, seed=2))
    back = packs.load_any(str(tmp_path / "b")).cfg
    assert (back.n_group, back.topk_group) == (4, 2)
