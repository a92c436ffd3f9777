"""Family registry (fail closed, refusals by name), packs of the MoE / MLA + MoE families, per-linear dense packs, hostile headers."""
import json
import os
import struct

import numpy as np
import pytest

from rexl3_b200.format import checkpoint
from rexl3_b200.models import dense, mla, moe, registry
from rexl3_b200.quant import packs, quantize

Q = {"quant_method": "exl3", "bits": 4.0}
BASE = {"hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512,
        "vocab_size": 1024, "quantization_config": Q}


def test_probe_picks_the_family_by_architecture_and_reads_hf_keys():
    R = registry.Registry()
    fam, plan = R.probe_config(dict(BASE, architectures=["LlamaForCausalLM"], model_type="llama"))
    assert fam.id == "dense" and plan.config.d_model == 256 and not plan.config.qk_norm and plan.tp_max == 8
    fam, plan = R.probe_config(dict(BASE, architectures=["Qwen3ForCausalLM"], model_type="qwen3"))
    assert plan.config.qk_norm and "qk_norm" in plan.components
    # no architecture list: the model type decides
    assert R.probe_config(dict(BASE, model_type="mistral"))[0].id == "dense"


def test_refusals_name_what_is_wrong():
    R = registry.Registry()
    with pytest.raises(registry.FamilyError, match="EXL3 packs only; found quant_method=gptq"):
        R.probe_config(dict(BASE, architectures=["LlamaForCausalLM"], quantization_config={"quant_method": "gptq"}))
    with pytest.raises(registry.FamilyError, match="found no quantization_config"):
        R.probe_config({k: v for k, v in BASE.items() if k != "quantization_config"})
    with pytest.raises(registry.FamilyError, match="`architectures` is not a list"):
        R.probe_config(dict(BASE, architectures="LlamaForCausalLM"))
    # an unknown architecture is never rescued by a familiar model type; the report names missing components and the nearest family
    with pytest.raises(registry.FamilyError) as e:
        R.probe_config(dict(BASE, architectures=["Qwen9FutureForCausalLM"], model_type="llama", rope_scaling={"type": "yarn"}, num_hyper_connections=4))
    msg = str(e.value)
    assert "no family serves `Qwen9FutureForCausalLM`" in msg and "yarn_rope" in msg and "hyper_connections" in msg and "LlamaForCausalLM" in msg
    assert e.value.report.nearest in ("dense", "moe")
    with pytest.raises(registry.FamilyError, match="tie_word_embeddings"):
        R.probe_config(dict(BASE, architectures=["LlamaForCausalLM"], tie_word_embeddings=True))
    with pytest.raises(registry.FamilyError, match="refused by family `dense`"):
        R.probe_config({"architectures": ["LlamaForCausalLM"], "quantization_config": Q})          # no geometry at all


def test_a_registry_with_a_name_claimed_twice_refuses_everything():
    class A(registry.DenseFamily):
        id = "a"

    class B(registry.DenseFamily):
        id = "b"
    R = registry.Registry([A(), B()])
    with pytest.raises(registry.FamilyError, match="claimed by both `a` and `b`"):
        R.probe_config(dict(BASE, architectures=["LlamaForCausalLM"]))


def test_moe_and_mla_packs_round_trip_and_probe(tmp_path):
    w = moe.random_moe_weights(moe.CONFIGS["test-moe"], seed=1)
    packs.write_moe_pack(str(tmp_path / "moe"), w)
    w2 = packs.load_any(str(tmp_path / "moe"))
    assert (w2.cfg.n_experts, w2.cfg.top_k, w2.cfg.expert_ffn, w2.cfg.bits, w2.cfg.d_model) == (w.cfg.n_experts, w.cfg.top_k, w.cfg.expert_ffn, w.cfg.bits, w.cfg.d_model)
    for a, b in ((w.layers[1].experts_gu[3], w2.layers[1].experts_gu[3]), (w.layers[2].experts_down[7], w2.layers[2].experts_down[7]), (w.lm_head, w2.lm_head)):
        assert np.array_equal(a.trellis, b.trellis) and np.array_equal(a.suh, b.suh) and np.array_equal(a.svh, b.svh) and a.codebook == b.codebook
    assert np.array_equal(w.layers[0].router, w2.layers[0].router)
    fam, plan = registry.probe(str(tmp_path / "moe"))
    assert fam.id == "moe" and plan.ep and plan.config.n_experts == 8
    m = mla.random_mla_weights(mla.CONFIGS["test-mla"], seed=2)
    packs.write_mla_pack(str(tmp_path / "mla"), m)
    m2 = packs.load_any(str(tmp_path / "mla"))
    assert m2.cfg == m.cfg
    assert np.array_equal(m.layers[2].ex_gu[1][0], m2.layers[2].ex_gu[1][0]) and np.array_equal(m.layers[2].ex_down[5][1], m2.layers[2].ex_down[5][1])
    assert np.array_equal(m.layers[0].w_uk, m2.layers[0].w_uk) and np.array_equal(m.layers[1].router_bias, m2.layers[1].router_bias)
    assert registry.probe(str(tmp_path / "mla"))[0].id == "mla_moe"
    # the MXFP4 tensors are refused by name when their shape does not fit the configuration
    c = json.load(open(tmp_path / "mla" / "config.json"))
    c["moe_intermediate_size"] = 256
    json.dump(c, open(tmp_path / "mla" / "config.json", "w"))
    with pytest.raises(ValueError, match=r"pack refused: .*(mlp\.experts\.0\.gate_up_proj\.weight|shared_experts)"):
        packs.load_any(str(tmp_path / "mla"))


def test_a_pack_quantised_one_linear_at_a_time_loads_and_matches_its_fused_meaning(tmp_path):
    import torch
    cfg = dense.CONFIGS["test-hd128"]
    w = dense.random_weights(cfg, seed=5, per_linear=True)
    assert isinstance(w.layers[0].qkv, dense.HostSplitLinear) and len(w.layers[0].qkv.parts) == 3 and len(w.layers[0].gate_up.parts) == 2
    quantize.write_pack(str(tmp_path / "p"), w)
    ck = checkpoint.scan(str(tmp_path / "p"))
    assert "model.layers.0.self_attn.k_proj" in ck.groups and "model.layers.0.mlp.up_proj" in ck.groups
    w2 = quantize.load_pack(str(tmp_path / "p"))
    assert isinstance(w2.layers[1].qkv, dense.HostSplitLinear)
    assert not np.array_equal(w2.layers[1].qkv.parts[0].suh, w2.layers[1].qkv.parts[1].suh)
    a, b = dense.ReferenceDense(w), dense.ReferenceDense(w2)
    toks = np.random.default_rng(0).integers(0, cfg.vocab, size=12).tolist()
    assert torch.equal(a.forward_seq(0, toks, 0), b.forward_seq(0, toks, 0))
    assert registry.probe(str(tmp_path / "p"))[0].id == "dense"


def _st(header: dict, data: bytes = b"") -> bytes:
    h = json.dumps(header).encode()
    return struct.pack("<Q", len(h)) + h + data


def test_hostile_headers_are_refusals_by_name_never_allocations(tmp_path):
    d = tmp_path / "h"
    d.mkdir()
    json.dump(dict(BASE, architectures=["LlamaForCausalLM"]), open(d / "config.json", "w"))
    # a 2^40-byte header in a tiny file
    (d / "a.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    ck = checkpoint.scan(str(d))
    assert any("a.safetensors" in i and "exceeds" in i for i in ck.issues)
    # a header that runs past the end of its file
    (d / "a.safetensors").write_bytes(struct.pack("<Q", 4096) + b"{}")
    assert any("past" in i for i in checkpoint.scan(str(d)).issues)
    # offsets outside the data section, data that ends before it starts, a shape that does not match its bytes
    tr = {"dtype": "I16", "shape": [8, 8, 64], "data_offsets": [0, 8 * 8 * 64 * 2]}
    good = {"g.trellis": tr, "g.suh": {"dtype": "F16", "shape": [128], "data_offsets": [8192, 8448]},
            "g.svh": {"dtype": "F16", "shape": [128], "data_offsets": [8448, 8704]}}
    for name, edit in (("past the end", {"g.suh": {"dtype": "F16", "shape": [128], "data_offsets": [8192, 1 << 50]}}),
                       ("ends before", {"g.suh": {"dtype": "F16", "shape": [128], "data_offsets": [8448, 8192]}}),
                       ("shape mismatch", {"g.suh": {"dtype": "F16", "shape": [1 << 40], "data_offsets": [8192, 8448]}}),
                       ("negative", {"g.suh": {"dtype": "F16", "shape": [128], "data_offsets": [-1, 255]}})):
        (d / "a.safetensors").write_bytes(_st(dict(good, **edit), bytes(8704)))
        ck = checkpoint.scan(str(d))
        assert "g" not in ck.groups and ck.issues, name
    # structure: both .suh and .su; a marker that holds the wrong value
    both = dict(good, **{"g.su": {"dtype": "I16", "shape": [8], "data_offsets": [8704, 8720]}})
    (d / "a.safetensors").write_bytes(_st(both, bytes(8720)))
    assert "both" in checkpoint.scan(str(d)).bad["g"]
    mark = dict(good, **{"g.mcg": {"dtype": "I32", "shape": [1], "data_offsets": [8704, 8708]}})
    (d / "a.safetensors").write_bytes(_st(mark, bytes(8704) + struct.pack("<I", 12345)))
    assert "g" in checkpoint.scan(str(d)).groups                         # header-only scan: the value is not read
    ck = checkpoint.scan(str(d), verify_markers=True)
    assert "g" not in ck.groups and "marker" in ck.bad["g"]
    with pytest.raises(ValueError, match="pack refused: g: .*marker"):
        quantize.load_pack(str(d))


def test_probe_only_family_is_sized_and_refused_by_name(tmp_path, capsys):
    """A MiMo-V2 config is recognised, inventoried and sized (`plan`), and the server refuses it as plan-only instead of guessing a family."""
    import json
    from rexl3_b200 import plan as plan_cli
    from rexl3_b200.models import registry
    folder = tmp_path / "mimo"
    folder.mkdir()
    cfg = {"architectures": ["MiMoV2ForCausalLM"], "model_type": "mimo_v2", "hidden_size": 4096, "num_hidden_layers": 48, "num_attention_heads": 32,
           "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 11008, "vocab_size": 151680, "n_routed_experts": 0,
           "quantization_config": {"quant_method": "exl3", "bits": 4.0}}
    (folder / "config.json").write_text(json.dumps(cfg))
    fam, p = registry.probe(str(folder))
    assert fam.id == "mimo" and not p.servable and p.memory["parameters"] > 7e9 and p.memory["kv_bytes_per_token"] == 2 * 48 * 8 * 128 * 2
    assert plan_cli.main(["--pack", str(folder), "--gpus", "1", "--slots", "4", "--max-model-len", "8192"]) == 0
    doc = json.loads(capsys.readouterr().out)
    assert doc["family"] == "mimo" and doc["servable"] is False and doc["fits"] and "probe / plan only" in doc["notes"][0]
    from rexl3_b200.server import main as srv
    args = srv.parser().parse_args(["--model", str(folder), "--backend", "cpu"])
    import pytest as _pt
    with _pt.raises(SystemExit) as e:
        srv.build(args)
    assert "plan_only" in str(e.value) and "mimo" in str(e.value)
    (folder / "config.json").write_text(json.dumps({**cfg, "hidden_size": "big"}))
    with _pt.raises(registry.FamilyError):
        registry.probe(str(folder))


@pytest.mark.parametrize("arch,fid", [("Glm5NextForConditionalGeneration", "glm"), ("DeepseekV41ForCausalLM", "deepseek_v41"),
                                      ("BailingMoeV3ForCausalLM", "bailing_moe_v3"), ("Qwen4ExpForCausalLM", "qwen_flash_next"),
                                      ("MiniCPMV4_7ForConditionalGeneration", "minicpmv4_7"), ("NemotronHForCausalLM", "nemotron_h_omni"),
                                      ("Qwen3_5MoeForCausalLM", "qwen")])
def test_every_reference_family_is_recognised_sized_and_refused_by_its_own_name(tmp_path, arch, fid):
    import json
    from rexl3_b200.models import registry
    cfg = {"architectures": [arch], "hidden_size": 4096, "num_hidden_layers": 40, "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 128,
           "intermediate_size": 12288, "vocab_size": 151936, "n_routed_experts": 128, "num_experts_per_tok": 8, "moe_intermediate_size": 1024,
           "n_shared_experts": 1, "first_k_dense_replace": 2, "kv_lora_rank": 512 if fid in ("glm", "deepseek_v41", "bailing_moe_v3") else 0,
           "q_lora_rank": 1536, "index_topk": 2048, "num_nextn_predict_layers": 1, "quantization_config": {"quant_method": "exl3", "bits": 3.0}}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    fam, p = registry.probe(str(tmp_path))
    assert fam.id == fid and p.servable is False and "probe / plan only" in p.notes[0]
    m = p.memory
    assert m["parameters"] > m["active_parameters_per_token"] > 0 and m["weight_bytes"] == int(m["parameters"] * 3.0 / 8)
    assert m["kv_bytes_per_token"] == (40 * (512 + 64) * 2 if cfg["kv_lora_rank"] else 40 * 2 * 4 * 128 * 2)
    assert "sparse_indexer" in p.components and "mtp_head" in p.components
    from rexl3_b200.server import main as srv
    with pytest.raises(SystemExit) as e:
        srv.build(srv.parser().parse_args(["--model", str(tmp_path), "--backend", "cpu"]))
    assert "plan_only" in str(e.value) and fid in str(e.value)
