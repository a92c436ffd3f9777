"""Pack (checkpoint directory) writer and loader for the mixture-of-experts families: the MoE GQA decoder (`rexl3_moe`: EXL3 experts) and
the MLA + MoE decoder (`rexl3_mla_moe`: EXL3 attention / shared / dense tensors, MXFP4 routed experts).  Same directory layout as the
dense packs (`quant.quantize.write_pack`): config.json with `quantization_config`, model.safetensors, its index, generation_config.json.

Tensor names (Hugging Face style, so the header scanner groups them as usual):
  model.layers.N.self_attn.{qkv_proj | qkv_a_proj | q_b_proj | o_proj}.{trellis,suh,svh,...}   EXL3 groups
  model.layers.N.self_attn.{q_a_layernorm,kv_a_layernorm}.weight, .w_uk, .w_uv                  BF16 (absorbed up-projections per head)
  model.layers.N.mlp.gate.weight (BF16 router), .mlp.gate.e_score_correction_bias (F32)
  model.layers.N.mlp.experts.E.{gate_up_proj,down_proj}.{trellis,...}                            EXL3 experts (MoE family)
  model.layers.N.mlp.experts.E.{gate_up_proj,down_proj}.weight (I8 E2M1 nibbles) + .weight_scale (F8_E8M0)   MXFP4 experts (MLA family)
  model.layers.N.mlp.{gate_up_proj,down_proj} (dense layer) / .mlp.shared_experts.{gate_up_proj,down_proj}   EXL3 groups
Refusals are by name, before any tensor is read (the scanner's group rules, reference crates/exl3/src/checkpoint.rs:194-271; MXFP4 layout
crates/cuda/csrc/fp4_linear.cu:5-18).
"""
from __future__ import annotations

import json
import os

import numpy as np

from ..format import checkpoint, exl3, safetensors_io
from ..models.dense import HostLinear, HostWeights
from .quantize import _f32_to_bf16_bits


class _Writer:
    def __init__(self):
        self.tensors, self.dtypes = {}, {}

    def plain(self, name, a):
        self.tensors[name] = _f32_to_bf16_bits(np.ascontiguousarray(a, dtype=np.float32))
        self.dtypes[name] = "BF16"

    def f32(self, name, a):
        self.tensors[name] = np.ascontiguousarray(a, dtype=np.float32)

    def lin(self, prefix, l: HostLinear):
        t = self.tensors
        t[prefix + ".trellis"] = l.trellis
        t[prefix + ".suh"] = l.suh.astype(np.float16)
        t[prefix + ".svh"] = l.svh.astype(np.float16)
        if l.codebook == "mcg":
            t[prefix + ".mcg"] = np.array([exl3.MARKER_MCG], dtype=np.uint32).view(np.int32)
        elif l.codebook == "mul1":
            t[prefix + ".mul1"] = np.array([exl3.MARKER_MUL1], dtype=np.uint32).view(np.int32)
        if l.bias is not None:
            t[prefix + ".bias"] = l.bias.astype(np.float32)

    def mxfp4(self, prefix, packed, scales):
        self.tensors[prefix + ".weight"] = np.ascontiguousarray(packed).view(np.int8)
        self.tensors[prefix + ".weight_scale"] = np.ascontiguousarray(scales, dtype=np.uint8)
        self.dtypes[prefix + ".weight_scale"] = "F8_E8M0"

    def finish(self, folder, conf):
        os.makedirs(folder, exist_ok=True)
        safetensors_io.write_file(os.path.join(folder, "model.safetensors"), self.tensors, {"format": "pt"}, self.dtypes)
        json.dump({"metadata": {}, "weight_map": {k: "model.safetensors" for k in sorted(self.tensors)}},
                  open(os.path.join(folder, "model.safetensors.index.json"), "w"), indent=1)
        json.dump(conf, open(os.path.join(folder, "config.json"), "w"), indent=1)
        json.dump({"eos_token_id": conf.get("eos_token_id", conf["vocab_size"] - 1)}, open(os.path.join(folder, "generation_config.json"), "w"))


def write_moe_pack(folder: str, w: HostWeights) -> None:
    cfg, W = w.cfg, _Writer()
    W.plain("model.embed_tokens.weight", w.embed)
    for i, L in enumerate(w.layers):
        p = f"model.layers.{i}."
        W.plain(p + "input_layernorm.weight", L.attn_norm)
        W.plain(p + "post_attention_layernorm.weight", L.ffn_norm)
        W.lin(p + "self_attn.qkv_proj", L.qkv)
        W.lin(p + "self_attn.o_proj", L.o)
        if L.q_norm is not None:
            W.plain(p + "self_attn.q_norm.weight", L.q_norm)
            W.plain(p + "self_attn.k_norm.weight", L.k_norm)
        W.plain(p + "mlp.gate.weight", L.router)
        if L.router_bias is not None:
            W.f32(p + "mlp.gate.e_score_correction_bias", L.router_bias)
        for e, (gu, dn) in enumerate(zip(L.experts_gu, L.experts_down)):
            W.lin(f"{p}mlp.experts.{e}.gate_up_proj", gu)
            W.lin(f"{p}mlp.experts.{e}.down_proj", dn)
    W.plain("model.norm.weight", w.final_norm)
    W.lin("lm_head", w.lm_head)
    W.finish(folder, {"architectures": ["Rexl3MoEForCausalLM"], "model_type": "rexl3_moe", "hidden_size": cfg.d_model, "num_hidden_layers": cfg.n_layers,
                      "num_attention_heads": cfg.n_q, "num_key_value_heads": cfg.n_kv, "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn,
                      "vocab_size": cfg.vocab, "rms_norm_eps": cfg.eps, "rope_theta": cfg.rope_theta, "qk_norm": cfg.qk_norm, "name": cfg.name,
                      "num_experts": cfg.n_experts, "num_experts_per_tok": cfg.top_k, "moe_intermediate_size": cfg.expert_ffn,
                      "router_mode": cfg.router_mode, "routed_scaling_factor": cfg.routed_scale, "draft_layers": cfg.draft_layers,
                      "expert_act": cfg.expert_act, "n_group": cfg.n_group, "topk_group": cfg.topk_group,
                      "quantization_config": {"quant_method": "exl3", "version": "0.0.1", "bits": cfg.bits, "head_bits": cfg.head_bits or cfg.bits,
                                              "codebook": cfg.codebook, "fused_projections": True}})


def write_mla_pack(folder: str, w) -> None:
    cfg, W = w.cfg, _Writer()
    W.plain("model.embed_tokens.weight", w.embed)
    for i, L in enumerate(w.layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        W.plain(p + "input_layernorm.weight", L.attn_norm)
        W.plain(p + "post_attention_layernorm.weight", L.ffn_norm)
        W.lin(a + "qkv_a_proj", L.qkv_a)
        W.plain(a + "q_a_layernorm.weight", L.q_norm)
        W.plain(a + "kv_a_layernorm.weight", L.kv_norm)
        W.lin(a + "q_b_proj", L.q_b)
        W.plain(a + "w_uk", L.w_uk)
        W.plain(a + "w_uv", L.w_uv)
        W.lin(a + "o_proj", L.o)
        if L.router is None:
            W.lin(p + "mlp.gate_up_proj", L.gate_up)
            W.lin(p + "mlp.down_proj", L.down)
            continue
        W.lin(p + "mlp.shared_experts.gate_up_proj", L.gate_up)
        W.lin(p + "mlp.shared_experts.down_proj", L.down)
        W.plain(p + "mlp.gate.weight", L.router)
        W.f32(p + "mlp.gate.e_score_correction_bias", L.router_bias)
        for e, ((gw, gs), (dw, ds)) in enumerate(zip(L.ex_gu, L.ex_down)):
            W.mxfp4(f"{p}mlp.experts.{e}.gate_up_proj", gw, gs)
            W.mxfp4(f"{p}mlp.experts.{e}.down_proj", dw, ds)
    W.plain("model.norm.weight", w.final_norm)
    W.lin("lm_head", w.lm_head)
    W.finish(folder, {"architectures": ["Rexl3MlaMoEForCausalLM"], "model_type": "rexl3_mla_moe", "hidden_size": cfg.d_model,
                      "num_hidden_layers": cfg.n_layers, "first_k_dense_replace": cfg.n_dense, "num_attention_heads": cfg.n_heads, "q_lora_rank": cfg.q_lora,
                      "kv_lora_rank": cfg.kv_lora, "qk_rope_head_dim": cfg.rope_dim, "qk_nope_head_dim": cfg.nope_dim, "v_head_dim": cfg.v_dim,
                      "intermediate_size": cfg.dense_ffn, "n_routed_experts": cfg.n_experts, "num_experts_per_tok": cfg.top_k,
                      "moe_intermediate_size": cfg.expert_ffn, "n_shared_experts": max(1, cfg.shared_ffn // cfg.expert_ffn), "scoring_func": "sigmoid",
                      "topk_method": "noaux_tc", "n_group": cfg.n_group, "topk_group": cfg.topk_group, "routed_scaling_factor": cfg.routed_scale, "vocab_size": cfg.vocab, "rms_norm_eps": cfg.eps,
                      "rope_theta": cfg.rope_theta, "name": cfg.name,
                      "quantization_config": {"quant_method": "exl3", "version": "0.0.1", "bits": 2.25, "bits_a": cfg.bits_a, "bits_b": cfg.bits_b,
                                              "expert_format": "mxfp4"}})


class _Reader:
    """Header scan + refusals by name, then tensor reads (prefetched in one parallel pass)."""

    def __init__(self, folder: str, threads: int = 8):
        self.folder = folder
        self.ck = ck = checkpoint.scan(folder, verify_markers=True)
        if ck.bad:
            name, why = sorted(ck.bad.items())[0]
            raise ValueError(f"pack refused: {name}: {why}")
        if ck.issues:
            raise ValueError(f"pack refused: {ck.issues[0]}")
        if threads > 0:
            safetensors_io.prefetch(folder, [e for g in ck.groups.values() for e in g.parts.values()] + list(ck.plain.values()), threads=threads)

    def lin(self, prefix) -> HostLinear:
        g = self.ck.groups.get(prefix)
        if g is None:
            raise ValueError(f"pack refused: no EXL3 group {prefix}")
        lg = checkpoint.load_group(self.folder, g)
        return HostLinear(lg.trellis, lg.suh, lg.svh, lg.bias, g.codebook)

    def plain(self, name, optional=False):
        e = self.ck.plain.get(name)
        if e is None:
            if optional:
                return None
            raise ValueError(f"pack refused: no tensor {name}")
        return checkpoint.load_plain(self.folder, e).astype(np.float32)

    def raw(self, name, dtype, shape):
        e = self.ck.plain.get(name)
        if e is None:
            raise ValueError(f"pack refused: no tensor {name}")
        if e.dtype not in dtype:
            raise ValueError(f"pack refused: {name}: dtype {e.dtype}, expected one of {sorted(dtype)}")
        if tuple(e.shape) != tuple(shape):
            raise ValueError(f"pack refused: {name}: shape {list(e.shape)}, expected {list(shape)}")
        return safetensors_io.read_tensor(self.folder, e)

    def mxfp4(self, prefix, n, k):
        """(int8 [n, k/2], uint8 [n, k/32]) of one MXFP4 matrix; shape and dtype are checked against the configuration."""
        w = self.raw(prefix + ".weight", {"I8", "U8"}, (n, k // 2))
        s = self.raw(prefix + ".weight_scale", {"F8_E8M0", "U8"}, (n, k // 32))
        return np.ascontiguousarray(w).view(np.int8), np.ascontiguousarray(s).view(np.uint8)


def load_moe_pack(folder: str, threads: int = 8) -> HostWeights:
    from ..models.moe import HostMoELayer, config_from_dict
    try:
        cfg = config_from_dict(json.load(open(os.path.join(folder, "config.json"))))
        R = _Reader(folder, threads)
        w = HostWeights(cfg, R.plain("model.embed_tokens.weight"))
        for i in range(cfg.n_layers):
            p = f"model.layers.{i}."
            lay = HostMoELayer(R.plain(p + "input_layernorm.weight"), R.lin(p + "self_attn.qkv_proj"), R.lin(p + "self_attn.o_proj"),
                               R.plain(p + "post_attention_layernorm.weight"), None, None)
            if cfg.qk_norm:
                lay.q_norm, lay.k_norm = R.plain(p + "self_attn.q_norm.weight"), R.plain(p + "self_attn.k_norm.weight")
            lay.router = R.plain(p + "mlp.gate.weight")
            if lay.router.shape != (cfg.n_experts, cfg.d_model):
                raise ValueError(f"pack refused: {p}mlp.gate.weight: shape {list(lay.router.shape)}, expected {[cfg.n_experts, cfg.d_model]}")
            lay.router_bias = R.plain(p + "mlp.gate.e_score_correction_bias", optional=cfg.router_mode != "sigmoid_bias")
            lay.experts_gu = [R.lin(f"{p}mlp.experts.{e}.gate_up_proj") for e in range(cfg.n_experts)]
            lay.experts_down = [R.lin(f"{p}mlp.experts.{e}.down_proj") for e in range(cfg.n_experts)]
            w.layers.append(lay)
        w.final_norm = R.plain("model.norm.weight")
        w.lm_head = R.lin("lm_head")
        return w
    finally:
        safetensors_io.drop_prefetched()


def load_mla_pack(folder: str, threads: int = 8):
    from ..models.mla import HostMla, HostMlaLayer, config_from_dict
    try:
        cfg = config_from_dict(json.load(open(os.path.join(folder, "config.json"))))
        R = _Reader(folder, threads)
        d, H = cfg.d_model, cfg.n_heads
        embed = R.plain("model.embed_tokens.weight")
        layers = []
        for i in range(cfg.n_layers):
            p = f"model.layers.{i}."
            a = p + "self_attn."
            lay = HostMlaLayer(R.plain(p + "input_layernorm.weight"), R.lin(a + "qkv_a_proj"), R.plain(a + "q_a_layernorm.weight"),
                               R.plain(a + "kv_a_layernorm.weight"), R.lin(a + "q_b_proj"), R.plain(a + "w_uk").reshape(H, cfg.nope_dim, cfg.kv_lora),
                               R.plain(a + "w_uv").reshape(H, cfg.kv_lora, cfg.v_dim), R.lin(a + "o_proj"), R.plain(p + "post_attention_layernorm.weight"))
            if i < cfg.n_dense:
                lay.gate_up, lay.down = R.lin(p + "mlp.gate_up_proj"), R.lin(p + "mlp.down_proj")
            else:
                lay.gate_up, lay.down = R.lin(p + "mlp.shared_experts.gate_up_proj"), R.lin(p + "mlp.shared_experts.down_proj")
                lay.router = R.plain(p + "mlp.gate.weight")
                lay.router_bias = R.plain(p + "mlp.gate.e_score_correction_bias")
                F = cfg.expert_ffn
                lay.ex_gu = [R.mxfp4(f"{p}mlp.experts.{e}.gate_up_proj", 2 * F, d) for e in range(cfg.n_experts)]
                lay.ex_down = [R.mxfp4(f"{p}mlp.experts.{e}.down_proj", d, F) for e in range(cfg.n_experts)]
            layers.append(lay)
        return HostMla(cfg, embed, layers, R.plain("model.norm.weight"), R.lin("lm_head"))
    finally:
        safetensors_io.drop_prefetched()


def load_any(folder: str, threads: int = 8):
    """Loads the pack of whichever family its config.json names."""
    mt = json.load(open(os.path.join(folder, "config.json"))).get("model_type")
    if mt == "rexl3_moe":
        return load_moe_pack(folder, threads)
    if mt == "rexl3_mla_moe":
        return load_mla_pack(folder, threads)
    from . import quantize
    return quantize.load_pack(folder, threads)
