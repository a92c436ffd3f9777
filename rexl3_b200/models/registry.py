"""Family registry: which executor serves a pack, decided from its `config.json` alone, failing closed.

`probe(folder)` reads the configuration, requires an EXL3 quantization record, finds the one family whose architecture list names
`architectures[0]` (the model type is consulted only when there is no architecture list: a present but unknown architecture is never
rescued by a familiar model type), lets the family validate the configuration, and returns (family, plan).  A configuration nobody
serves is refused with a capability report: what was asked for, which components the configuration implies, which of those this build
has, and the nearest family by name.  A registry in which two families claim one name refuses everything.

Same role and refusal rules as the reference's registry (crates/model/src/family.rs:456-540, `require_exl3` :430-452, component
inventory :243-370); families, plans and executors are this repository's.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

# components this build has executors for (a family may serve a configuration only if every component it implies is here)
BUILT_COMPONENTS = frozenset({
    "exl3_linear", "gqa_attention", "rope", "qk_norm", "swiglu_ffn", "paged_kv_bf16", "paged_kv_fp8", "paged_kv_int8", "paged_kv_q4", "mla_attention", "moe_softmax_topk",
    "moe_sigmoid_bias_topk", "mxfp4_experts", "shared_expert", "mamba2_mixer", "gated_delta_net", "kimi_delta_attention", "self_speculative_draft",
    "copy_draft", "ngram_draft", "prefix_cache", "tensor_parallel", "expert_parallel", "mtp_head", "vision_tower", "mrope", "sparse_indexer",
    "relu2_experts", "draft_trees", "expert_paging", "image_ingress",
})


class FamilyError(ValueError):
    """kind: "config" (unreadable or invalid configuration), "unsupported" (no family accepts it), "registry" (malformed registry)."""

    def __init__(self, kind: str, message: str, report: "CapabilityReport | None" = None):
        super().__init__(message)
        self.kind, self.report = kind, report


@dataclass
class CapabilityReport:
    architecture: str | None
    model_type: str | None
    inferred: list = field(default_factory=list)       # components the configuration implies
    missing: list = field(default_factory=list)        # of those, what this build lacks
    nearest: str | None = None                         # the family whose names share the longest prefix with what was asked for
    served: list = field(default_factory=list)

    def __str__(self) -> str:
        asked = self.architecture or self.model_type or "(no architecture)"
        s = f"no family serves `{asked}`"
        if self.missing:
            s += f"; it needs components this build does not have: {', '.join(self.missing)}"
        if self.nearest:
            s += f"; nearest family: {self.nearest}"
        return s + f"; served architectures: {', '.join(self.served)}"


@dataclass
class FamilyPlan:
    family: str
    config: object               # the family's validated configuration object
    components: list
    tp_max: int = 1
    ep: bool = False
    drafters: tuple = ()
    kv_dtypes: tuple = ("bf16",)
    prefix_cache: bool = True
    vision: bool = False
    notes: list = field(default_factory=list)
    servable: bool = True        # False: the family is known well enough to inventory and size it (probe / plan), no executor serves it
    memory: dict = field(default_factory=dict)


class Family:
    """One served model family.  Subclasses name what they accept and turn a configuration into a plan."""
    id = ""
    architectures: tuple = ()
    model_types: tuple = ()
    tp_max = 1
    drafters: tuple = ("copy", "ngram")
    kv_dtypes: tuple = ("bf16",)

    def plan(self, root: dict, folder: str | None) -> FamilyPlan:
        raise NotImplementedError


def _q(root: dict) -> dict | None:
    for section in (root, root.get("text_config") or {}):
        q = section.get("quantization_config")
        if isinstance(q, dict) and q.get("quant_method") == "exl3":
            return q
    return None


def require_exl3(root: dict) -> dict:
    q = _q(root)
    if q is not None:
        return q
    found = []
    for section in (root, root.get("text_config") or {}):
        for key in ("quantization_config", "quantization"):
            m = (section.get(key) or {}).get("quant_method") if isinstance(section.get(key), dict) else None
            if isinstance(m, str):
                found.append(m)
    what = f"found quant_method={found[0]}" if found else "found no quantization_config with a quant_method"
    raise FamilyError("config", f"this engine serves EXL3 packs only; {what}")


class DenseFamily(Family):
    """Dense GQA decoders (Llama / Qwen3 / Mistral shaped, and this repository's own dense packs)."""
    id = "dense"
    architectures = ("Rexl3DenseForCausalLM", "LlamaForCausalLM", "Qwen3ForCausalLM", "Qwen2ForCausalLM", "MistralForCausalLM")
    model_types = ("rexl3_dense", "llama", "qwen3", "qwen2", "mistral")
    tp_max = 8
    drafters = ("self", "copy", "ngram")
    kv_dtypes = ("bf16", "fp8", "int8", "q4")

    def plan(self, root, folder):
        from ..quant import quantize
        cfg = quantize.config_from_dict(root)
        comps = ["exl3_linear", "gqa_attention", "rope", "swiglu_ffn", "paged_kv_bf16"] + (["qk_norm"] if cfg.qk_norm else [])
        if root.get("attention_bias") or root.get("mlp_bias"):
            raise FamilyError("config", "config.json: attention_bias / mlp_bias: biased projections are not served by the dense family")
        if root.get("sliding_window") and root.get("use_sliding_window", False):
            raise FamilyError("config", "config.json: sliding-window attention is not served by the dense family")
        if root.get("tie_word_embeddings"):
            raise FamilyError("config", "config.json: tie_word_embeddings: the pack must carry its own quantised lm_head")
        mtp = bool(getattr(cfg, "mtp", False))
        if mtp:
            comps.append("mtp_head")
        # the multi-token-prediction block is served on one GPU with a bf16 cache (it is not in the tensor-parallel shard)
        return FamilyPlan(self.id, cfg, comps, tp_max=1 if mtp else self.tp_max, drafters=(("mtp",) if mtp else ()) + self.drafters,
                          kv_dtypes=("bf16",) if mtp else self.kv_dtypes,
                          notes=["multi-token-prediction block: single GPU, bf16 KV cache"] if mtp else [])


class HybridFamily(Family):
    """Recurrent-plus-attention decoders: gated delta net / Kimi delta attention / Mamba2 layers between GQA attention layers."""
    id = "hybrid"
    architectures = ("Rexl3HybridForCausalLM",)
    model_types = ("rexl3_hybrid",)
    drafters = ("copy", "ngram")

    def plan(self, root, folder):
        from ..quant import quantize
        cfg = quantize.config_from_dict(root)
        kinds = set(cfg.pattern)
        comps = ["exl3_linear", "swiglu_ffn"] + (["gqa_attention", "paged_kv_bf16"] if "A" in kinds else []) + (["mamba2_mixer"] if "M" in kinds else []) + \
                (["gated_delta_net"] if "G" in kinds else []) + (["kimi_delta_attention"] if "K" in kinds else [])
        return FamilyPlan(self.id, cfg, comps, drafters=self.drafters)


class MoEFamily(Family):
    """Mixture-of-experts GQA decoders (softmax top-k router, EXL3 experts)."""
    id = "moe"
    architectures = ("Rexl3MoEForCausalLM", "Qwen3MoeForCausalLM")
    model_types = ("rexl3_moe", "qwen3_moe")
    tp_max = 8
    drafters = ("self", "copy", "ngram")

    def plan(self, root, folder):
        from ..models import moe
        cfg = moe.config_from_dict(root)
        return FamilyPlan(self.id, cfg, ["exl3_linear", "gqa_attention", "rope", "moe_softmax_topk", "paged_kv_bf16"], tp_max=8, ep=True, drafters=self.drafters)


class MlaMoEFamily(Family):
    """Multi-head latent attention with sigmoid-bias routed MXFP4 experts and a shared expert (DeepSeek-V3 shaped)."""
    id = "mla_moe"
    architectures = ("Rexl3MlaMoEForCausalLM", "DeepseekV3ForCausalLM")
    model_types = ("rexl3_mla_moe", "deepseek_v3")
    tp_max = 8

    def plan(self, root, folder):
        from ..models import mla
        cfg = mla.config_from_dict(root)
        return FamilyPlan(self.id, cfg, ["exl3_linear", "mla_attention", "moe_sigmoid_bias_topk", "mxfp4_experts", "shared_expert"], tp_max=8, ep=True)


class MimoFamily(Family):
    """MiMo-V2: probe and plan only (config, tensor inventory by count, memory), as in the reference (crates/model/src/families/mimo): the pack is
    recognised, sized and refused by name instead of being mistaken for another family."""
    id = "mimo"
    architectures = ("MiMoV2ForCausalLM",)
    model_types = ("mimo_v2",)

    def plan(self, root, folder):
        t = root.get("text_config") if isinstance(root.get("text_config"), dict) else root

        def need(key, kind=int):
            v = t.get(key)
            if not isinstance(v, kind) or isinstance(v, bool) or v <= 0:
                raise FamilyError("config", f"config.json: `{key}` must be a positive {kind.__name__}")
            return v
        d, L, nq, vocab = need("hidden_size"), need("num_hidden_layers"), need("num_attention_heads"), need("vocab_size")
        nkv = t.get("num_key_value_heads", nq)
        hd = t.get("head_dim", d // nq)
        ffn = need("intermediate_size")
        E, k, eff = t.get("n_routed_experts", t.get("num_experts", 0)) or 0, t.get("num_experts_per_tok", 0) or 0, t.get("moe_intermediate_size", 0) or 0
        bits = float((_q(root) or {}).get("bits", 4.0))
        attn = d * (nq + 2 * nkv) * hd + nq * hd * d
        ffn_params = 3 * d * eff * E + d * E if E else 3 * d * ffn
        params = L * (attn + ffn_params) + 2 * vocab * d
        mem = dict(parameters=int(params), weight_bytes=int(params * bits / 8), kv_bytes_per_token=int(2 * L * nkv * hd * 2),
                   active_parameters_per_token=int(L * (attn + (3 * d * eff * k if E else 3 * d * ffn)) + vocab * d))
        comps = ["exl3_linear", "gqa_attention", "rope"] + (["moe_softmax_topk"] if E else ["swiglu_ffn"])
        return FamilyPlan(self.id, dict(d_model=d, n_layers=L, n_q=nq, n_kv=nkv, head_dim=hd, ffn=ffn, n_experts=E, top_k=k, expert_ffn=eff, vocab=vocab,
                                        bits=bits), comps, servable=False, memory=mem,
                          notes=["probe / plan only: this family's executor (hybrid sliding-window attention, MTP layers, audio and vision towers) is not built"])


def generic_memory(root: dict) -> tuple:
    """(config summary, memory model) of a decoder described by well-known Hugging Face keys: GQA or latent attention, dense or routed
    feed-forward blocks (+ shared experts), recurrent layers counted from a layer-type list where the configuration carries one."""
    t = root.get("text_config") if isinstance(root.get("text_config"), dict) else root

    def need(key):
        v = t.get(key)
        if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
            raise FamilyError("config", f"config.json: `{key}` must be a positive int")
        return v
    d, L, nq, vocab = need("hidden_size"), need("num_hidden_layers"), need("num_attention_heads"), need("vocab_size")
    nkv = t.get("num_key_value_heads") or nq
    hd = t.get("head_dim") or d // nq
    bits = float((_q(root) or {}).get("bits", 4.0))
    kv_lora = t.get("kv_lora_rank") or 0
    if kv_lora:
        q_lora, rope, nope, vd = t.get("q_lora_rank") or 0, t.get("qk_rope_head_dim") or 64, t.get("qk_nope_head_dim") or 128, t.get("v_head_dim") or 128
        attn = (d * q_lora + q_lora * nq * (nope + rope) if q_lora else d * nq * (nope + rope)) + d * (kv_lora + rope) + kv_lora * nq * (nope + vd) + nq * vd * d
        kv_tok = (kv_lora + rope) * 2
    else:
        attn = d * (nq + 2 * nkv) * hd + nq * hd * d
        kv_tok = 2 * nkv * hd * 2
    kinds = t.get("layer_types") or t.get("layers_block_type") or []
    n_attn = sum(1 for k in kinds if "attention" in str(k) and "linear" not in str(k)) if kinds else L
    E = t.get("n_routed_experts") or t.get("num_experts") or t.get("num_local_experts") or 0
    k = t.get("num_experts_per_tok") or 0
    eff = t.get("moe_intermediate_size") or 0
    shared = (t.get("n_shared_experts") or 0) * eff
    ffn = t.get("intermediate_size") or 0
    n_dense = t.get("first_k_dense_replace") or 0 if E else L
    moe_layers = L - n_dense if E else 0
    params = L * attn + n_dense * 3 * d * ffn + moe_layers * (3 * d * eff * E + d * E + 3 * d * shared) + 2 * vocab * d
    active = L * attn + n_dense * 3 * d * ffn + moe_layers * (3 * d * eff * k + 3 * d * shared) + vocab * d
    cfg = dict(d_model=d, n_layers=L, attention_layers=n_attn, n_q=nq, n_kv=nkv, head_dim=hd, kv_lora_rank=kv_lora, ffn=ffn, n_experts=E, top_k=k, expert_ffn=eff,
               vocab=vocab, bits=bits)
    mem = dict(parameters=int(params), weight_bytes=int(params * bits / 8), kv_bytes_per_token=int(kv_tok * n_attn), active_parameters_per_token=int(active))
    return cfg, mem


class ProbeOnlyFamily(Family):
    """A family of the reference that this build recognises, inventories and sizes, but has no executor for: the pack is refused for serving
    by its own name with the parts that exist and the parts that are missing, instead of being mistaken for a neighbour."""

    def __init__(self, fid: str, architectures: tuple, model_types: tuple, have: list, missing: str):
        self.id, self.architectures, self.model_types, self.have, self.missing = fid, tuple(architectures), tuple(model_types), list(have), missing

    def plan(self, root, folder):
        cfg, mem = generic_memory(root)
        comps = infer_components(root)
        return FamilyPlan(self.id, cfg, comps, servable=False, memory=mem, vision=bool(root.get("vision_config")),
                          notes=[f"probe / plan only: parts this build has: {', '.join(self.have)}; not built as a family executor: {self.missing}"])


PROBE_ONLY = (
    ProbeOnlyFamily("qwen_flash_next", ("Qwen4ExpForConditionalGeneration", "Qwen4ExpForCausalLM"), (),
                    ["gqa_attention", "gated_delta_net", "hyper_connection kernels", "mtp block (dense family)", "vision tower"],
                    "the QSA indexer, per-layer embedding tables and the composition of hyper-connections with the mixers"),
    ProbeOnlyFamily("glm", ("Glm5NextForConditionalGeneration",), (),
                    ["mla_attention", "kimi_delta_attention", "sparse indexer (DSA with pooled keys)", "hyper_connection kernels", "moe_sigmoid_bias_topk", "mtp block"],
                    "one executor that alternates KDA and sparse MLA layers under hyper-connections, its TP=2 schedule and its vision tower"),
    ProbeOnlyFamily("minicpmv4_7", ("MiniCPMV4_7ForConditionalGeneration", "MiniCPMV4_6ForConditionalGeneration"), ("minicpmv4_7", "minicpmv4_6"),
                    ["gated_delta_net", "gqa_attention", "moe_softmax_topk", "vision preprocessing"],
                    "the GDN + MoE composition, the DSpark drafter and the SigLIP tower with its resampler"),
    ProbeOnlyFamily("bailing_moe_v3", ("BailingMoeV3ForCausalLM",), (),
                    ["mla_attention", "kimi_delta_attention", "moe_sigmoid_bias_topk", "prefix spill tier"],
                    "gated latent attention, the group-limited router and the MTP head of this family"),
    ProbeOnlyFamily("deepseek_v41", ("DeepseekV41ForCausalLM",), ("deepseek_v41_text", "deepseek_v4_1_vision"),
                    ["mla_attention (bf16)", "sparse indexer", "mxfp4_experts", "fp8 block-scaled linear", "hyper_connection kernels", "expert page cache"],
                    "FP8 latent cache and the compressor planes, Engram tables, q4 KV rows and the NextN head on the latent executor"),
    ProbeOnlyFamily("qwen", ("Qwen3_5ForConditionalGeneration", "Qwen3_5ForCausalLM", "Qwen3_5MoeForConditionalGeneration", "Qwen3_5MoeForCausalLM"),
                    ("qwen3_5", "qwen3_5_moe"),
                    ["gated_delta_net + gqa_attention (served from this repository's rexl3_hybrid packs)", "record / commit of recurrent state", "mrope",
                     "vision tower"],
                    "the mapping of this family's own tensor names onto the hybrid executor, the DFlash2 drafter and the MoE variant's composition"),
    ProbeOnlyFamily("nemotron_h_omni", ("NemotronHOmniForConditionalGeneration", "NemotronHForCausalLM"), ("nemotron_h_omni", "nemotron_h"),
                    ["mamba2_mixer", "gqa_attention (NoPE)", "paged_kv_int8", "vision tower", "relu2_experts (gate-free experts in the MoE executor)"],
                    "the latent projections around the latent-MoE feed-forward and its composition with the Mamba2 hybrid, its MTP head and the audio / video towers"),
)

FAMILIES = (DenseFamily(), HybridFamily(), MoEFamily(), MlaMoEFamily(), MimoFamily()) + PROBE_ONLY


def infer_components(root: dict) -> list:
    """What a configuration implies, read from well-known keys (used only for the refusal report)."""
    t = root.get("text_config") or root
    out = ["exl3_linear"]
    if t.get("kv_lora_rank"):
        out.append("mla_attention")
    elif t.get("num_attention_heads"):
        out.append("gqa_attention")
    if t.get("n_routed_experts") or t.get("num_experts") or t.get("num_local_experts"):
        out.append("moe_sigmoid_bias_topk" if t.get("scoring_func") == "sigmoid" or t.get("topk_method") == "noaux_tc" else "moe_softmax_topk")
    if t.get("n_shared_experts"):
        out.append("shared_expert")
    if t.get("mamba_num_heads") or t.get("ssm_state_size"):
        out.append("mamba2_mixer")
    if t.get("linear_num_key_heads") or t.get("linear_key_head_dim"):
        out.append("gated_delta_net")
    if t.get("index_topk") or t.get("index_n_heads"):
        out.append("sparse_indexer")
    if t.get("hc_mult") or t.get("num_hyper_connections") or t.get("mhc_streams"):
        out.append("hyper_connections")
    if t.get("num_nextn_predict_layers"):
        out.append("mtp_head")
    if root.get("vision_config"):
        out.append("vision_tower")
    rs = t.get("rope_scaling") or {}
    if rs.get("mrope_section"):
        out.append("mrope")
    if rs.get("type") == "yarn" or rs.get("rope_type") == "yarn":
        out.append("yarn_rope")
    return out


def _norm(s: str) -> str:
    return "".join(c.lower() for c in s if c.isalnum())


class Registry:
    def __init__(self, families=FAMILIES):
        self.families, self.broken = list(families), None
        seen = {}
        for fam in self.families:
            if not fam.id:
                self.broken = "a family has an empty id"
            if not fam.architectures:
                self.broken = f"family `{fam.id}` accepts no architecture, so nothing could reach it"
            for what, names in (("id", (fam.id,)), ("architecture", fam.architectures), ("model type", fam.model_types)):
                for n in names:
                    if (what, n) in seen:
                        self.broken = f"{what} `{n}` is claimed by both `{seen[(what, n)]}` and `{fam.id}`"
                    seen[(what, n)] = fam.id

    def served(self) -> list:
        return [a for f in self.families for a in f.architectures]

    def detect(self, root: dict) -> Family:
        if self.broken:
            raise FamilyError("registry", f"the family registry is malformed and refuses every pack: {self.broken}")
        arch = root.get("architectures")
        if arch is not None and not isinstance(arch, list):
            raise FamilyError("config", "config.json: `architectures` is not a list")
        a0 = None
        if arch:
            if not isinstance(arch[0], str):
                raise FamilyError("config", "config.json: `architectures[0]` is not a string")
            a0 = arch[0]
        mt = root.get("model_type") if isinstance(root.get("model_type"), str) else None
        for fam in self.families:
            if (a0 is not None and a0 in fam.architectures) or (a0 is None and mt is not None and mt in fam.model_types):
                return fam
        raise FamilyError("unsupported", "", self.report(root, a0, mt))

    def report(self, root: dict, architecture, model_type) -> CapabilityReport:
        inferred = infer_components(root)
        probe = _norm(architecture or model_type or "")
        best, best_len = None, 0
        for fam in self.families:
            for n in (*fam.architectures, *fam.model_types, fam.id):
                m = _norm(n)
                k = 0
                while k < min(len(m), len(probe)) and m[k] == probe[k]:
                    k += 1
                if k > best_len:
                    best, best_len = fam.id, k
        return CapabilityReport(architecture, model_type, inferred, [c for c in inferred if c not in BUILT_COMPONENTS], best if best_len >= 4 else None,
                                self.served())

    def probe(self, folder: str):
        """-> (family, plan) of the pack in `folder`, or FamilyError naming the refusal."""
        path = os.path.join(folder, "config.json")
        try:
            root = json.load(open(path))
        except (OSError, ValueError) as e:
            raise FamilyError("config", f"{path}: {e}")
        if not isinstance(root, dict):
            raise FamilyError("config", f"{path}: not a JSON object")
        return self.probe_config(root, folder)

    def probe_config(self, root: dict, folder: str | None = None):
        require_exl3(root)
        try:
            fam = self.detect(root)
        except FamilyError as e:
            if e.kind == "unsupported":
                raise FamilyError("unsupported", str(e.report), e.report)
            raise
        try:
            plan = fam.plan(root, folder)
        except FamilyError:
            raise
        except (KeyError, TypeError, ValueError) as e:
            raise FamilyError("config", f"config.json refused by family `{fam.id}`: {e.__class__.__name__}: {e}")
        missing = [c for c in plan.components if c not in BUILT_COMPONENTS] if plan.servable else []     # a probe-only plan lists what it would need
        if missing:
            raise FamilyError("unsupported", f"family `{fam.id}` needs components this build does not have: {', '.join(missing)}")
        return fam, plan


_GLOBAL = None


def global_registry() -> Registry:
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = Registry()
    return _GLOBAL


def probe(folder: str):
    return global_registry().probe(folder)
