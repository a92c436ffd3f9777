"""EXL3 quantizer: sign flips + 128-block Hadamard rotation on both sides, global scale, trellis (Viterbi) coding, and
the pack writer / loader.

Stages (behaviour parity with the reference's quantizer outline, crates/quant/src/lib.rs:1-30): W~ = H_K (su * W * sv) H_N / scale
is coded tile by tile to the nearest trellis path, so that suh * (H W_q H) * svh reproduces W.  Without calibration data that is all
(a pure "nearest trellis path" quantizer writes valid EXL3, and random-init benchmark weights need no more); with a Hessian per layer
(`teacher.capture_hessians`) the 16-row tile blocks are coded with LDL error feedback and the scale is refit (`ldlq.py`).
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

from ..format import checkpoint, exl3, safetensors_io
from ..models.dense import DenseConfig, HostLayer, HostLinear, HostWeights
from .trellis import encode_tiles

CODEBOOK_STD = {}
SCALE_GRID = (0.85, 0.92, 1.0, 1.08, 1.17, 1.27)


def _cb_std(cb: str) -> float:
    if cb not in CODEBOOK_STD:
        CODEBOOK_STD[cb] = float(exl3.codebook_f32(cb).astype(np.float64).std())
    return CODEBOOK_STD[cb]


def to_stream_tiles(w: np.ndarray) -> np.ndarray:
    """[K, N] -> [K/16 * N/16, 256] with each tile's values in trellis stream order."""
    k, n = w.shape
    r, c = exl3.tile_positions()
    t = w.reshape(k // 16, 16, n // 16, 16).transpose(0, 2, 1, 3)      # [kt, nt, 16, 16]
    return np.ascontiguousarray(t[:, :, r, c]).reshape(-1, 256)


def quantize_linear(w: np.ndarray, bits: float, codebook: str = "3inst", seed: int = 0, bias=None, threads: int = 0, device: str = "cpu",
                    hessian: np.ndarray | None = None, damp: float = 0.01, refit: bool | None = None, scale_search: bool = False,
                    scale_search_tiles: int = 96) -> HostLinear:
    """w: float [K, N] with y = x @ w.  K and N must be multiples of 128 (pad first).  `device="cuda"` runs the trellis search on the GPU
    (the CUDA encoder emits the same bits as the host one).

    `hessian` [K, K] (second moment of the layer's inputs, e.g. from `teacher.capture_hessians`): the 16-row tile blocks are coded last to
    first with LDL error feedback (LDLQ) instead of independently, and the output scale is refit against the Hessian-weighted error
    (`refit`, default: on with a Hessian, off without).  `scale_search`: instead of matching the codebook's spread exactly, try the scales of
    `SCALE_GRID` around it on a sample of tiles and keep the best (after the rotation the optimum is flat near 1: a small gain, cheap to take)."""
    w = np.asarray(w, dtype=np.float64)
    k, n = w.shape
    if k % 128 or n % 128:
        raise ValueError(f"K={k} and N={n} must be multiples of 128")
    b = exl3.Bits.of(bits)
    if not b.is_integer:
        codebook = "mul1"
    rng = np.random.default_rng(seed)
    su = np.where(rng.random(k) < 0.5, -1.0, 1.0)
    sv = np.where(rng.random(n) < 0.5, -1.0, 1.0)
    rot = exl3.rotate(exl3.rotate((w * su[:, None] * sv[None, :]).T.copy()).T.copy())     # H_K (.) H_N, H symmetric and orthonormal
    std = float(rot.std())
    scale = std / _cb_std(codebook) if std > 0 else 1.0

    def encode_err(tiles):
        if device == "cpu":
            return encode_tiles(tiles, b, codebook, threads)
        from .trellis import encode_tiles_cuda
        out, err = encode_tiles_cuda(tiles, b, codebook, device=device)
        return out.cpu().numpy(), err.cpu().numpy()

    if scale_search and std > 0:
        # global scale search: code a sample of tiles at a few scales around the spread-matched one and keep the scale with the smallest
        # error in weight units (err is in coded units, so it is multiplied back by scale^2)
        all_tiles = to_stream_tiles(rot)
        pick = np.random.default_rng(seed + 99).choice(all_tiles.shape[0], size=min(scale_search_tiles, all_tiles.shape[0]), replace=False)
        sample = all_tiles[np.sort(pick)]
        best = None
        for f in SCALE_GRID:
            err = float(encode_err(sample / (scale * f))[1].astype(np.float64).sum()) * (scale * f) ** 2
            if best is None or err < best[0]:
                best = (err, f)
        scale *= best[1]

    def encode(tiles):
        if device == "cpu":
            return encode_tiles(tiles, b, codebook, threads)[0]
        from .trellis import encode_tiles_cuda
        return encode_tiles_cuda(tiles, b, codebook, device=device)[0].cpu().numpy()

    if hessian is None:
        trellis = encode(to_stream_tiles(rot / scale)).reshape(k // 16, n // 16, b.tile_words)
        hr = None
    else:
        from . import ldlq
        if hessian.shape != (k, k):
            raise ValueError(f"hessian is {hessian.shape}, the layer has {k} inputs")
        hr = ldlq.rotate_hessian(ldlq.finalize_hessian(hessian, damp), su)
        trellis = np.zeros((k // 16, n // 16, b.tile_words), dtype=np.int16)

        def code_block(bi, target):
            trellis[bi] = encode(to_stream_tiles(target)).reshape(n // 16, b.tile_words)
            return exl3.unpack(trellis[bi:bi + 1], codebook).view(np.float16).astype(np.float64)

        ldlq.ldlq(rot / scale, hr, code_block)
    if refit if refit is not None else hessian is not None:
        from . import ldlq
        scale *= ldlq.refit_scale(rot / scale, exl3.unpack(trellis, codebook).view(np.float16).astype(np.float64), hr)
    suh = su.astype(np.float16)
    svh = (sv * scale).astype(np.float16)
    return HostLinear(trellis, suh, svh, None if bias is None else np.asarray(bias, dtype=np.float32), codebook)


def pad_to(w: np.ndarray, k: int, n: int) -> np.ndarray:
    out = np.zeros((k, n), dtype=w.dtype)
    out[:w.shape[0], :w.shape[1]] = w
    return out


def quantize_dense(cfg: DenseConfig, fp: dict, seed: int = 0, threads: int = 0, device: str = "cpu", hessians: dict | None = None,
                   damp: float = 0.01, scale_search: bool = False) -> HostWeights:
    """fp: float weights of a dense GQA decoder, [in, out] matrices: embed [V, d], final_norm [d], lm_head [d, V] and per layer
    attn_norm, q, k, v, o, ffn_norm, gate, up, down (optionally q_norm, k_norm).  `hessians` (from `teacher.capture_hessians`): layers
    found there are coded with LDLQ error feedback, the others tile by tile."""
    d, F, V = cfg.d_model, cfg.ffn_padded, cfg.vocab_padded
    hs = hessians or {}
    ql = lambda m, bits, sd, key: quantize_linear(m, bits, cfg.codebook, sd, threads=threads, device=device, hessian=hs.get(key), damp=damp,  # noqa: E731
                                                  scale_search=scale_search)
    w = HostWeights(cfg, np.asarray(fp["embed"], dtype=np.float32))
    for i, L in enumerate(fp["layers"]):
        qkv = np.concatenate([L["q"], L["k"], L["v"]], axis=1)
        gu = np.concatenate([pad_to(L["gate"], d, F), pad_to(L["up"], d, F)], axis=1)
        lay = HostLayer(np.asarray(L["attn_norm"], np.float32), ql(qkv, cfg.bits, seed + 10 * i + 1, (i, "qkv")),
                        ql(L["o"], cfg.bits, seed + 10 * i + 2, (i, "o")), np.asarray(L["ffn_norm"], np.float32),
                        ql(gu, cfg.bits, seed + 10 * i + 3, (i, "gate_up")), ql(pad_to(L["down"], F, d), cfg.bits, seed + 10 * i + 4, (i, "down")),
                        None if "q_norm" not in L else np.asarray(L["q_norm"], np.float32), None if "k_norm" not in L else np.asarray(L["k_norm"], np.float32))
        w.layers.append(lay)
    w.final_norm = np.asarray(fp["final_norm"], np.float32)
    w.lm_head = ql(pad_to(fp["lm_head"], d, V), cfg.head_bits or cfg.bits, seed + 7777, ("lm_head",))
    if getattr(cfg, "mtp", False):
        # the multi-token-prediction block: fp["mtp"] = {enorm, hnorm, eh_proj [2d, d] (embedding rows first), final_norm, layer: {...}}
        from ..models.dense import HostMtp
        m = fp.get("mtp")
        if m is None:
            raise ValueError("config.mtp is set but the float weights carry no `mtp` block")
        L = m["layer"]
        i = cfg.n_layers
        lay = HostLayer(np.asarray(L["attn_norm"], np.float32), ql(np.concatenate([L["q"], L["k"], L["v"]], axis=1), cfg.bits, seed + 10 * i + 1, (i, "qkv")),
                        ql(L["o"], cfg.bits, seed + 10 * i + 2, (i, "o")), np.asarray(L["ffn_norm"], np.float32),
                        ql(np.concatenate([pad_to(L["gate"], d, F), pad_to(L["up"], d, F)], axis=1), cfg.bits, seed + 10 * i + 3, (i, "gate_up")),
                        ql(pad_to(L["down"], F, d), cfg.bits, seed + 10 * i + 4, (i, "down")),
                        None if "q_norm" not in L else np.asarray(L["q_norm"], np.float32), None if "k_norm" not in L else np.asarray(L["k_norm"], np.float32))
        eh = np.asarray(m["eh_proj"], np.float32)
        w.mtp = HostMtp(np.asarray(m["enorm"], np.float32), np.asarray(m["hnorm"], np.float32), ql(eh[:d], cfg.bits, seed + 10 * i + 5, (i, "e_proj")),
                        ql(eh[d:], cfg.bits, seed + 10 * i + 6, (i, "h_proj")), lay, np.asarray(m["final_norm"], np.float32))
    return w


def quantize_hybrid(cfg, fp: dict, seed: int = 0, threads: int = 0, device: str = "cpu") -> HostWeights:
    """fp: float weights of a hybrid decoder (`random_fp_weights_hybrid` shows the keys): attention layers as in `quantize_dense`; recurrent
    layers carry in_proj [d, real width] (padded here to the stored width with zero columns), out_proj [inner, d] and their small tensors."""
    from ..models.hybrid import HostGdnLayer, HostMambaLayer
    cfg.validate()
    d, F, V = cfg.d_model, cfg.ffn_padded, cfg.vocab_padded
    ql = lambda m, bits, sd: quantize_linear(m, bits, cfg.codebook, sd, threads=threads, device=device)  # noqa: E731
    f32 = lambda a: np.asarray(a, np.float32)  # noqa: E731
    bf = lambda a: _bf16_bits_to_f32(_f32_to_bf16_bits(f32(a)))  # noqa: E731  (stored as bf16: round now so the pack round trip is exact)
    w = HostWeights(cfg, bf(fp["embed"]))
    for i, (kind, L) in enumerate(zip(cfg.pattern, fp["layers"])):
        gu = ql(np.concatenate([pad_to(L["gate"], d, F), pad_to(L["up"], d, F)], axis=1), cfg.bits, seed + 10 * i + 3)
        down = ql(pad_to(L["down"], F, d), cfg.bits, seed + 10 * i + 4)
        if kind == "A":
            w.layers.append(HostLayer(bf(L["attn_norm"]), ql(np.concatenate([L["q"], L["k"], L["v"]], axis=1), cfg.bits, seed + 10 * i + 1),
                                      ql(L["o"], cfg.bits, seed + 10 * i + 2), bf(L["ffn_norm"]), gu, down))
            continue
        width = cfg.in_proj_width if kind == "M" else cfg.delta_proj_width(kind)
        ip = ql(pad_to(L["in_proj"], d, width), cfg.bits, seed + 10 * i + 1)
        op = ql(L["out_proj"], cfg.bits, seed + 10 * i + 2)
        if kind == "M":
            w.layers.append(HostMambaLayer(bf(L["attn_norm"]), ip, op, bf(L["conv_w"]), bf(L["conv_b"]), f32(L["dt_bias"]), f32(L["a_log"]), f32(L["d_skip"]),
                                           bf(L["norm_w"]), bf(L["ffn_norm"]), gu, down))
        else:
            w.layers.append(HostGdnLayer(bf(L["attn_norm"]), ip, op, bf(L["conv_w"]), bf(L["conv_b"]), f32(L["dt_bias"]), f32(L["a_log"]), bf(L["norm_w"]),
                                         bf(L["ffn_norm"]), gu, down, kind == "K"))
    w.final_norm = bf(fp["final_norm"])
    w.lm_head = ql(pad_to(fp["lm_head"], d, V), cfg.head_bits or cfg.bits, seed + 7777)
    return w


def random_fp_weights_hybrid(cfg, seed: int = 0, std: float = 0.02) -> dict:
    """N(0, std) matrices and usual-range SSM parameters for every layer kind of a hybrid config."""
    rng = np.random.default_rng(seed)
    d, hd = cfg.d_model, cfg.head_dim
    g = lambda *s: rng.normal(0, std, size=s).astype(np.float32)  # noqa: E731
    ones = lambda n: np.ones(n, np.float32)  # noqa: E731
    layers = []
    for kind in cfg.pattern:
        L = dict(attn_norm=ones(d), ffn_norm=ones(d), gate=g(d, cfg.ffn), up=g(d, cfg.ffn), down=g(cfg.ffn, d))
        if kind == "A":
            L.update(q=g(d, cfg.n_q * hd), k=g(d, cfg.n_kv * hd), v=g(d, cfg.n_kv * hd), o=g(cfg.n_q * hd, d))
        elif kind == "M":
            H, DI, C = cfg.ssm_heads, cfg.d_inner, cfg.conv_channels
            L.update(in_proj=g(d, DI + C + H), out_proj=g(DI, d), conv_w=rng.normal(0, 0.5, size=(C, 4)).astype(np.float32), conv_b=np.zeros(C, np.float32),
                     dt_bias=rng.uniform(-3, -1, size=H).astype(np.float32), a_log=np.log(rng.uniform(1, 16, size=H)).astype(np.float32),
                     d_skip=ones(H), norm_w=ones(DI))
        else:
            Hv, GI, C = cfg.gdn_v_heads, cfg.gdn_inner, cfg.gdn_conv_channels
            L.update(in_proj=g(d, GI + C + Hv + (GI if kind == "K" else Hv)), out_proj=g(GI, d), conv_w=rng.normal(0, 0.5, size=(C, 4)).astype(np.float32),
                     conv_b=np.zeros(C, np.float32), dt_bias=rng.uniform(-2, 0, size=GI if kind == "K" else Hv).astype(np.float32),
                     a_log=np.log(rng.uniform(0.5, 4, size=Hv)).astype(np.float32), norm_w=ones(128))
        layers.append(L)
    return dict(embed=g(cfg.vocab, d), layers=layers, final_norm=ones(d), lm_head=g(d, cfg.vocab))


def random_fp_weights(cfg: DenseConfig, seed: int = 0, std: float = 0.02) -> dict:
    """N(0, std) matrices from a seed (norm weights 1), the shape of the CPU plumbing benchmark configuration."""
    rng = np.random.default_rng(seed)
    d, hd = cfg.d_model, cfg.head_dim
    g = lambda *s: rng.normal(0, std, size=s).astype(np.float32)  # noqa: E731
    layer = lambda: dict(attn_norm=np.ones(d, np.float32), q=g(d, cfg.n_q * hd), k=g(d, cfg.n_kv * hd), v=g(d, cfg.n_kv * hd), o=g(cfg.n_q * hd, d),  # noqa: E731
                         ffn_norm=np.ones(d, np.float32), gate=g(d, cfg.ffn), up=g(d, cfg.ffn), down=g(cfg.ffn, d))
    layers = [layer() for _ in range(cfg.n_layers)]
    out = dict(embed=g(cfg.vocab, d), layers=layers, final_norm=np.ones(d, np.float32), lm_head=g(d, cfg.vocab))
    if getattr(cfg, "mtp", False):
        out["mtp"] = dict(enorm=np.ones(d, np.float32), hnorm=np.ones(d, np.float32), eh_proj=g(2 * d, d), final_norm=np.ones(d, np.float32), layer=layer())
    return out


# ----------------------------------------------------------------------------------------------------- pack I/O
def _bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def _f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def write_pack(folder: str, w: HostWeights, extra_config: dict | None = None) -> None:
    """A pack directory: config.json (+quantization_config), model.safetensors, model.safetensors.index.json, generation_config.json."""
    os.makedirs(folder, exist_ok=True)
    cfg = w.cfg
    tensors, dtypes = {}, {}

    def put_plain(name, a):
        tensors[name] = _f32_to_bf16_bits(a)
        dtypes[name] = "BF16"

    def put_lin(prefix, l: HostLinear):
        tensors[prefix + ".trellis"] = l.trellis
        tensors[prefix + ".suh"] = l.suh.astype(np.float16)
        tensors[prefix + ".svh"] = l.svh.astype(np.float16)
        if l.codebook == "mcg":
            tensors[prefix + ".mcg"] = np.array([exl3.MARKER_MCG], dtype=np.uint32).view(np.int32)
        elif l.codebook == "mul1":
            tensors[prefix + ".mul1"] = np.array([exl3.MARKER_MUL1], dtype=np.uint32).view(np.int32)
        if l.bias is not None:
            tensors[prefix + ".bias"] = l.bias.astype(np.float32)

    def put_group(prefix, fused_name, part_names, l):
        """A fused projection under its fused name, or - when its parts keep their own input rotations - one group per part under the
        per-linear names other EXL3 packs use (q_proj / k_proj / v_proj, gate_proj / up_proj)."""
        from ..models.dense import HostSplitLinear
        if isinstance(l, HostSplitLinear):
            for name, part in zip(part_names, l.parts):
                put_lin(prefix + name, part)
        else:
            put_lin(prefix + fused_name, l)

    def put_f32(name, a):
        tensors[name] = np.ascontiguousarray(a, dtype=np.float32)

    put_plain("model.embed_tokens.weight", w.embed)
    for i, L in enumerate(w.layers):
        p = f"model.layers.{i}."
        put_plain(p + "input_layernorm.weight", L.attn_norm)
        put_plain(p + "post_attention_layernorm.weight", L.ffn_norm)
        put_group(p + "mlp.", "gate_up_proj", ["gate_proj", "up_proj"], L.gate_up)
        put_lin(p + "mlp.down_proj", L.down)
        if not isinstance(L, HostLayer):              # a recurrent mixer of the hybrid family (Mamba2: "mixer", delta-net: "linear_attn")
            m = p + ("mixer." if hasattr(L, "d_skip") else "linear_attn.")
            put_lin(m + "in_proj", L.in_proj)
            put_lin(m + "out_proj", L.out_proj)
            put_plain(m + "conv1d.weight", L.conv_w)
            put_plain(m + "conv1d.bias", L.conv_b)
            put_plain(m + "norm.weight", L.norm_w)
            put_f32(m + "dt_bias", L.dt_bias)
            put_f32(m + "A_log", L.a_log)
            if hasattr(L, "d_skip"):
                put_f32(m + "D", L.d_skip)
            continue
        put_group(p + "self_attn.", "qkv_proj", ["q_proj", "k_proj", "v_proj"], L.qkv)
        put_lin(p + "self_attn.o_proj", L.o)
        if L.q_norm is not None:
            put_plain(p + "self_attn.q_norm.weight", L.q_norm)
            put_plain(p + "self_attn.k_norm.weight", L.k_norm)
    put_plain("model.norm.weight", w.final_norm)
    put_lin("lm_head", w.lm_head)
    if getattr(w, "mtp", None) is not None:           # the multi-token-prediction block: layer index n_layers, DeepSeek-style names
        m, p = w.mtp, f"model.layers.{cfg.n_layers}."
        put_plain(p + "enorm.weight", m.enorm)
        put_plain(p + "hnorm.weight", m.hnorm)
        put_lin(p + "eh_proj.e", m.e_proj)
        put_lin(p + "eh_proj.h", m.h_proj)
        put_plain(p + "shared_head.norm.weight", m.final_norm)
        put_plain(p + "input_layernorm.weight", m.layer.attn_norm)
        put_plain(p + "post_attention_layernorm.weight", m.layer.ffn_norm)
        put_group(p + "mlp.", "gate_up_proj", ["gate_proj", "up_proj"], m.layer.gate_up)
        put_lin(p + "mlp.down_proj", m.layer.down)
        put_group(p + "self_attn.", "qkv_proj", ["q_proj", "k_proj", "v_proj"], m.layer.qkv)
        put_lin(p + "self_attn.o_proj", m.layer.o)
        if m.layer.q_norm is not None:
            put_plain(p + "self_attn.q_norm.weight", m.layer.q_norm)
            put_plain(p + "self_attn.k_norm.weight", m.layer.k_norm)
    safetensors_io.write_file(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"}, dtypes)
    json.dump({"metadata": {}, "weight_map": {k: "model.safetensors" for k in sorted(tensors)}},
              open(os.path.join(folder, "model.safetensors.index.json"), "w"), indent=1)
    conf = {"architectures": ["Rexl3DenseForCausalLM"], "model_type": "rexl3_dense", "hidden_size": cfg.d_model, "num_hidden_layers": cfg.n_layers,
            "num_attention_heads": cfg.n_q, "num_key_value_heads": cfg.n_kv, "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn,
            "vocab_size": cfg.vocab, "rms_norm_eps": cfg.eps, "rope_theta": cfg.rope_theta, "qk_norm": cfg.qk_norm, "name": cfg.name,
            "quantization_config": {"quant_method": "exl3", "version": "0.0.1", "bits": cfg.bits, "head_bits": cfg.head_bits or cfg.bits,
                                    "codebook": cfg.codebook, "fused_projections": True}}
    if getattr(cfg, "mtp", False):
        conf["num_nextn_predict_layers"] = 1
    if hasattr(cfg, "pattern"):
        conf.update({"architectures": ["Rexl3HybridForCausalLM"], "model_type": "rexl3_hybrid",
                     "hybrid": {"pattern": cfg.pattern, "ssm_heads": cfg.ssm_heads, "ssm_head_dim": cfg.ssm_head_dim, "ssm_groups": cfg.ssm_groups,
                                "ssm_state": cfg.ssm_state, "conv_k": cfg.conv_k, "nope": cfg.nope, "gdn_k_heads": cfg.gdn_k_heads,
                                "gdn_v_heads": cfg.gdn_v_heads}})
    extra = dict(extra_config or {})
    if "calibration" in extra:                    # what the pack was calibrated on belongs to the quantization record
        conf["quantization_config"]["calibration"] = extra.pop("calibration")
    conf.update(extra)
    json.dump(conf, open(os.path.join(folder, "config.json"), "w"), indent=1)
    json.dump({"eos_token_id": conf.get("eos_token_id", cfg.vocab - 1)}, open(os.path.join(folder, "generation_config.json"), "w"))


def config_from_pack(folder: str):
    """The configuration object of the pack's family (dense, hybrid, MoE or MLA + MoE), from config.json."""
    c = json.load(open(os.path.join(folder, "config.json")))
    mt = c.get("model_type")
    if mt == "rexl3_moe":
        from ..models import moe
        return moe.config_from_dict(c)
    if mt == "rexl3_mla_moe":
        from ..models import mla
        return mla.config_from_dict(c)
    return config_from_dict(c)


def config_from_dict(c: dict) -> DenseConfig:
    """Dense / hybrid configuration from a config.json dictionary.  Reads the Hugging Face keys, so Llama / Qwen3 / Mistral shaped
    configurations map directly; `qk_norm` defaults to true for the qwen3 model type (per-head q / k RMSNorm)."""
    q = c.get("quantization_config") or (c.get("text_config") or {}).get("quantization_config")
    if not q or q.get("quant_method") != "exl3":
        raise ValueError("config.json has no quantization_config with quant_method exl3")
    common = dict(n_layers=c["num_hidden_layers"], d_model=c["hidden_size"], n_q=c["num_attention_heads"], n_kv=c["num_key_value_heads"],
                  head_dim=c.get("head_dim", c["hidden_size"] // c["num_attention_heads"]), ffn=c["intermediate_size"], vocab=c["vocab_size"],
                  eps=c.get("rms_norm_eps", 1e-6), rope_theta=c.get("rope_theta", 1e4), qk_norm=bool(c.get("qk_norm", c.get("model_type") in ("qwen3", "qwen3_moe"))),
                  bits=float(q.get("bits", 4.0)), head_bits=q.get("head_bits"), codebook=q.get("codebook", "3inst"), name=c.get("name", "dense"))
    if c.get("model_type") == "rexl3_hybrid":
        from ..models.hybrid import HybridConfig
        cfg = HybridConfig(**common, **(c.get("hybrid") or {}))
        cfg.validate()
        return cfg
    n_mtp = int(c.get("num_nextn_predict_layers") or 0)
    if n_mtp > 1:
        raise ValueError(f"config.json asks for {n_mtp} multi-token-prediction layers; one is built")
    return DenseConfig(**common, mtp=n_mtp == 1)


def load_pack(folder: str, threads: int = 8, direct: bool = False) -> HostWeights:
    """Scan (headers only), refuse bad groups by name, then read the tensors: all of them in one pass of the native parallel range
    reader (`threads` readers, optionally O_DIRECT), from which the per-tensor reads are served."""
    try:
        return _load_pack(folder, threads, direct)
    finally:
        safetensors_io.drop_prefetched()          # staged tensors nobody asked for, also when a refusal ends the load early


def _load_pack(folder: str, threads: int, direct: bool) -> HostWeights:
    cfg = config_from_pack(folder)
    ck = checkpoint.scan(folder, verify_markers=True)
    if ck.bad:
        name, why = sorted(ck.bad.items())[0]
        raise ValueError(f"pack refused: {name}: {why}")
    if ck.issues:
        raise ValueError(f"pack refused: {ck.issues[0]}")
    from ..utils import loadstats
    t_assemble = time.perf_counter()
    if threads > 0:
        safetensors_io.prefetch(folder, [e for g in ck.groups.values() for e in g.parts.values()] + list(ck.plain.values()), threads=threads, direct=direct)

    def lin(prefix):
        g = ck.groups.get(prefix)
        if g is None:
            raise ValueError(f"pack refused: no EXL3 group {prefix}")
        lg = checkpoint.load_group(folder, g)
        return HostLinear(lg.trellis, lg.suh, lg.svh, lg.bias, g.codebook)

    def fused(prefix, fused_name, parts):
        if prefix + fused_name in ck.groups:
            return lin(prefix + fused_name)
        ls = [lin(prefix + p) for p in parts]
        if any(l.codebook != ls[0].codebook or l.trellis.shape[2] != ls[0].trellis.shape[2] for l in ls[1:]):
            raise ValueError(f"pack refused: {prefix}{'/'.join(parts)} differ in codebook or bit width; projections of one group must share both")
        if any(not np.array_equal(l.suh, ls[0].suh) for l in ls[1:]):
            # quantised one linear at a time (each projection has its own input rotation): served as one GEMM per part
            from ..models.dense import HostSplitLinear
            return HostSplitLinear(ls)
        bias = None if ls[0].bias is None else np.concatenate([l.bias for l in ls])
        return HostLinear(np.concatenate([l.trellis for l in ls], axis=1), ls[0].suh, np.concatenate([l.svh for l in ls]), bias, ls[0].codebook)

    def plain(name):
        e = ck.plain.get(name)
        if e is None:
            raise ValueError(f"pack refused: no tensor {name}")
        return checkpoint.load_plain(folder, e).astype(np.float32)

    def f32(name):
        e = ck.plain.get(name)
        if e is None:
            raise ValueError(f"pack refused: no tensor {name}")
        return checkpoint.load_plain(folder, e).astype(np.float32)

    w = HostWeights(cfg, plain("model.embed_tokens.weight"))
    for i in range(cfg.n_layers):
        p = f"model.layers.{i}."
        kind = getattr(cfg, "pattern", "A" * cfg.n_layers)[i]
        if kind != "A":
            from ..models.hybrid import HostGdnLayer, HostMambaLayer
            m = p + ("mixer." if kind == "M" else "linear_attn.")
            shared = (plain(p + "input_layernorm.weight"), lin(m + "in_proj"), lin(m + "out_proj"), plain(m + "conv1d.weight"), plain(m + "conv1d.bias"),
                      f32(m + "dt_bias"), f32(m + "A_log"))
            tail = (plain(p + "post_attention_layernorm.weight"), fused(p + "mlp.", "gate_up_proj", ["gate_proj", "up_proj"]), lin(p + "mlp.down_proj"))
            if kind == "M":
                w.layers.append(HostMambaLayer(*shared, f32(m + "D"), plain(m + "norm.weight"), *tail))
            else:
                w.layers.append(HostGdnLayer(*shared, plain(m + "norm.weight"), *tail, kind == "K"))
            continue
        lay = HostLayer(plain(p + "input_layernorm.weight"), fused(p + "self_attn.", "qkv_proj", ["q_proj", "k_proj", "v_proj"]), lin(p + "self_attn.o_proj"),
                        plain(p + "post_attention_layernorm.weight"), fused(p + "mlp.", "gate_up_proj", ["gate_proj", "up_proj"]), lin(p + "mlp.down_proj"))
        if cfg.qk_norm:
            lay.q_norm, lay.k_norm = plain(p + "self_attn.q_norm.weight"), plain(p + "self_attn.k_norm.weight")
        w.layers.append(lay)
    w.final_norm = plain("model.norm.weight")
    w.lm_head = lin("lm_head")
    if getattr(cfg, "mtp", False):
        from ..models.dense import HostMtp
        p = f"model.layers.{cfg.n_layers}."
        lay = HostLayer(plain(p + "input_layernorm.weight"), fused(p + "self_attn.", "qkv_proj", ["q_proj", "k_proj", "v_proj"]), lin(p + "self_attn.o_proj"),
                        plain(p + "post_attention_layernorm.weight"), fused(p + "mlp.", "gate_up_proj", ["gate_proj", "up_proj"]), lin(p + "mlp.down_proj"))
        if cfg.qk_norm:
            lay.q_norm, lay.k_norm = plain(p + "self_attn.q_norm.weight"), plain(p + "self_attn.k_norm.weight")
        w.mtp = HostMtp(plain(p + "enorm.weight"), plain(p + "hnorm.weight"), lin(p + "eh_proj.e"), lin(p + "eh_proj.h"), lay, plain(p + "shared_head.norm.weight"))
    read_s = loadstats.snapshot().get(("pack", "read"), (0.0, 0, 0))[0] if threads > 0 else 0.0
    loadstats.add("pack", "assemble", max(0.0, time.perf_counter() - t_assemble - read_s), ck.total_bytes())
    return w
