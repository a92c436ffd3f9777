"""Mixture-of-experts GQA decoder (the Qwen3-MoE-shaped target of the speculative-decode benchmark: 48 layers, d_model 2048,
32q/4kv x 128, 128 experts of FFN 768, top-8, EXL3 3.0 bpw) on the dense executor's attention path.

FFN of a layer: router (f16/bf16 gate, fp32 scores, exact top-k) -> on-device plan (pairs sorted by expert) -> per-expert input
rotation -> grouped EXL3 GEMM gate|up -> SwiGLU + rotation -> grouped EXL3 GEMM down -> top-k weighted sum in slot order ->
residual / norm / next rotation.  Under expert parallelism every rank holds the experts [e_lo, e_hi); activations are replicated,
so dispatch moves no bytes and the combine is a one-shot all-reduce of each rank's weighted partial rows (summed in rank order).
With data-parallel rows (`a2a=`) the pairs travel to the expert's owner and back over peer memory (token all-to-all, `_ffn_a2a`).
Semantics: reference crates/cuda/csrc/fmoe.cu:11-13 (softmax top-k, renormalised), moe_router.cu:3-13 (sigmoid + bias),
moe_experts.cu:379 (combine), crates/cuda/src/moe_owned.rs:1-30 (expert ownership).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field

import numpy as np
import torch

from ..format import exl3
from ..ops import lib as _lib
from .dense import CONFIGS, DenseConfig, DenseGPU, HostLayer, HostWeights, ReferenceDense, _bf16_round, random_linear

TP_MAX = 8


@dataclass
class MoEConfig(DenseConfig):
    n_experts: int = 8
    top_k: int = 2
    expert_ffn: int = 128
    router_mode: str = "softmax"       # "softmax" (renormalised top-k) | "sigmoid_bias" (DeepSeek-V3: rank by score + bias)
    routed_scale: float = 1.0
    draft_layers: int = 4              # self-speculative draft depth
    n_group: int = 0                   # group-limited routing: experts in `n_group` groups, a row keeps its `topk_group` best groups (0: off)
    topk_group: int = 0
    expert_act: str = "swiglu"         # "swiglu": down(silu(gate) * up), the stack holds gate | up; "relu2": down(relu(up)^2), no gate (the
                                       # feed-forward of the Mamba2 hybrids' experts, reference crates/cuda/csrc/nemotron_moe.cu)

    @property
    def expert_up_width(self) -> int:
        return self.expert_ffn * (2 if self.expert_act == "swiglu" else 1)

    def weight_params(self) -> int:
        attn = self.d_model * self.qkv_width + self.n_q * self.head_dim * self.d_model
        ffn = self.n_experts * (3 if self.expert_act == "swiglu" else 2) * self.d_model * self.expert_ffn
        return (attn + ffn) * self.n_layers + self.vocab_padded * self.d_model


CONFIGS["moe-spec-30b"] = MoEConfig(n_layers=48, d_model=2048, n_q=32, n_kv=4, head_dim=128, ffn=128, vocab=151936, eps=1e-6, rope_theta=1e6,
                                    bits=3.0, name="moe-spec-30b", n_experts=128, top_k=8, expert_ffn=768)
CONFIGS["test-moe-relu2"] = MoEConfig(n_layers=2, d_model=256, n_q=4, n_kv=2, head_dim=128, ffn=128, vocab=1024, bits=3.0, name="test-moe-relu2",
                                      n_experts=16, top_k=6, expert_ffn=128, draft_layers=1, expert_act="relu2", router_mode="sigmoid_bias")
CONFIGS["test-moe"] = MoEConfig(n_layers=3, d_model=256, n_q=4, n_kv=2, head_dim=128, ffn=128, vocab=1024, bits=3.0, name="test-moe",
                                n_experts=8, top_k=2, expert_ffn=128, draft_layers=1)


def _expert_act(c: dict) -> str:
    a = c.get("expert_act", "relu2" if c.get("mlp_hidden_act") == "relu2" else "swiglu")
    if a not in ("swiglu", "relu2"):
        raise ValueError(f"expert activation {a!r}: this executor runs swiglu and relu2 experts")
    return a


def config_from_dict(c: dict) -> MoEConfig:
    """MoE configuration from a config.json dictionary (this repository's `rexl3_moe` packs and Qwen3-MoE shaped Hugging Face keys)."""
    q = c.get("quantization_config") or {}
    if q.get("quant_method") != "exl3":
        raise ValueError("config.json has no quantization_config with quant_method exl3")
    n_exp = c.get("num_experts", c.get("n_routed_experts"))
    if not n_exp:
        raise ValueError("config.json names no experts (num_experts)")
    return MoEConfig(n_layers=c["num_hidden_layers"], d_model=c["hidden_size"], n_q=c["num_attention_heads"], n_kv=c["num_key_value_heads"],
                     head_dim=c.get("head_dim", c["hidden_size"] // c["num_attention_heads"]), ffn=c.get("intermediate_size", 128), vocab=c["vocab_size"],
                     eps=c.get("rms_norm_eps", 1e-6), rope_theta=c.get("rope_theta", 1e6), qk_norm=bool(c.get("qk_norm", False)),
                     bits=float(q.get("bits", 3.0)), head_bits=q.get("head_bits"), codebook=q.get("codebook", "3inst"), name=c.get("name", "moe"),
                     n_experts=int(n_exp), top_k=int(c.get("num_experts_per_tok", 2)), expert_ffn=int(c.get("moe_intermediate_size", 128)),
                     router_mode=c.get("router_mode", "sigmoid_bias" if c.get("scoring_func") == "sigmoid" else "softmax"),
                     routed_scale=float(c.get("routed_scaling_factor", 1.0)), draft_layers=int(c.get("draft_layers", 4)),
                     expert_act=_expert_act(c), n_group=int(c.get("n_group", 0) or 0), topk_group=int(c.get("topk_group", 0) or 0))


@dataclass
class HostMoELayer(HostLayer):
    router: np.ndarray = None            # f32 [E, d] (bf16-rounded)
    router_bias: np.ndarray | None = None
    experts_gu: list = field(default_factory=list)
    experts_down: list = field(default_factory=list)


def random_moe_weights(cfg: MoEConfig, seed: int = 0) -> HostWeights:
    rng = np.random.default_rng(seed)
    d, F = cfg.d_model, cfg.expert_ffn
    s_in = 1.0 / math.sqrt(d)
    w = HostWeights(cfg, _bf16_round(rng.normal(0, 1.0, size=(cfg.vocab, d)).astype(np.float32)))
    for _ in range(cfg.n_layers):
        qkv = random_linear(d, cfg.qkv_width, cfg.bits, rng, cfg.codebook, s_in)
        o = random_linear(cfg.n_q * cfg.head_dim, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(cfg.n_q * cfg.head_dim))
        lay = HostMoELayer(_bf16_round(1.0 + 0.1 * rng.normal(size=d)), qkv, o, _bf16_round(1.0 + 0.1 * rng.normal(size=d)), None, None)
        lay.router = _bf16_round(rng.normal(0, 1.0 / math.sqrt(d), size=(cfg.n_experts, d)))
        if cfg.router_mode == "sigmoid_bias":
            lay.router_bias = rng.normal(0, 0.1, size=cfg.n_experts).astype(np.float32)
        lay.experts_gu = [random_linear(d, cfg.expert_up_width, cfg.bits, rng, cfg.codebook, s_in) for _ in range(cfg.n_experts)]
        lay.experts_down = [random_linear(F, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(F)) for _ in range(cfg.n_experts)]
        w.layers.append(lay)
    w.final_norm = _bf16_round(1.0 + 0.1 * rng.normal(size=d))
    w.lm_head = random_linear(d, cfg.vocab_padded, cfg.head_bits or cfg.bits, rng, cfg.codebook, s_in,
                              zero_cols_from=cfg.vocab if cfg.vocab_padded != cfg.vocab else None)
    return w


def route_reference(logits: torch.Tensor, cfg: MoEConfig, bias: torch.Tensor | None, n_group: int = 0, topk_group: int = 0):
    """fp32 router: (ids [T, k], weights [T, k]) with ties to the lowest expert id.  n_group / topk_group: group-limited routing (a row keeps
    the experts of its `topk_group` best groups, a group's score being the sum of its two best selection keys)."""
    if cfg.router_mode == "softmax":
        p = torch.softmax(logits.float(), dim=-1)
        key = p
    else:
        p = torch.sigmoid(logits.float())
        key = p + (bias if bias is not None else 0)
    if n_group > 1 and topk_group < n_group:
        T, E = key.shape
        per = E // n_group
        gk = key.view(T, n_group, per)
        gs = gk.topk(min(2, per), dim=-1).values.sum(-1)
        _, gorder = torch.sort(gs, dim=-1, descending=True, stable=True)
        keep = torch.zeros(T, n_group, dtype=torch.bool, device=key.device)
        keep.scatter_(1, gorder[:, :topk_group], True)
        key = torch.where(keep[:, :, None].expand(T, n_group, per).reshape(T, E), key, torch.full_like(key, float("-inf")))
    _, ids = torch.sort(key, dim=-1, descending=True, stable=True)
    ids = ids[:, :cfg.top_k]
    wts = torch.gather(p, 1, ids)
    return ids, wts / wts.sum(-1, keepdim=True) * cfg.routed_scale


class ReferenceMoE(ReferenceDense):
    """fp32 oracle: the dense reference with the FFN replaced by routed experts."""

    def __init__(self, w: HostWeights, device="cpu", dtype=torch.float32):
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=dtype)  # noqa: E731
        self.cfg = cfg = w.cfg
        self.device, self.dtype = device, dtype
        self.embed = t(w.embed)
        self.layers = []
        for lay in w.layers:
            self.layers.append(dict(attn_norm=t(lay.attn_norm), qkv=t(lay.qkv.dense()), o=t(lay.o.dense()), ffn_norm=t(lay.ffn_norm),
                                    q_norm=None if lay.q_norm is None else t(lay.q_norm), k_norm=None if lay.k_norm is None else t(lay.k_norm),
                                    router=t(lay.router), router_bias=None if lay.router_bias is None else t(lay.router_bias),
                                    gu=[t(e.dense()) for e in lay.experts_gu], down=[t(e.dense()) for e in lay.experts_down]))
        self.final_norm = t(w.final_norm)
        self.lm_head = t(w.lm_head.dense())[:, :cfg.vocab]
        from .dense import rope_inv_freq
        self.inv_freq = torch.from_numpy(rope_inv_freq(cfg)).to(device)
        self.kv = {}

    def _ffn(self, li, L, h):
        cfg = self.cfg
        x = self._rms(h, L["ffn_norm"], cfg.eps)
        ids, wts = route_reference(x @ L["router"].T, cfg, L["router_bias"], cfg.n_group, cfg.topk_group)
        F = cfg.expert_ffn
        out = torch.zeros_like(h)
        for t in range(x.shape[0]):
            for j in range(cfg.top_k):
                e = int(ids[t, j])
                gu = x[t] @ L["gu"][e]
                act = torch.relu(gu) ** 2 if cfg.expert_act == "relu2" else torch.nn.functional.silu(gu[:F]) * gu[F:]
                out[t] += wts[t, j] * (act @ L["down"][e])
        return h + out


class _ExpertStack:
    """E EXL3 tensors of one shape stacked for the grouped GEMM: trellis [E, K/16, N/16, words], suh [E, K], svh [E, N]."""

    def __init__(self, trellis, suh, svh, codebook):
        self.trellis, self.suh, self.svh, self.codebook = trellis, suh, svh, codebook
        self.E, kt, nt, words = trellis.shape
        self.K, self.N = kt * 16, nt * 16
        self.twice = words * 2 // 16
        self.expert_elems = kt * nt * words          # int16 elements per expert

    @property
    def nbytes(self):
        return self.trellis.numel() * 2 + self.suh.numel() * 2 + self.svh.numel() * 2

    @staticmethod
    def from_host(lins: list, device):
        tr = torch.from_numpy(np.stack([l.trellis for l in lins])).to(device)
        suh = torch.from_numpy(np.stack([l.suh for l in lins]).astype(np.float16)).to(device)
        svh = torch.from_numpy(np.stack([l.svh for l in lins]).astype(np.float16)).to(device)
        return _ExpertStack(tr, suh, svh, lins[0].codebook)


class CombineDst(ctypes.Structure):
    _fields_ = [("ranks", ctypes.c_int), ("rank", ctypes.c_int), ("dst", ctypes.c_void_p * TP_MAX), ("dst_flag", ctypes.c_void_p * TP_MAX),
                ("local_count", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("use_index", ctypes.c_uint), ("rows_cap", ctypes.c_int)]


class MoEGPU(DenseGPU):
    """sm_100a executor.  `experts=(lo, hi)` keeps only those experts on this GPU (expert parallelism); `ep` is then the object
    that supplies the all-reduce slots (see parallel/ep.py); with all experts local the combine writes a local slot."""

    def __init__(self, w, num_pages, max_rows=256, max_seqs=64, max_blocks_per_seq=256, device="cuda", max_prefill_rows=4096, seed=0,
                 experts=None, ep=None, a2a=None, expert_paging=None):
        """`expert_paging` = dict(path=FILE, budget_bytes=N[, fill_threads, direct]): the routed experts stay in a record file (written there
        from the host weights when FILE does not exist yet) and are paged into a device slab of N bytes as the router asks for them
        (models/expert_paging.py); one rank, weights from host tensors.  Every layer's call then costs a device -> host read of its picks.
        `a2a` (parallel.ep.A2aComm): expert parallelism with DATA-PARALLEL rows - every rank feeds its own sequences, a (row, slot) pair
        travels to the rank that owns its expert and its result travels back (token all-to-all); `experts` is then this rank's range."""
        cfg = w if isinstance(w, DenseConfig) else w.cfg
        self.e_lo, self.e_hi = experts or (0, cfg.n_experts)
        self.ep = ep
        self.a2a = a2a
        if a2a is not None and ep is not None:
            raise ValueError("replicated-row expert parallelism (ep) and the token all-to-all (a2a) are two different layouts: pick one")
        self.paged = None
        self._paging = expert_paging
        if expert_paging is not None and (ep is not None or a2a is not None or experts is not None or isinstance(w, DenseConfig)):
            raise ValueError("expert paging runs on one rank that owns every expert, over host weights")
        if ctypes.sizeof(CombineDst) != _lib.load().rx_moe_combine_desc_size():
            raise _lib.KernelError("MoE combine descriptor layout mismatch")
        super().__init__(w, num_pages, max_rows, max_seqs, max_blocks_per_seq, device, max_prefill_rows, seed)

    # ------------------------------------------------------------------ weights
    def _load_host(self, w: HostWeights) -> None:
        K, device = self.K, self.device
        dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=dt)  # noqa: E731
        up = lambda l: K.Exl3Weight.from_numpy(l.trellis, l.suh, l.svh, l.bias, l.codebook, device)  # noqa: E731
        self.embed = dev(w.embed, torch.bfloat16)
        self.layers = []
        lo, hi = self.e_lo, self.e_hi
        stacks = None
        if self._paging is not None:
            from . import expert_paging as xp
            pg = dict(self._paging)
            layout = xp.write_records(w, pg.pop("path"), tag=pg.pop("tag", ""))       # (an existing file of the right size and tag is kept)
            self.paged = xp.PagedExperts(layout, pg.pop("budget_bytes"), device, **pg)
            t, cb = self.paged.slab.t, layout.codebook
            # every layer reads "its experts" from the same slab: a layer's call translates expert ids to slot ids first
            stacks = (_ExpertStack(t["gu_trellis"], t["gu_suh"], t["gu_svh"], cb), _ExpertStack(t["dn_trellis"], t["dn_suh"], t["dn_svh"], cb))
        for lay in w.layers:
            self.layers.append(dict(attn_norm=dev(lay.attn_norm, torch.bfloat16), qkv=up(lay.qkv), o=up(lay.o), ffn_norm=dev(lay.ffn_norm, torch.bfloat16),
                                    q_norm=None if lay.q_norm is None else dev(lay.q_norm, torch.bfloat16),
                                    k_norm=None if lay.k_norm is None else dev(lay.k_norm, torch.bfloat16),
                                    router=dev(lay.router, torch.bfloat16),
                                    router_bias=None if lay.router_bias is None else dev(lay.router_bias, torch.float32),
                                    gu=stacks[0] if stacks else _ExpertStack.from_host(lay.experts_gu[lo:hi], device),
                                    down=stacks[1] if stacks else _ExpertStack.from_host(lay.experts_down[lo:hi], device)))
        self.final_norm = dev(w.final_norm, torch.bfloat16)
        self.lm_head = up(w.lm_head)

    def _load_random(self, seed: int) -> None:
        """Random-init model on the device.  Shared tensors (attention, router, norms, head) come from the seed alone so that every
        expert-parallel rank holds the same ones; the expert stacks are drawn per expert range."""
        cfg, K, device = self.cfg, self.K, self.device
        g = torch.Generator(device=device).manual_seed(seed)
        ge = torch.Generator(device=device).manual_seed(seed * 7919 + 13 + self.e_lo)
        b = exl3.Bits.of(cfg.bits)
        tw = b.tile_words
        cb = cfg.codebook if b.is_integer else "mul1"
        sg = lambda shape, gen: (torch.randint(0, 2, shape, device=device, generator=gen) * 2 - 1)  # noqa: E731

        def lin(k, n, scale):
            tr = torch.randint(-32768, 32768, (k // 16, n // 16, tw), dtype=torch.int16, device=device, generator=g)
            return K.Exl3Weight(tr, sg((k,), g).to(torch.float16), (sg((n,), g) * scale).to(torch.float16), None, cb)

        def stack(e, k, n, scale):
            tr = torch.randint(-32768, 32768, (e, k // 16, n // 16, tw), dtype=torch.int16, device=device, generator=ge)
            return _ExpertStack(tr, sg((e, k), ge).to(torch.float16), (sg((e, n), ge) * scale).to(torch.float16), cb)

        norm = lambda: (1.0 + 0.1 * torch.randn(cfg.d_model, device=device, generator=g)).to(torch.bfloat16)  # noqa: E731
        d, F, HQ, E = cfg.d_model, cfg.expert_ffn, cfg.n_q * cfg.head_dim, self.e_hi - self.e_lo
        self.embed = torch.randn(cfg.vocab, d, device=device, generator=g).to(torch.bfloat16)
        self.layers = []
        for _ in range(cfg.n_layers):
            self.layers.append(dict(attn_norm=norm(), qkv=lin(d, cfg.qkv_width, 1.0 / math.sqrt(d)), o=lin(HQ, d, 0.5 / math.sqrt(HQ)), ffn_norm=norm(),
                                    q_norm=None, k_norm=None,
                                    router=(torch.randn(cfg.n_experts, d, device=device, generator=g) / math.sqrt(d)).to(torch.bfloat16),
                                    router_bias=None if cfg.router_mode == "softmax" else 0.1 * torch.randn(cfg.n_experts, device=device, generator=g),
                                    gu=stack(E, d, cfg.expert_up_width, 1.0 / math.sqrt(d)), down=stack(E, F, d, 0.5 / math.sqrt(F))))
        self.final_norm = norm()
        self.lm_head = lin(d, cfg.vocab_padded, 1.0 / math.sqrt(d))
        if cfg.vocab_padded != cfg.vocab:
            self.lm_head.svh[cfg.vocab:] = 0

    def weight_bytes(self) -> int:
        n = self.embed.numel() * 2 + self.lm_head.nbytes
        for L in self.layers:
            n += L["qkv"].nbytes + L["o"].nbytes + L["router"].numel() * 2 + (0 if self.paged is not None else L["gu"].nbytes + L["down"].nbytes)
        return n + (self.paged.slab.nbytes() if self.paged is not None else 0)

    # ------------------------------------------------------------------ buffers
    def _alloc_scratch(self, R: int):
        cfg, K, dev = self.cfg, self.K, self.device
        super()._alloc_scratch(R)       # the dense scratch sizes its (unused) FFN buffers from cfg.ffn; the expert buffers follow
        k, d, F, E = cfg.top_k, cfg.d_model, cfg.expert_ffn, cfg.n_experts
        S = self.paged.slots if getattr(self, "paged", None) is not None else 0      # paged experts: the kernels see slot ids, 0 .. S - 1
        # token all-to-all: the expert side of a rank may receive every rank's pairs, so its buffers are sized for ranks x rows
        # (whatever class this rank's own window has: a peer may be prefilling while this rank decodes)
        a2a = getattr(self, "a2a", None) is not None
        mult = self.a2a.R if a2a else 1
        Rd = R if a2a else min(R, 256)
        self.pairs_cap = {"decode": Rd * k * mult, "prefill": R * k * mult}   # rows of the sorted-pair buffers a launch of the class addresses
        self.moe_splits = {}
        part = 0
        for cls, rows in (("decode", Rd * mult), ("prefill", R * mult)):
            decode = cls == "decode"
            # the grouped launch already spreads over experts: K splits only where a window has few pairs
            s_gu = K.plan_splits(d, cfg.expert_up_width, decode) if decode else 1
            s_dn = K.plan_splits(F, d, decode) if decode else 1
            s_gu, s_dn = max(1, min(s_gu, 4)), max(1, min(s_dn, 4))
            self.moe_splits[cls] = (s_gu, s_dn)
            part = max(part, s_gu * rows * k * 2 * F, s_dn * rows * k * d)
        if part > self.part.numel():
            self.part = torch.empty(part, dtype=torch.float32, device=dev)
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)  # noqa: E731
        self.xn = torch.empty(R, d, dtype=torch.bfloat16, device=dev)
        self.pick_ids, self.pick_w = i32(R * k), torch.zeros(R * k, dtype=torch.float32, device=dev)
        self.offs, self.pos_of_pair, self.pair_of_pos, self.expert_of_pos, self.total = i32(max(E, S) + 1), i32(R * k * mult), i32(R * k * mult), i32(R * k * mult), i32(1)
        self.recv_ids = i32(R * k * mult) if a2a else None
        El = max(self.e_hi - self.e_lo, S)                               # the tile table only ever names owned experts (or slots)
        if S:
            self.pick_slot = i32(R * k)
            self.slot_table_h = torch.zeros(E, dtype=torch.int32).pin_memory()
            self.slot_table = i32(E)
        # windows use 16- or 32-row tiles (small tiles keep two CTAs per SM); with the all-to-all a 16-row-tile window may receive a peer's slice
        self.max_tiles_decode = El + ((R * k * mult + 15) // 16 if a2a else (min(R, 256) * k + 31) // 32)
        self.max_tiles_prefill = El + (R * k * mult + 127) // 128
        self.router_logits = torch.empty(R, E, dtype=torch.float32, device=dev)
        self.tile_tab = i32(3 * max(self.max_tiles_decode, self.max_tiles_prefill))
        self.xs = torch.zeros(R * k * mult, d, dtype=torch.float16, device=dev)
        self.xs2 = torch.zeros(R * k * mult, F, dtype=torch.float16, device=dev)
        self.slot = torch.zeros(R, d, dtype=torch.float32, device=dev)        # one-rank all-reduce slot
        self._dst = CombineDst()
        self._dst.ranks, self._dst.rank, self._dst.rows_cap = 1, 0, R
        self._dst.dst[0] = self.slot.data_ptr()

    def _begin_forward(self) -> None:
        if self.ep is not None:
            self.ep.begin()
        if self.a2a is not None:
            self.a2a.begin()

    # ------------------------------------------------------------------ the routed FFN
    def _ffn(self, *a):
        for _ in self._ffn_phases(*a):
            pass

    def _ffn_phases(self, li, L, M, cls, s_o, h, xr_d, xr_f, next_norm, next_suh):
        cfg, K = self.cfg, self.K
        Lib = _lib.load()
        st = _lib.stream_ptr()
        k, d, F, E = cfg.top_k, cfg.d_model, cfg.expert_ffn, cfg.n_experts
        pairs = M * k
        cap = self.pairs_cap[cls]
        xn = self.xn[:M]
        K.finish_add_norm_rot(self.part, s_o, M, L["o"], h, L["ffn_norm"], cfg.eps, None, None, xn_out=xn)
        if cfg.n_group > 1 and 0 < cfg.topk_group < cfg.n_group:
            _lib.check(Lib.rx_moe_router_grouped(xn.data_ptr(), L["router"].data_ptr(), _lib.ptr(L["router_bias"]), M, d, E, k,
                                                 0 if cfg.router_mode == "softmax" else 1, cfg.routed_scale, cfg.n_group, cfg.topk_group,
                                                 self.router_logits.data_ptr(), self.pick_ids.data_ptr(), self.pick_w.data_ptr(), st), "rx_moe_router_grouped")
        else:
            _lib.check(Lib.rx_moe_router2(xn.data_ptr(), L["router"].data_ptr(), _lib.ptr(L["router_bias"]), M, d, E, k,
                                          0 if cfg.router_mode == "softmax" else 1, cfg.routed_scale, self.router_logits.data_ptr(),
                                          self.pick_ids.data_ptr(), self.pick_w.data_ptr(), st), "rx_moe_router2")
        if cls == "decode":
            tile_rows, max_tiles = (16 if M <= 16 else 32), self.max_tiles_decode
        else:
            tile_rows, max_tiles = 128, self.max_tiles_prefill
        if self.a2a is not None:
            yield from self._ffn_a2a(li, L, M, cls, xn, tile_rows, max_tiles, h, xr_d, next_norm, next_suh)
            return
        picks, e_lo, e_hi = self.pick_ids, self.e_lo, self.e_hi
        if self.paged is not None:
            # the picks come to the host (which also means every kernel queued so far has run: the last call's leases can go), the experts
            # they name are made resident, and the rest of the layer runs over slot ids
            ids_h = self.pick_ids[:pairs].cpu().numpy()
            self.paged.release_held()
            self.slot_table_h.copy_(torch.from_numpy(self.paged.resolve(li, ids_h)))
            self.slot_table.copy_(self.slot_table_h, non_blocking=True)
            torch.index_select(self.slot_table, 0, self.pick_ids[:pairs].long(), out=self.pick_slot[:pairs])
            picks, E, e_lo, e_hi = self.pick_slot, self.paged.slots, 0, self.paged.slots
        _lib.check(Lib.rx_moe_plan(picks.data_ptr(), pairs, E, e_lo, e_hi, tile_rows, max_tiles, self.offs.data_ptr(),
                                   self.pos_of_pair.data_ptr(), self.pair_of_pos.data_ptr(), self.expert_of_pos.data_ptr(), self.tile_tab.data_ptr(),
                                   self.total.data_ptr(), st), "rx_moe_plan")
        # local expert index = global - e_lo: the stacks hold only the owned experts, so shift the pointers instead of the ids
        gu, dn = L["gu"], L["down"]
        suh_gu = gu.suh.data_ptr() - 2 * self.e_lo * gu.K
        _lib.check(Lib.rx_moe_gather_rot(xn.data_ptr(), picks.data_ptr(), self.pos_of_pair.data_ptr(), pairs, k, d, ctypes.c_void_p(suh_gu),
                                         self.xs.data_ptr(), st), "rx_moe_gather_rot")
        s_gu, s_dn = self.moe_splits[cls]
        self._grouped_shifted(self.xs, gu, s_gu, max_tiles, tile_rows, cap)
        act_rot = Lib.rx_moe_relu2_rot if cfg.expert_act == "relu2" else Lib.rx_moe_swiglu_rot
        _lib.check(act_rot(self.part.data_ptr(), s_gu, cap, F, self.expert_of_pos.data_ptr(), self.total.data_ptr(),
                           ctypes.c_void_p(gu.svh.data_ptr() - 2 * self.e_lo * gu.N), ctypes.c_void_p(dn.suh.data_ptr() - 2 * self.e_lo * dn.K),
                           self.xs2.data_ptr(), st), "rx_moe_act_rot")
        self._grouped_shifted(self.xs2, dn, s_dn, max_tiles, tile_rows, cap)
        dst, ar, flags, ranks, rows_cap, epoch, use = self._combine_target(li, M)
        _lib.check(Lib.rx_moe_combine(self.part.data_ptr(), s_dn, cap, M, d, k, picks.data_ptr(), self.pick_w.data_ptr(),
                                      self.pos_of_pair.data_ptr(), ctypes.c_void_p(dn.svh.data_ptr() - 2 * self.e_lo * dn.N), None, ctypes.byref(dst), st),
                   "rx_moe_combine")
        if self.ep is not None:
            yield          # every rank's combine must be in flight before any rank's sum may wait for it
        _lib.check(Lib.rx_tp_allsum_add_norm_rot(ar, flags, ranks, rows_cap, epoch, use, M, d, h.data_ptr(), next_norm.data_ptr(), cfg.eps,
                                                 next_suh.data_ptr(), xr_d.data_ptr(), self.status.data_ptr(), st, None), "rx_tp_allsum_add_norm_rot")
        _lib.count(8)

    def _ffn_a2a(self, li, L, M, cls, xn, tile_rows, max_tiles, h, xr_d, next_norm, next_suh):
        """The routed FFN with a token all-to-all (the picks of this rank's rows are already in pick_ids / pick_w): dispatch -> (every rank has
        dispatched) -> list what arrived, plan, gather + rotate, gate|up, SwiGLU, down, return -> (every rank has returned) -> weighted sum in
        slot order, residual, norm, rotation."""
        cfg, a = self.cfg, self.a2a
        Lib = _lib.load()
        st = _lib.stream_ptr()
        k, d, F, E = cfg.top_k, cfg.d_model, cfg.expert_ffn, cfg.n_experts
        cap = self.pairs_cap[cls]
        desc = a.desc(li)
        if M * k > desc.cap:
            raise ValueError(f"{M} rows x {k} picks exceed the {desc.cap}-pair all-to-all regions")
        _lib.check(Lib.rx_moe_a2a_dispatch(xn.data_ptr(), self.pick_ids.data_ptr(), M * k, k, self.status.data_ptr(), ctypes.byref(desc), st), "rx_moe_a2a_dispatch")
        yield          # every rank's rows must be on their way before any rank waits for them
        recv_pairs = a.R * desc.cap
        if recv_pairs > cap:
            raise ValueError(f"the expert buffers hold {cap} pairs, the all-to-all may deliver {recv_pairs}")
        _lib.check(Lib.rx_moe_a2a_recv_ids(self.recv_ids.data_ptr(), self.status.data_ptr(), ctypes.byref(desc), st), "rx_moe_a2a_recv_ids")
        _lib.check(Lib.rx_moe_plan(self.recv_ids.data_ptr(), recv_pairs, E, self.e_lo, self.e_hi, tile_rows, max_tiles, self.offs.data_ptr(),
                                   self.pos_of_pair.data_ptr(), self.pair_of_pos.data_ptr(), self.expert_of_pos.data_ptr(), self.tile_tab.data_ptr(),
                                   self.total.data_ptr(), st), "rx_moe_plan")
        gu, dn = L["gu"], L["down"]
        # a received row is a "pair" of its own (one slot per row): the flat receive index addresses the row
        _lib.check(Lib.rx_moe_gather_rot(ctypes.c_void_p(a.rx_rows_ptr(li)), self.recv_ids.data_ptr(), self.pos_of_pair.data_ptr(), recv_pairs, 1, d,
                                         ctypes.c_void_p(gu.suh.data_ptr() - 2 * self.e_lo * gu.K), self.xs.data_ptr(), st), "rx_moe_gather_rot")
        s_gu, s_dn = self.moe_splits[cls]
        self._grouped_shifted(self.xs, gu, s_gu, max_tiles, tile_rows, cap)
        act_rot = Lib.rx_moe_relu2_rot if cfg.expert_act == "relu2" else Lib.rx_moe_swiglu_rot
        _lib.check(act_rot(self.part.data_ptr(), s_gu, cap, F, self.expert_of_pos.data_ptr(), self.total.data_ptr(),
                           ctypes.c_void_p(gu.svh.data_ptr() - 2 * self.e_lo * gu.N), ctypes.c_void_p(dn.suh.data_ptr() - 2 * self.e_lo * dn.K),
                           self.xs2.data_ptr(), st), "rx_moe_act_rot")
        self._grouped_shifted(self.xs2, dn, s_dn, max_tiles, tile_rows, cap)
        _lib.check(Lib.rx_moe_a2a_return(self.part.data_ptr(), s_dn, cap, self.pair_of_pos.data_ptr(), self.expert_of_pos.data_ptr(), self.total.data_ptr(),
                                         ctypes.c_void_p(dn.svh.data_ptr() - 2 * self.e_lo * dn.N), ctypes.byref(desc), st), "rx_moe_a2a_return")
        yield          # every rank's results must be on their way home before any rank sums them
        _lib.check(Lib.rx_moe_a2a_home(self.pick_w.data_ptr(), M, k, None, self.slot.data_ptr(), self.status.data_ptr(), ctypes.byref(desc), st), "rx_moe_a2a_home")
        _lib.check(Lib.rx_tp_allsum_add_norm_rot(self.slot.data_ptr(), None, 1, self._dst.rows_cap, None, 0, M, d, h.data_ptr(), next_norm.data_ptr(), cfg.eps,
                                                 next_suh.data_ptr(), xr_d.data_ptr(), self.status.data_ptr(), st, None), "rx_tp_allsum_add_norm_rot")
        _lib.count(10)

    def _grouped_shifted(self, xs, st: _ExpertStack, splits, max_tiles, tile_rows, cap):
        """The tile table names GLOBAL expert ids; the stack starts at expert e_lo."""
        L = _lib.load()
        base = st.trellis.data_ptr() - 2 * self.e_lo * st.expert_elems
        if splits * cap * st.N > self.part.numel():
            raise _lib.KernelError(f"grouped GEMM partials ({splits} x {cap} x {st.N}) exceed the scratch buffer")
        _lib.check(L.rx_exl3_gemm_grouped(xs.data_ptr(), cap, st.K, ctypes.c_void_p(base), st.expert_elems, st.N, st.twice,
                                          self.K.CB_ID[st.codebook], self.part.data_ptr(), splits, self.tile_tab.data_ptr(), max_tiles, tile_rows,
                                          self.status.data_ptr(), _lib.stream_ptr()), "rx_exl3_gemm_grouped")

    def _combine_target(self, li, M):
        """-> (CombineDst, all-reduce slots pointer, flags pointer or None, ranks, rows_cap, epoch pointer, use index)."""
        if self.ep is None:
            return self._dst, self.slot.data_ptr(), None, 1, self._dst.rows_cap, None, 0
        return self.ep.combine_target(li, M)
