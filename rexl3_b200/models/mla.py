"""MLA + MoE decoder (DeepSeek-V3 shape: 61 layers, d_model 7168, 128 heads, q_lora 1536, kv_lora 512, rope 64, nope 128, v 128;
3 dense layers of FFN 18432, then 256 routed experts of FFN 2048 top-8 with a sigmoid+bias router and one shared expert).
Attention and shared weights are EXL3 (2.25 bpw = a mix of 2.0 and 2.5 bit tensors), routed experts MXFP4.

Per layer on the GPU:
  fused q_a | kv_a EXL3 GEMM (the 576-wide kv_a is padded to 640 columns with zero scales; EXL3 needs multiples of 128) ->
  row kernel (q_a RMSNorm + q_b's rotation; latent RMSNorm + RoPE into the paged latent cache) -> q_b EXL3 GEMM -> RoPE of the
  rope part, per-head absorb GEMM (q_nope @ W_uk) -> split-KV latent attention -> per-head expand GEMM (@ W_uv) -> o_proj
  rotation -> o_proj EXL3 GEMM -> residual / norm -> dense SwiGLU FFN, or: router -> plan -> MXFP4 grouped gate|up -> SwiGLU ->
  MXFP4 grouped down -> weighted sum + shared expert -> residual / norm.
Parallel form: heads [h_lo, h_hi) and experts [e_lo, e_hi) live on this rank; the o_proj partial rows and the MoE partial rows
are exchanged with the one-shot all-reduce (replicated residual stream, replicated latent cache).
Semantics: reference crates/cuda/csrc/mla_gated.cu, ling_mla_attn.cu, glm_p2_mla.cu (MLA), moe_router.cu:3-13, fp4_linear.cu:5-18.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field

import numpy as np
import torch

from ..format import exl3, mxfp4
from ..ops import kernels as K
from ..ops import lib as _lib
from .dense import PAGE, HostLinear, _bf16_round, random_linear
from .moe import CombineDst, route_reference

DSA_H, DSA_D, DSA_P = 32, 128, 4            # index heads, index head dim, tokens per pool (the kernels' geometry)
DSA_GROUP = 128                             # sparse rows selected / gathered / attended per launch group
DSA_COL_K, DSA_COL_G, DSA_COL_W = 2176, 2304, 2432


@dataclass
class MlaConfig:
    n_layers: int = 61
    n_dense: int = 3
    d_model: int = 7168
    n_heads: int = 128
    q_lora: int = 1536
    kv_lora: int = 512
    rope_dim: int = 64
    nope_dim: int = 128
    v_dim: int = 128
    dense_ffn: int = 18432
    n_experts: int = 256
    top_k: int = 8
    expert_ffn: int = 2048
    shared_ffn: int = 2048
    routed_scale: float = 2.5
    n_group: int = 0           # group-limited routing (DeepSeek-V3: 8 groups, a token keeps its 4 best); 0 = every expert competes
    topk_group: int = 0
    vocab: int = 129280
    eps: float = 1e-6
    rope_theta: float = 1e4
    bits_a: float = 2.0        # 2.25 bpw overall: the big projections at 2.0 ...
    bits_b: float = 2.5        # ... and the small / sensitive ones at 2.5 (half widths use the mul1 codebook)
    name: str = "mla-moe-671b"
    # sparse attention (DeepSeek sparse attention with pooled index keys, reference crates/cuda/csrc/dsa.cuh:1-16): 32 index heads x 128, 4-token
    # pools; a row with more than `dsa_dense_below` tokens of context attends to its `dsa_sel_pools` best pools (+ the incomplete last pool) only
    dsa: bool = False
    dsa_sel_pools: int = 512
    dsa_dense_below: int = 2048

    @property
    def a_width(self):
        """Columns of the fused q_a | kv_a projection: 1536 | 512 | 64 | pad 64, then with the indexer: key 128 | gate 128 | head weights 32 | pad 96."""
        return 2176 + (384 if self.dsa else 0)

    @property
    def qb_extra(self):
        """Index-query columns appended to q_b (32 heads x 128), replicated on every head-parallel rank."""
        return DSA_H * DSA_D if self.dsa else 0

    @property
    def vocab_padded(self):
        return (self.vocab + 127) // 128 * 128

    def kv_bytes_per_token(self):
        return 9 * 64 * 2 * self.n_layers


def config_from_dict(c: dict) -> MlaConfig:
    """MLA + MoE configuration from a config.json dictionary (this repository's `rexl3_mla_moe` packs; DeepSeek-V3 key names)."""
    q = c.get("quantization_config") or {}
    if q.get("quant_method") != "exl3":
        raise ValueError("config.json has no quantization_config with quant_method exl3")
    cfg = MlaConfig(n_layers=c["num_hidden_layers"], n_dense=int(c.get("first_k_dense_replace", 0)), d_model=c["hidden_size"], n_heads=c["num_attention_heads"],
                    q_lora=int(c.get("q_lora_rank", 1536)), kv_lora=int(c.get("kv_lora_rank", 512)), rope_dim=int(c.get("qk_rope_head_dim", 64)),
                    nope_dim=int(c.get("qk_nope_head_dim", 128)), v_dim=int(c.get("v_head_dim", 128)), dense_ffn=int(c.get("intermediate_size", 18432)),
                    n_experts=int(c.get("n_routed_experts", 256)), top_k=int(c.get("num_experts_per_tok", 8)), expert_ffn=int(c.get("moe_intermediate_size", 2048)),
                    shared_ffn=int(c.get("moe_intermediate_size", 2048)) * int(c.get("n_shared_experts", 1)), routed_scale=float(c.get("routed_scaling_factor", 2.5)),
                    n_group=int(c.get("n_group", 0) or 0), topk_group=int(c.get("topk_group", 0) or 0),
                    vocab=c["vocab_size"], eps=c.get("rms_norm_eps", 1e-6), rope_theta=c.get("rope_theta", 1e4), bits_a=float(q.get("bits_a", 2.0)),
                    bits_b=float(q.get("bits_b", 2.5)), name=c.get("name", "mla-moe"), dsa=bool(c.get("index_topk")) and bool(c.get("index_kpool", 4)),
                    dsa_sel_pools=int(c.get("index_topk", 2048)) // DSA_P, dsa_dense_below=int(c.get("index_dense_below", c.get("index_topk", 2048))))
    if cfg.dsa and (int(c.get("index_n_heads", DSA_H)), int(c.get("index_head_dim", DSA_D)), int(c.get("index_kpool", DSA_P))) != (DSA_H, DSA_D, DSA_P):
        raise ValueError("the sparse-attention indexer kernels are written for 32 index heads x 128 with 4-token pools")
    if (cfg.q_lora, cfg.kv_lora, cfg.rope_dim, cfg.nope_dim, cfg.v_dim) != (1536, 512, 64, 128, 128):
        raise ValueError(f"MLA geometry q_lora {cfg.q_lora} / kv_lora {cfg.kv_lora} / rope {cfg.rope_dim} / nope {cfg.nope_dim} / v {cfg.v_dim} "
                         f"is not the 1536 / 512 / 64 / 128 / 128 the latent attention kernels are written for")
    return cfg


CONFIGS = {
    "mla-moe-671b": MlaConfig(),
    "test-mla": MlaConfig(n_layers=3, n_dense=1, d_model=256, n_heads=16, dense_ffn=256, n_experts=8, top_k=2, expert_ffn=128, shared_ffn=128,
                          vocab=1024, name="test-mla"),
}
assert MlaConfig().q_lora == 1536 and MlaConfig().kv_lora == 512 and MlaConfig().rope_dim == 64      # the row kernel is written for these


@dataclass
class HostMlaLayer:
    attn_norm: np.ndarray
    qkv_a: HostLinear            # d -> 1536 | 512 | 64 | pad 64
    q_norm: np.ndarray
    kv_norm: np.ndarray
    q_b: HostLinear              # 1536 -> H * 192
    w_uk: np.ndarray             # f32 [H, 128, 512] (bf16-rounded)
    w_uv: np.ndarray             # f32 [H, 512, 128]
    o: HostLinear                # H * 128 -> d
    ffn_norm: np.ndarray
    gate_up: HostLinear = None   # dense layers, or the shared expert of a routed layer
    down: HostLinear = None
    router: np.ndarray = None
    router_bias: np.ndarray = None
    ex_gu: list = field(default_factory=list)     # per expert (packed uint8 [2F, d/2], scales uint8 [2F, d/32])
    ex_down: list = field(default_factory=list)   # per expert (packed uint8 [d, F/2], scales uint8 [d, F/32])
    idx_ln_w: np.ndarray = None  # sparse indexer: LayerNorm weight / bias of the index key (f32 [128]) ...
    idx_ln_b: np.ndarray = None
    idx_ape: np.ndarray = None   # ... and the pool-member bias of the gate softmax (f32 [4, 128])


@dataclass
class HostMla:
    cfg: MlaConfig
    embed: np.ndarray
    layers: list
    final_norm: np.ndarray
    lm_head: HostLinear


def random_mla_weights(cfg: MlaConfig, seed: int = 0) -> HostMla:
    rng = np.random.default_rng(seed)
    d, H = cfg.d_model, cfg.n_heads
    nrm = lambda n: _bf16_round(1.0 + 0.1 * rng.normal(size=n))  # noqa: E731
    layers = []
    for li in range(cfg.n_layers):
        qkv_a = random_linear(d, cfg.a_width, cfg.bits_b, rng, "mul1", 1.0 / math.sqrt(d), zero_cols_from=None if cfg.dsa else 2112)
        q_b = random_linear(1536, H * 192 + cfg.qb_extra, cfg.bits_a, rng, "3inst", 1.0 / math.sqrt(1536))
        o = random_linear(H * 128, d, cfg.bits_a, rng, "3inst", 0.5 / math.sqrt(H * 128))
        lay = HostMlaLayer(nrm(d), qkv_a, nrm(1536), nrm(512), q_b, _bf16_round(rng.normal(0, 1 / math.sqrt(128), size=(H, 128, 512))),
                           _bf16_round(rng.normal(0, 1 / math.sqrt(512), size=(H, 512, 128))), o, nrm(d))
        if cfg.dsa:
            lay.idx_ln_w = (1.0 + 0.1 * rng.normal(size=DSA_D)).astype(np.float32)
            lay.idx_ln_b = (0.1 * rng.normal(size=DSA_D)).astype(np.float32)
            lay.idx_ape = (0.5 * rng.normal(size=(DSA_P, DSA_D))).astype(np.float32)
        if li < cfg.n_dense:
            F = cfg.dense_ffn
            lay.gate_up = random_linear(d, 2 * F, cfg.bits_a, rng, "3inst", 1.0 / math.sqrt(d))
            lay.down = random_linear(F, d, cfg.bits_b, rng, "mul1", 0.5 / math.sqrt(F))
        else:
            F, Fs = cfg.expert_ffn, cfg.shared_ffn
            lay.gate_up = random_linear(d, 2 * Fs, cfg.bits_a, rng, "3inst", 1.0 / math.sqrt(d))
            lay.down = random_linear(Fs, d, cfg.bits_b, rng, "mul1", 0.5 / math.sqrt(Fs))
            lay.router = _bf16_round(rng.normal(0, 1.0 / math.sqrt(d), size=(cfg.n_experts, d)))
            lay.router_bias = rng.normal(0, 0.1, size=cfg.n_experts).astype(np.float32)
            for _ in range(cfg.n_experts):
                lay.ex_gu.append(mxfp4.quantize(rng.normal(0, 1.0 / math.sqrt(d), size=(2 * F, d)).astype(np.float32)))
                lay.ex_down.append(mxfp4.quantize(rng.normal(0, 0.5 / math.sqrt(F), size=(d, F)).astype(np.float32)))
        layers.append(lay)
    head = random_linear(d, cfg.vocab_padded, cfg.bits_b, rng, "mul1", 1.0 / math.sqrt(d), zero_cols_from=cfg.vocab if cfg.vocab_padded != cfg.vocab else None)
    return HostMla(cfg, _bf16_round(rng.normal(0, 1.0, size=(cfg.vocab, d)).astype(np.float32)), layers, nrm(d), head)


def mla_inv_freq(cfg: MlaConfig) -> np.ndarray:
    i = np.arange(0, cfg.rope_dim, 2, dtype=np.float32)
    return (1.0 / (np.float32(cfg.rope_theta) ** (i / np.float32(cfg.rope_dim)))).astype(np.float32)


class ReferenceMla:
    """fp32 oracle (non-absorbed arithmetic order is not required: the absorbed form is algebraically the same and is what runs)."""

    def __init__(self, w: HostMla, device="cpu"):
        self.cfg, self.device = w.cfg, device
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)  # noqa: E731
        self.embed = t(w.embed)
        self.layers = []
        for lay in w.layers:
            L = dict(attn_norm=t(lay.attn_norm), qkv_a=t(lay.qkv_a.dense()), q_norm=t(lay.q_norm), kv_norm=t(lay.kv_norm), q_b=t(lay.q_b.dense()),
                     w_uk=t(lay.w_uk), w_uv=t(lay.w_uv), o=t(lay.o.dense()), ffn_norm=t(lay.ffn_norm), gate_up=t(lay.gate_up.dense()),
                     down=t(lay.down.dense()), router=None)
            if w.cfg.dsa:
                L.update(idx_ln_w=t(lay.idx_ln_w), idx_ln_b=t(lay.idx_ln_b), idx_ape=t(lay.idx_ape))
            if lay.router is not None:
                L.update(router=t(lay.router), router_bias=t(lay.router_bias), gu=[t(mxfp4.dequant(*e)) for e in lay.ex_gu],
                         dn=[t(mxfp4.dequant(*e)) for e in lay.ex_down])
            self.layers.append(L)
        self.final_norm = t(w.final_norm)
        self.lm_head = t(w.lm_head.dense())[:, :w.cfg.vocab]
        self.inv_freq = torch.from_numpy(mla_inv_freq(w.cfg)).to(device)
        self.kv = {}
        self.idx = {}          # sparse indexer: per sequence and layer the (key, gate) rows of every token
        self.last_selection = {}

    def _dsa_allowed(self, seq, li, L, a, q_idx, pos, start):
        """-> bool [T, keys]: which keys each row of the sparse regime may attend to (None: every row is dense).  Planes and scores are rounded to
        the storage types of the device path (bf16 planes, fp16 scores) so that ties fall the same way."""
        cfg = self.cfg
        bf = lambda x: x.to(torch.bfloat16).float()  # noqa: E731
        k_n = bf(torch.nn.functional.layer_norm(bf(a[:, DSA_COL_K:DSA_COL_K + DSA_D]), (DSA_D,), L["idx_ln_w"], L["idx_ln_b"], 1e-6))
        gate = bf(a[:, DSA_COL_G:DSA_COL_G + DSA_D])
        wh = bf(a[:, DSA_COL_W:DSA_COL_W + DSA_H])
        pk, pg = self.idx.setdefault(seq, {}).get(li, (k_n[:0], gate[:0]))
        kk, gg = torch.cat([pk[:start], k_n]), torch.cat([pg[:start], gate])
        self.idx[seq][li] = (kk, gg)
        if int(pos[-1]) + 1 <= cfg.dsa_dense_below:
            return None
        n_pools = kk.shape[0] // DSA_P
        km, gm = kk[:n_pools * DSA_P].view(n_pools, DSA_P, DSA_D), gg[:n_pools * DSA_P].view(n_pools, DSA_P, DSA_D)
        pooled = bf((torch.softmax(gm + L["idx_ape"][None], dim=1) * km).sum(1))                          # [pools, 128]
        T, n_keys = a.shape[0], kk.shape[0]
        allowed = torch.ones(T, n_keys, dtype=torch.bool, device=a.device)
        for t in range(T):
            p = int(pos[t])
            if p + 1 <= cfg.dsa_dense_below:
                continue
            vis = (p + 1) // DSA_P
            dots = torch.relu(bf(q_idx[t]) @ pooled[:vis].T)                                               # [32, vis]
            sc = ((dots * wh[t][:, None]).sum(0) / math.sqrt(DSA_H * DSA_D)).to(torch.float16)
            order = torch.sort(sc.float(), descending=True, stable=True).indices[:cfg.dsa_sel_pools]      # ties: lowest pool index first
            pools = torch.sort(order).values
            toks = (pools[:, None] * DSA_P + torch.arange(DSA_P, device=a.device)[None]).reshape(-1)
            toks = torch.cat([toks, torch.arange(vis * DSA_P, p + 1, device=a.device)])
            allowed[t] = False
            allowed[t, toks] = True
            self.last_selection[(seq, li, p)] = toks.tolist()
        return allowed

    @staticmethod
    def _rms(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def _rope(self, x, pos):
        ang = pos.to(torch.float32)[:, None] * self.inv_freq[None, :]
        cos, sin = torch.cos(ang), torch.sin(ang)
        while cos.dim() < x.dim():
            cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        x1, x2 = x[..., :32], x[..., 32:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    @torch.no_grad()
    def forward_seq(self, seq, tokens, start: int) -> torch.Tensor:
        cfg = self.cfg
        ids = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        T, H = ids.shape[0], cfg.n_heads
        pos = torch.arange(start, start + T, device=self.device)
        h = self.embed[ids]
        if seq not in self.kv:
            self.kv[seq] = [(torch.zeros(0, 512, device=self.device), torch.zeros(0, 64, device=self.device)) for _ in self.layers]
        for li, L in enumerate(self.layers):
            x = self._rms(h, L["attn_norm"], cfg.eps)
            a = x @ L["qkv_a"]
            qb_out = self._rms(a[:, :1536], L["q_norm"], cfg.eps) @ L["q_b"]
            q = qb_out[:, :H * 192].view(T, H, 192)
            allowed = self._dsa_allowed(seq, li, L, a, qb_out[:, H * 192:].view(T, DSA_H, DSA_D), pos, start) if cfg.dsa else None
            c = self._rms(a[:, 1536:2048], L["kv_norm"], cfg.eps)
            kr = self._rope(a[:, 2048:2112], pos)
            pc, pr = self.kv[seq][li]
            cc, rr = torch.cat([pc[:start], c]), torch.cat([pr[:start], kr])
            self.kv[seq][li] = (cc, rr)
            q_lat = torch.einsum("thk,hkc->thc", q[..., :128], L["w_uk"])
            q_rope = self._rope(q[..., 128:], pos)
            s = (torch.einsum("thc,sc->hts", q_lat, cc) + torch.einsum("thr,sr->hts", q_rope, rr)) / math.sqrt(192)
            kpos = torch.arange(cc.shape[0], device=self.device)
            s = s.masked_fill((kpos[None, :] > pos[:, None])[None], float("-inf"))
            if allowed is not None:
                s = s.masked_fill(~allowed[None], float("-inf"))
            o_lat = torch.einsum("hts,sc->thc", torch.softmax(s, dim=-1), cc)
            o = torch.einsum("thc,hcv->thv", o_lat, L["w_uv"]).reshape(T, H * 128)
            h = h + o @ L["o"]
            x = self._rms(h, L["ffn_norm"], cfg.eps)
            gu = x @ L["gate_up"]
            F = gu.shape[1] // 2
            y = (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ L["down"]
            if L["router"] is not None:
                mc = _RouteCfg(cfg)
                ids_e, wts = route_reference(x @ L["router"].T, mc, L["router_bias"], cfg.n_group, cfg.topk_group)
                Fe = cfg.expert_ffn
                for t in range(T):
                    for j in range(cfg.top_k):
                        e = int(ids_e[t, j])
                        g = L["gu"][e] @ x[t]
                        y[t] += wts[t, j] * (L["dn"][e] @ (torch.nn.functional.silu(g[:Fe]) * g[Fe:]))
            h = h + y
        return (self._rms(h, self.final_norm, cfg.eps) @ self.lm_head).float()


class _RouteCfg:
    def __init__(self, cfg):
        self.router_mode, self.top_k, self.routed_scale = "sigmoid_bias", cfg.top_k, cfg.routed_scale


class _Local:
    """One-rank stand-in for the exchange object: both collectives write a local slot."""

    def __init__(self, rows_cap, d, device):
        self.slot = torch.zeros(rows_cap, d, dtype=torch.float32, device=device)
        self.dst = CombineDst()
        self.dst.ranks, self.dst.rank, self.dst.rows_cap = 1, 0, rows_cap
        self.dst.dst[0] = self.slot.data_ptr()
        self.rows_cap = rows_cap

    def begin(self):
        pass

    def target(self, use, M):
        return self.dst, self.slot.data_ptr(), None, 1, self.rows_cap, None, 0


class MlaMoEGPU:
    def __init__(self, w: "HostMla | MlaConfig", num_pages: int, max_rows: int = 256, max_seqs: int = 64, max_blocks_per_seq: int = 256, device="cuda",
                 max_prefill_rows: int = 4096, seed: int = 0, heads=None, experts=None, comm=None, rank: int = 0, expert_paging=None):
        """`expert_paging` = dict(path=FILE, budget_bytes=N[, fill_threads, direct]): the routed MXFP4 experts stay in a record file (written from
        the host weights when it is not there yet) and are paged into a device slab of N bytes as the router asks for them
        (models/expert_paging.py); one rank, weights from host tensors.  Each routed layer then reads its picks on the host."""
        self.K = K
        self.paged = None
        self._paging = expert_paging
        if expert_paging is not None and (isinstance(w, MlaConfig) or heads is not None or experts is not None or comm is not None):
            raise ValueError("expert paging runs on one rank that owns every head and expert, over host weights")
        self.device = device
        self.cfg = cfg = w if isinstance(w, MlaConfig) else w.cfg
        self.h_lo, self.h_hi = heads or (0, cfg.n_heads)
        self.e_lo, self.e_hi = experts or (0, cfg.n_experts)
        self.Hl = self.h_hi - self.h_lo
        self.rank = rank
        if self.Hl % 16:
            raise ValueError("a rank must own a multiple of 16 heads")
        self.num_pages, self.max_seqs, self.max_blocks = num_pages, max_seqs, max_blocks_per_seq
        self.max_rows = R = max(max_rows, max_prefill_rows)
        self.max_ctx_alloc = max_blocks_per_seq * PAGE
        if isinstance(w, MlaConfig):
            self._load_random(seed)
        else:
            self._load_host(w)
        self.inv_freq = torch.from_numpy(mla_inv_freq(cfg)).to(device)
        self.cache = [torch.zeros(num_pages, 9, PAGE, 64, dtype=torch.bfloat16, device=device) for _ in range(cfg.n_layers)]
        self.tc = [K.KvTensorMap(c) for c in self.cache]
        self.status = K.new_status(device)
        self.local = _Local(R, cfg.d_model, device)       # dense FFN layers are computed on every rank: their sum needs no exchange
        self.comm = comm or self.local
        self._alloc(R)

    # ------------------------------------------------------------------ weights
    def _load_host(self, w: HostMla):
        dev = self.device
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=dev, dtype=dt)  # noqa: E731
        up = lambda l: K.Exl3Weight.from_numpy(l.trellis, l.suh, l.svh, l.bias, l.codebook, dev)  # noqa: E731
        hl, hh, el, eh = self.h_lo, self.h_hi, self.e_lo, self.e_hi
        self.embed = t(w.embed, torch.bfloat16)
        self.layers = []
        slab = None
        if self._paging is not None:
            from . import expert_paging as xp
            pg = dict(self._paging)
            layout = xp.write_mx_records(w, pg.pop("path"), tag=pg.pop("tag", ""))
            self.paged = xp.PagedExperts(layout, pg.pop("budget_bytes"), dev, **pg)
            slab = self.paged.slab.t          # every routed layer reads "its experts" from the same slab, through slot ids
        for lay in w.layers:
            qb = lay.q_b
            H = self.cfg.n_heads      # this rank's heads, then (sparse attention) the index-query columns every rank keeps
            qb_l = HostLinear(np.ascontiguousarray(np.concatenate([qb.trellis[:, hl * 12:hh * 12], qb.trellis[:, H * 12:]], axis=1)), qb.suh,
                              np.ascontiguousarray(np.concatenate([qb.svh[hl * 192:hh * 192], qb.svh[H * 192:]])), None, qb.codebook)
            o = lay.o
            o_l = HostLinear(np.ascontiguousarray(o.trellis[hl * 8:hh * 8]), np.ascontiguousarray(o.suh[hl * 128:hh * 128]), o.svh, None, o.codebook)
            L = dict(attn_norm=t(lay.attn_norm, torch.bfloat16), qkv_a=up(lay.qkv_a), q_norm=t(lay.q_norm, torch.bfloat16), kv_norm=t(lay.kv_norm, torch.bfloat16),
                     q_b=up(qb_l), w_uk=t(lay.w_uk[hl:hh], torch.bfloat16), w_uv=t(lay.w_uv[hl:hh], torch.bfloat16), o=up(o_l),
                     ffn_norm=t(lay.ffn_norm, torch.bfloat16), gate_up=up(lay.gate_up), down=up(lay.down), router=None)
            if self.cfg.dsa:
                L.update(idx_ln_w=t(lay.idx_ln_w, torch.float32), idx_ln_b=t(lay.idx_ln_b, torch.float32), idx_ape=t(lay.idx_ape, torch.float32))
            if lay.router is not None and slab is not None:
                L.update(router=t(lay.router, torch.bfloat16), router_bias=t(lay.router_bias, torch.float32),
                         gu_w=slab["gu_w"], gu_s=slab["gu_s"], dn_w=slab["dn_w"], dn_s=slab["dn_s"])
            elif lay.router is not None:
                L.update(router=t(lay.router, torch.bfloat16), router_bias=t(lay.router_bias, torch.float32),
                         gu_w=torch.from_numpy(np.stack([e[0].view(np.uint8) for e in lay.ex_gu[el:eh]])).to(dev),
                         gu_s=torch.from_numpy(np.stack([e[1] for e in lay.ex_gu[el:eh]])).to(dev),
                         dn_w=torch.from_numpy(np.stack([e[0].view(np.uint8) for e in lay.ex_down[el:eh]])).to(dev),
                         dn_s=torch.from_numpy(np.stack([e[1] for e in lay.ex_down[el:eh]])).to(dev))
            self.layers.append(L)
        self.final_norm = t(w.final_norm, torch.bfloat16)
        self.lm_head = up(w.lm_head)

    def _load_random(self, seed: int):
        """Random-init model on the device: shared tensors from `seed` (identical on every rank), this rank's heads and experts from
        rank-specific streams.  Random nibbles and scale bytes in a trained model's range are valid MXFP4."""
        cfg, dev = self.cfg, self.device
        g = torch.Generator(device=dev).manual_seed(seed)
        gl = torch.Generator(device=dev).manual_seed(seed * 7919 + 101 + self.h_lo * 131 + self.e_lo)
        d, Hl = cfg.d_model, self.Hl
        sg = lambda n, gen: (torch.randint(0, 2, (n,), device=dev, generator=gen) * 2 - 1)  # noqa: E731

        def lin(k, n, scale, bits, gen, suh=None):
            b = exl3.Bits.of(bits)
            tr = torch.randint(-32768, 32768, (k // 16, n // 16, b.tile_words), dtype=torch.int16, device=dev, generator=gen)
            su = sg(k, gen).to(torch.float16) if suh is None else suh
            return K.Exl3Weight(tr, su, (sg(n, gen) * scale).to(torch.float16), None, "3inst" if b.is_integer else "mul1")
        nrm = lambda n: (1.0 + 0.1 * torch.randn(n, device=dev, generator=g)).to(torch.bfloat16)  # noqa: E731

        def mx(e, n, k, amp):
            wq = torch.randint(0, 256, (e, n, k // 2), dtype=torch.uint8, device=dev, generator=gl)
            sc = torch.randint(0, 3, (e, n, k // 32), dtype=torch.uint8, device=dev, generator=gl) + int(127 + math.log2(amp)) - 3
            return wq, sc.to(torch.uint8)
        self.embed = torch.randn(cfg.vocab, d, device=dev, generator=g).to(torch.bfloat16)
        self.layers = []
        E = self.e_hi - self.e_lo
        for li in range(cfg.n_layers):
            qkv_a = lin(d, cfg.a_width, 1.0 / math.sqrt(d), cfg.bits_b, g)
            qkv_a.svh[2112:2176] = 0
            su_qb = sg(1536, g).to(torch.float16)
            L = dict(attn_norm=nrm(d), qkv_a=qkv_a, q_norm=nrm(1536), kv_norm=nrm(512),
                     q_b=lin(1536, Hl * 192 + cfg.qb_extra, 1.0 / math.sqrt(1536), cfg.bits_a, gl, su_qb),
                     w_uk=(torch.randn(Hl, 128, 512, device=dev, generator=gl) / math.sqrt(128)).to(torch.bfloat16),
                     w_uv=(torch.randn(Hl, 512, 128, device=dev, generator=gl) / math.sqrt(512)).to(torch.bfloat16),
                     o=lin(Hl * 128, d, 0.5 / math.sqrt(cfg.n_heads * 128), cfg.bits_a, gl), ffn_norm=nrm(d), router=None)
            if cfg.dsa:
                L.update(idx_ln_w=1.0 + 0.1 * torch.randn(DSA_D, device=dev, generator=g), idx_ln_b=0.1 * torch.randn(DSA_D, device=dev, generator=g),
                         idx_ape=0.5 * torch.randn(DSA_P, DSA_D, device=dev, generator=g))
            F = cfg.dense_ffn if li < cfg.n_dense else cfg.shared_ffn
            L["gate_up"] = lin(d, 2 * F, 1.0 / math.sqrt(d), cfg.bits_a, g)
            L["down"] = lin(F, d, 0.5 / math.sqrt(F), cfg.bits_b, g)
            if li >= cfg.n_dense:
                L["router"] = (torch.randn(cfg.n_experts, d, device=dev, generator=g) / math.sqrt(d)).to(torch.bfloat16)
                L["router_bias"] = 0.1 * torch.randn(cfg.n_experts, device=dev, generator=g)
                L["gu_w"], L["gu_s"] = mx(E, 2 * cfg.expert_ffn, d, 1.0 / math.sqrt(d))
                L["dn_w"], L["dn_s"] = mx(E, d, cfg.expert_ffn, 0.5 / math.sqrt(cfg.expert_ffn))
            self.layers.append(L)
        self.final_norm = nrm(d)
        self.lm_head = lin(d, cfg.vocab_padded, 1.0 / math.sqrt(d), cfg.bits_b, g)
        if cfg.vocab_padded != cfg.vocab:
            self.lm_head.svh[cfg.vocab:] = 0

    @staticmethod
    def weight_bytes_estimate(cfg: MlaConfig) -> float:
        """Bytes of the whole model (all heads, all experts) for the memory plan."""
        d, H = cfg.d_model, cfg.n_heads
        attn = (d * 2176 * cfg.bits_b + 1536 * H * 192 * cfg.bits_a + H * 128 * d * cfg.bits_a) / 8 + 2 * H * 128 * 512 * 2
        dense_ffn = 3 * d * cfg.dense_ffn * (2 * cfg.bits_a + cfg.bits_b) / 3 / 8
        routed = cfg.n_experts * 3 * d * cfg.expert_ffn * (0.5 + 1 / 32) + 3 * d * cfg.shared_ffn * (2 * cfg.bits_a + cfg.bits_b) / 3 / 8
        return cfg.n_layers * attn + cfg.n_dense * dense_ffn + (cfg.n_layers - cfg.n_dense) * routed + (cfg.vocab_padded * d * cfg.bits_b) / 8 + cfg.vocab * d * 2

    def weight_bytes(self) -> int:
        n = self.embed.numel() * 2 + self.lm_head.nbytes
        for L in self.layers:
            n += sum(L[k].nbytes for k in ("qkv_a", "q_b", "o", "gate_up", "down")) + (L["w_uk"].numel() + L["w_uv"].numel()) * 2
            if L["router"] is not None:
                n += L["router"].numel() * 2 + (0 if self.paged is not None else sum(L[k].numel() for k in ("gu_w", "gu_s", "dn_w", "dn_s")))
        return n + (self.paged.slab.nbytes() if self.paged is not None else 0)

    # ------------------------------------------------------------------ buffers
    def _alloc(self, R):
        cfg, dev = self.cfg, self.device
        d, Hl, k = cfg.d_model, self.Hl, cfg.top_k
        Rw = min(R, 256)
        self.splits = {}
        part = 0
        Fmax = max(cfg.dense_ffn, cfg.shared_ffn)
        shapes = dict(qkv_a=(d, cfg.a_width), q_b=(1536, Hl * 192 + cfg.qb_extra), o=(Hl * 128, d), gu_dense=(d, 2 * cfg.dense_ffn), dn_dense=(cfg.dense_ffn, d),
                      gu_sh=(d, 2 * cfg.shared_ffn), dn_sh=(cfg.shared_ffn, d), lm_head=(d, cfg.vocab_padded))
        for cls, rows in (("decode", Rw), ("prefill", R)):
            for name, (kk, nn) in shapes.items():
                s = K.plan_splits(kk, nn, cls == "decode")
                self.splits[(cls, name)] = s
                part = max(part, s * (rows if name != "lm_head" else Rw) * nn)
        self.pairs_cap = {"decode": Rw * k, "prefill": R * k}
        self.mx_splits = {"decode": (2, 2), "prefill": (1, 1)}
        for cls in ("decode", "prefill"):
            sg_, sd_ = self.mx_splits[cls]
            part = max(part, sg_ * self.pairs_cap[cls] * 2 * cfg.expert_ffn, sd_ * self.pairs_cap[cls] * d)
        self.part = torch.empty(part, dtype=torch.float32, device=dev)
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
        hf = lambda *s: torch.empty(*s, dtype=torch.float16, device=dev)  # noqa: E731
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)  # noqa: E731
        self.h, self.xn = bf(R, d), bf(R, d)
        self.xr_d = hf(R, d)
        self.a_out = bf(R, cfg.a_width)
        self.xr_q = hf(R, 1536)
        self.q_full = bf(R, Hl * 192 + cfg.qb_extra)
        if cfg.dsa:
            self._alloc_dsa(R)
        self.q = bf(R, Hl, 576)
        self.o_lat = bf(R, Hl, 512)
        self.o_heads = bf(R, Hl * 128)
        self.xr_o = hf(R, Hl * 128)
        self.xr_f = hf(R, Fmax)
        self.shared = torch.zeros(R, d, dtype=torch.float32, device=dev)
        self.logits = torch.empty(Rw, cfg.vocab_padded, dtype=torch.float32, device=dev)
        n_scratch = _lib.load().rx_mla_scratch_floats(R, Hl, self.max_ctx_alloc)
        if cfg.dsa:        # a group of sparse rows attends over its scratch pages: fewer rows, but up to 3 splits each
            n_scratch = max(n_scratch, _lib.load().rx_mla_scratch_floats(min(R, DSA_GROUP), Hl, self.dsa_pages * PAGE))
        self.attn_scratch = torch.empty(n_scratch, dtype=torch.float32, device=dev)
        self.pick_ids, self.pick_w = i32(R * k), torch.zeros(R * k, dtype=torch.float32, device=dev)
        E = cfg.n_experts
        S = self.paged.slots if self.paged is not None else 0            # paged experts: the kernels see slot ids, 0 .. S - 1
        self.offs, self.pos_of_pair, self.pair_of_pos, self.expert_of_pos, self.total = i32(max(E, S) + 1), i32(R * k), i32(R * k), i32(R * k), i32(1)
        El = max(self.e_hi - self.e_lo, S)      # the tile table only ever names owned experts (or slots)
        if S:
            self.pick_slot = i32(R * k)
            self.slot_table_h = torch.zeros(E, dtype=torch.int32).pin_memory()
            self.slot_table = i32(E)
        self.max_tiles = {"decode": El + (Rw * k + 31) // 32, "prefill": El + (R * k + 127) // 128}
        self.router_logits = torch.empty(R, E, dtype=torch.float32, device=dev)
        self.tile_tab = i32(3 * max(self.max_tiles.values()))
        self.xs = torch.zeros(R * k, d, dtype=torch.float16, device=dev)
        self.xs2 = torch.zeros(R * k, cfg.expert_ffn, dtype=torch.float16, device=dev)
        self.topk_scratch = K.topk_scratch(Rw, cfg.vocab_padded, 64, dev)
        self.cand_ids = torch.empty(Rw, 64, dtype=torch.int32, device=dev)
        self.cand_vals = torch.empty(Rw, 64, dtype=torch.float32, device=dev)

    def _alloc_dsa(self, R):
        """Planes and scratch of the sparse-attention indexer.  Per layer: the ring of each sequence's last tokens (key | gate rows) and the pooled
        keys (one 4 KB slab per latent-cache page: + 5.5 %).  Shared by the layers: this call's staging rows, the score / selection buffers of one
        row group and the scratch pages the selected latent rows are gathered into (33 pages per row at 512 pools)."""
        cfg, dev = self.cfg, self.device
        i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device=dev)  # noqa: E731
        if cfg.dsa_sel_pools < 1 or cfg.dsa_sel_pools > 8192:
            raise ValueError("dsa_sel_pools must be in 1..8192")
        self.dsa_ring_len = (min(R, 256) + DSA_P + DSA_P - 1) // DSA_P * DSA_P
        self.dsa_ring = [torch.zeros(self.max_seqs, self.dsa_ring_len, 2 * DSA_D, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]
        self.dsa_pool = [torch.zeros(self.num_pages, PAGE // DSA_P, DSA_D, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]
        self.dsa_stage = torch.zeros(R, 2 * DSA_D, dtype=torch.bfloat16, device=dev)
        self.dsa_s_stride = (self.max_ctx_alloc // DSA_P + 7) // 8 * 8
        self.dsa_k_stride = (cfg.dsa_sel_pools * DSA_P + DSA_P - 1 + 3) // 4 * 4
        self.dsa_pages = (self.dsa_k_stride + PAGE - 1) // PAGE
        G = min(R, DSA_GROUP)
        self.dsa_scores = torch.zeros(G, self.dsa_s_stride, dtype=torch.float16, device=dev)
        self.dsa_sel = i32(G, self.dsa_k_stride)
        self.dsa_flag, self.dsa_ctx = i32(R), i32(R)
        self.dsa_scratch = torch.zeros(G * self.dsa_pages, 9, PAGE, 64, dtype=torch.bfloat16, device=dev)
        self.dsa_tc = K.KvTensorMap(self.dsa_scratch)
        self.dsa_vbt = torch.arange(G * self.dsa_pages, dtype=torch.int32, device=dev).view(G, self.dsa_pages).contiguous()
        self.dsa_rowid = torch.arange(G, dtype=torch.int32, device=dev)

    def _dsa_sparse_rows(self, li, L, M, q_ld, block_table, row_seq, positions, ctx_cap):
        """Rows of the sparse regime: scores over the pooled keys, exact top-`sel_pools` selection, gather of the selected latent rows into the
        scratch pages, attention over those through the virtual block table; DSA_GROUP rows per launch group."""
        cfg, Lib, st, Hl = self.cfg, _lib.load(), _lib.stream_ptr, self.Hl
        max_pools = min(ctx_cap // DSA_P, self.dsa_s_stride)
        for g0 in range(0, M, DSA_GROUP):
            n = min(DSA_GROUP, M - g0)
            qi = self.q_full.data_ptr() + 2 * (g0 * q_ld + Hl * 192)
            _lib.check(Lib.rx_dsa_select(ctypes.c_void_p(qi), q_ld, ctypes.c_void_p(self.a_out.data_ptr() + 2 * g0 * cfg.a_width), cfg.a_width, DSA_COL_W,
                                         self.dsa_pool[li].data_ptr(), block_table.data_ptr(), block_table.shape[1], ctypes.c_void_p(row_seq.data_ptr() + 4 * g0),
                                         ctypes.c_void_p(positions.data_ptr() + 4 * g0), cfg.dsa_dense_below, 1.0 / math.sqrt(DSA_H * DSA_D), cfg.dsa_sel_pools,
                                         max_pools, self.dsa_scores.data_ptr(), self.dsa_s_stride, self.dsa_sel.data_ptr(), self.dsa_k_stride,
                                         ctypes.c_void_p(self.dsa_flag.data_ptr() + 4 * g0), ctypes.c_void_p(self.dsa_ctx.data_ptr() + 4 * g0), n, st()),
                       "rx_dsa_select")
            _lib.check(Lib.rx_dsa_gather(self.cache[li].data_ptr(), block_table.data_ptr(), block_table.shape[1], ctypes.c_void_p(row_seq.data_ptr() + 4 * g0),
                                         self.dsa_sel.data_ptr(), self.dsa_k_stride, ctypes.c_void_p(self.dsa_flag.data_ptr() + 4 * g0),
                                         ctypes.c_void_p(self.dsa_ctx.data_ptr() + 4 * g0), self.dsa_scratch.data_ptr(), self.dsa_pages, n, st()), "rx_dsa_gather")
            _lib.check(Lib.rx_mla_attn_sel(self.dsa_tc.ptr, ctypes.c_void_p(self.q.data_ptr() + 2 * g0 * Hl * 576), self.dsa_vbt.data_ptr(), self.dsa_pages,
                                           self.dsa_rowid.data_ptr(), ctypes.c_void_p(self.dsa_ctx.data_ptr() + 4 * g0), self.attn_scratch.data_ptr(), n, Hl,
                                           self.dsa_pages * PAGE, 1.0 / math.sqrt(192), ctypes.c_void_p(self.o_lat.data_ptr() + 2 * g0 * Hl * 512),
                                           self.status.data_ptr(), ctypes.c_void_p(self.dsa_flag.data_ptr() + 4 * g0), 1, st()), "rx_mla_attn_sel")
            _lib.count(5)

    def _lin(self, xr, w, cls, name):
        s = self.splits[(cls, name)]
        K.exl3_gemm(xr, w, self.part, s, self.status)
        return s

    def _allsum(self, tgt, M, h, norm_w, suh_next, xr_out, xn_out=None):
        dst, ar, flags, ranks, rows_cap, epoch, use = tgt
        _lib.check(_lib.load().rx_tp_allsum_add_norm_rot(ar, flags, ranks, rows_cap, epoch, use, M, self.cfg.d_model, h.data_ptr(), norm_w.data_ptr(),
                                                         self.cfg.eps, _lib.ptr(suh_next), _lib.ptr(xr_out), self.status.data_ptr(), _lib.stream_ptr(),
                                                         _lib.ptr(xn_out)), "rx_tp_allsum_add_norm_rot")
        _lib.count()

    # ------------------------------------------------------------------ forward
    def forward_rows(self, *a, **kw):
        g = self.forward_phases(*a, **kw)
        try:
            while True:
                next(g)
        except StopIteration as e:
            return e.value

    def forward_phases(self, ids, positions, slots, row_seq, ctx_len, block_table, *, prefill=None, logit_rows=None, max_ctx=None, want_logits=True,
                       n_layers=None):
        cfg = self.cfg
        Lib = _lib.load()
        st = _lib.stream_ptr
        M = ids.shape[0]
        cls = "decode" if (prefill is None and M <= 256) else "prefill"
        d, Hl, k, E = cfg.d_model, self.Hl, cfg.top_k, cfg.n_experts
        multi = not isinstance(self.comm, _Local)
        h, xn, xr_d = self.h[:M], self.xn[:M], self.xr_d[:M]
        a_out, xr_q, q_full, q, o_lat, o_heads, xr_o = self.a_out[:M], self.xr_q[:M], self.q_full[:M], self.q[:M], self.o_lat[:M], self.o_heads[:M], self.xr_o[:M]
        ctx_cap = max_ctx or self.max_ctx_alloc
        self.comm.begin()
        K.embed(ids, self.embed, h)
        K.norm_rot_in(h, self.layers[0]["attn_norm"], cfg.eps, self.layers[0]["qkv_a"].suh, xr_d)
        nl = n_layers or len(self.layers)
        use = 0        # collectives are numbered in launch order: consecutive ones alternate between the two slot sets
        q_ld = Hl * 192 + cfg.qb_extra
        sparse = cfg.dsa and ctx_cap > cfg.dsa_dense_below      # no row of this call can be in the sparse regime otherwise
        for li in range(nl):
            L = self.layers[li]
            s = self._lin(xr_d, L["qkv_a"], cls, "qkv_a")
            K.finish_store(self.part, s, M, L["qkv_a"], a_out)
            _lib.check(Lib.rx_mla_row_ld(a_out.data_ptr(), cfg.a_width, L["q_norm"].data_ptr(), L["kv_norm"].data_ptr(), cfg.eps, L["q_b"].suh.data_ptr(),
                                         positions.data_ptr(), self.inv_freq.data_ptr(), slots.data_ptr(), xr_q.data_ptr(), self.cache[li].data_ptr(), M, st()),
                       "rx_mla_row")
            if cfg.dsa:
                _lib.check(Lib.rx_dsa_append(a_out.data_ptr(), cfg.a_width, DSA_COL_K, DSA_COL_G, L["idx_ln_w"].data_ptr(), L["idx_ln_b"].data_ptr(), 1e-6,
                                             L["idx_ape"].data_ptr(), row_seq.data_ptr(), positions.data_ptr(), block_table.data_ptr(),
                                             block_table.shape[1], self.dsa_stage.data_ptr(), self.dsa_ring[li].data_ptr(), self.dsa_ring_len,
                                             self.dsa_pool[li].data_ptr(), M, st()), "rx_dsa_append")
                _lib.count(3)
            s = self._lin(xr_q, L["q_b"], cls, "q_b")
            K.finish_store(self.part, s, M, L["q_b"], q_full)
            _lib.check(Lib.rx_mla_q_rope_ld(q_full.data_ptr(), q_ld, positions.data_ptr(), self.inv_freq.data_ptr(), Hl, q.data_ptr(), M, st()), "rx_mla_q_rope")
            _lib.check(Lib.rx_head_gemm(q_full.data_ptr(), q_ld, 192, L["w_uk"].data_ptr(), Hl, 128, 512, q.data_ptr(), Hl * 576, 576, M, st()), "absorb")
            if sparse:
                self._dsa_sparse_rows(li, L, M, q_ld, block_table, row_seq, positions, ctx_cap)
            _lib.check(Lib.rx_mla_attn_sel(self.tc[li].ptr, q.data_ptr(), block_table.data_ptr(), block_table.shape[1], row_seq.data_ptr(), ctx_len.data_ptr(),
                                           self.attn_scratch.data_ptr(), M, Hl, ctx_cap, 1.0 / math.sqrt(192), o_lat.data_ptr(), self.status.data_ptr(),
                                           self.dsa_flag.data_ptr() if sparse else None, 0, st()), "rx_mla_attn")
            _lib.check(Lib.rx_head_gemm(o_lat.data_ptr(), Hl * 512, 512, L["w_uv"].data_ptr(), Hl, 512, 128, o_heads.data_ptr(), Hl * 128, 128, M, st()), "expand")
            _lib.count(6)
            K.norm_rot_in(o_heads, None, cfg.eps, L["o"].suh, xr_o)
            s = self._lin(xr_o, L["o"], cls, "o")
            # o_proj partial rows -> every rank's slot, then residual + ffn norm (+ the rotation of the dense / shared FFN input)
            use += 1
            tgt = self.comm.target(use, M)
            _lib.check(Lib.rx_tp_finish_bcast(self.part.data_ptr(), s, M, d, L["o"].svh.data_ptr(), None, ctypes.byref(tgt[0]), st()), "rx_tp_finish_bcast") \
                if multi else self._finish_local(s, M, L["o"], tgt)
            if multi:
                yield
            routed = L["router"] is not None
            self._allsum(tgt, M, h, L["ffn_norm"], L["gate_up"].suh, xr_d, xn if routed else None)
            # dense FFN or shared expert
            F = L["gate_up"].N // 2
            run_shared = (not routed) or (not multi) or self.rank == 0
            gname, dname = ("gu_sh", "dn_sh") if routed else ("gu_dense", "dn_dense")
            xr_f = self.xr_f.view(-1)[:M * F].view(M, F)
            nn_, ns_ = (self.layers[li + 1]["attn_norm"], self.layers[li + 1]["qkv_a"].suh) if li + 1 < nl else (self.final_norm, self.lm_head.suh)
            if routed:
                use += 1
            tgt2 = self.comm.target(use, M) if routed else None
            if run_shared:
                s = self._lin(xr_d, L["gate_up"], cls, gname)
                K.finish_swiglu_rot(self.part, s, M, L["gate_up"], L["down"].suh, xr_f)
                s = self._lin(xr_f, L["down"], cls, dname)
            if not routed:
                # a dense layer: every rank computes the same FFN on the replicated stream, so the sum stays local
                K.finish_store(self.part, s, M, L["down"], self.local.slot[:M])
                self._allsum(self.local.target(0, M), M, h, nn_, ns_, xr_d)
                continue
            if run_shared:
                K.finish_store(self.part, s, M, L["down"], self.shared[:M])
            pairs, cap = M * k, self.pairs_cap[cls]
            tile_rows = (16 if M <= 16 else 32) if cls == "decode" else 128
            mt = self.max_tiles[cls]
            if cfg.n_group > 1 and 0 < cfg.topk_group < cfg.n_group:
                _lib.check(Lib.rx_moe_router_grouped(xn.data_ptr(), L["router"].data_ptr(), L["router_bias"].data_ptr(), M, d, E, k, 1, cfg.routed_scale,
                                                     cfg.n_group, cfg.topk_group, self.router_logits.data_ptr(), self.pick_ids.data_ptr(),
                                                     self.pick_w.data_ptr(), st()), "rx_moe_router_grouped")
            else:
                _lib.check(Lib.rx_moe_router2(xn.data_ptr(), L["router"].data_ptr(), L["router_bias"].data_ptr(), M, d, E, k, 1, cfg.routed_scale,
                                              self.router_logits.data_ptr(), self.pick_ids.data_ptr(), self.pick_w.data_ptr(), st()), "rx_moe_router2")
            picks, En, e_lo, e_hi = self.pick_ids, E, self.e_lo, self.e_hi
            if self.paged is not None:
                # the picks come to the host (every kernel queued so far has then run: the last call's leases can go), the experts they name
                # are made resident, and the rest of the layer runs over slot ids
                ids_h = self.pick_ids[:pairs].cpu().numpy()
                self.paged.release_held()
                self.slot_table_h.copy_(torch.from_numpy(self.paged.resolve(li, ids_h)))
                self.slot_table.copy_(self.slot_table_h, non_blocking=True)
                torch.index_select(self.slot_table, 0, self.pick_ids[:pairs].long(), out=self.pick_slot[:pairs])
                picks, En, e_lo, e_hi = self.pick_slot, self.paged.slots, 0, self.paged.slots
            _lib.check(Lib.rx_moe_plan(picks.data_ptr(), pairs, En, e_lo, e_hi, tile_rows, mt, self.offs.data_ptr(), self.pos_of_pair.data_ptr(),
                                       self.pair_of_pos.data_ptr(), self.expert_of_pos.data_ptr(), self.tile_tab.data_ptr(), self.total.data_ptr(), st()),
                       "rx_moe_plan")
            _lib.check(Lib.rx_moe_gather_rot(xn.data_ptr(), picks.data_ptr(), self.pos_of_pair.data_ptr(), pairs, k, d, None, self.xs.data_ptr(), st()),
                       "rx_moe_gather_rot")
            sg_, sd_ = self.mx_splits[cls]
            Fe = cfg.expert_ffn
            self._mx(self.xs, L["gu_w"], L["gu_s"], d, 2 * Fe, sg_, cap, mt, tile_rows)
            _lib.check(Lib.rx_moe_swiglu_rot(self.part.data_ptr(), sg_, cap, Fe, self.expert_of_pos.data_ptr(), self.total.data_ptr(), None, None,
                                             self.xs2.data_ptr(), st()), "rx_moe_swiglu_rot")
            self._mx(self.xs2, L["dn_w"], L["dn_s"], Fe, d, sd_, cap, mt, tile_rows)
            _lib.check(Lib.rx_moe_combine(self.part.data_ptr(), sd_, cap, M, d, k, picks.data_ptr(), self.pick_w.data_ptr(), self.pos_of_pair.data_ptr(),
                                          None, self.shared.data_ptr() if run_shared else None, ctypes.byref(tgt2[0]), st()), "rx_moe_combine")
            _lib.count(8)
            if multi:
                yield
            self._allsum(tgt2, M, h, nn_, ns_, xr_d)
        if not want_logits:
            return None
        xl = xr_d if logit_rows is None else xr_d.index_select(0, logit_rows).contiguous()
        Rr = xl.shape[0]
        s = self._lin(xl, self.lm_head, "decode", "lm_head")
        logits = self.logits[:Rr]
        K.finish_store(self.part, s, Rr, self.lm_head, logits)
        return logits

    def _mx(self, xs, wq, sc, Kd, N, splits, cap, max_tiles, tile_rows):
        if splits * cap * N > self.part.numel():
            raise _lib.KernelError("grouped MXFP4 partials exceed the scratch buffer")
        El = self.paged.slots if self.paged is not None else self.e_hi - self.e_lo      # paged: the stacks are the slab, one row per slot
        wbase = wq.data_ptr() - self.e_lo * N * (Kd // 2)
        sbase = sc.data_ptr() - self.e_lo * N * (Kd // 32)
        _lib.check(_lib.load().rx_mxfp4_gemm_grouped(xs.data_ptr(), cap, Kd, ctypes.c_void_p(wbase), ctypes.c_void_p(sbase), self.e_lo + El, N,
                                                     self.part.data_ptr(), splits, self.tile_tab.data_ptr(), max_tiles, tile_rows, self.status.data_ptr(),
                                                     _lib.stream_ptr()), "rx_mxfp4_gemm_grouped")

    def _finish_local(self, s, M, w, tgt):
        """One rank: the finished rows go straight to the local slot (f32), no flags."""
        K.finish_store(self.part, s, M, w, self.local.slot[:M])

    def candidates(self, logits, count):
        R = logits.shape[0]
        if self.cfg.vocab_padded != self.cfg.vocab:
            logits[:, self.cfg.vocab:] = float("-inf")
        ids, vals = self.cand_ids.view(-1)[:R * count].view(R, count), self.cand_vals.view(-1)[:R * count].view(R, count)
        K.topk(logits, count, self.topk_scratch, ids, vals)
        return ids, vals

    def _ids_view(self, R, count):
        return self.cand_ids.view(-1)[:R * count].view(R, count)

    def _vals_view(self, R, count):
        return self.cand_vals.view(-1)[:R * count].view(R, count)

    def check(self, what="forward"):
        K.check_status(self.status, what)
