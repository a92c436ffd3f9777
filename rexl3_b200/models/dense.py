"""Dense GQA decoder (Llama / Qwen3-style): config, EXL3 weight sets, fp32 reference executor, sm_100a executor.

Layer: RMSNorm -> fused qkv EXL3 linear -> (q/k norm) RoPE -> paged GQA attention -> o_proj -> residual ->
RMSNorm -> fused gate|up EXL3 linear -> SwiGLU -> down_proj -> residual; final RMSNorm -> EXL3 lm_head.
The reference engine's Qwen executor plays the same role (crates/model/src/forward.rs:986-1301); the launch
schedule here is different: every elementwise stage is fused into the finish kernel of the GEMM before it, so a
layer is 9 launches (4 GEMMs, 4 finishes, attention + merge).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, asdict

import numpy as np
import torch

from ..format import exl3

PAGE = 64


@dataclass
class DenseConfig:
    n_layers: int
    d_model: int
    n_q: int
    n_kv: int
    head_dim: int
    ffn: int                 # true FFN width (may be padded up to a multiple of 128 in storage)
    vocab: int
    eps: float = 1e-6
    rope_theta: float = 1e4
    qk_norm: bool = False
    bits: float = 4.0
    head_bits: float | None = None
    codebook: str = "3inst"
    name: str = "dense-gqa"
    mrope_sections: tuple | None = None   # (t, h, w) frequency-pair counts of interleaved M-RoPE (sum = head_dim / 2); None = plain RoPE
    # one multi-token-prediction (NextN) block after the trunk: x = e_proj(norm(embed(next token))) + h_proj(norm(trunk hidden)) - the
    # `eh_proj` of the concatenation, split along K - then one decoder layer with its own KV cache, its own final norm and the shared head;
    # row i predicts token i + 2 (reference crates/cuda/csrc/glm_mtp.cu:1-22, mtp.cu:1-6)
    mtp: bool = False

    @property
    def ffn_padded(self) -> int:
        return (self.ffn + 127) // 128 * 128

    @property
    def vocab_padded(self) -> int:
        return (self.vocab + 127) // 128 * 128

    @property
    def qkv_width(self) -> int:
        return (self.n_q + 2 * self.n_kv) * self.head_dim

    def to_json(self) -> dict:
        return asdict(self)

    def weight_params(self) -> int:
        per = self.d_model * self.qkv_width + self.n_q * self.head_dim * self.d_model + 3 * self.d_model * self.ffn_padded
        return per * self.n_layers + self.vocab_padded * self.d_model

    def kv_bytes_per_token(self, elem_bytes: int = 2) -> int:
        return 2 * self.n_kv * self.head_dim * elem_bytes * self.n_layers


CONFIGS = {
    # benchmark configuration 1: CPU plumbing model
    "tiny-llama": DenseConfig(n_layers=2, d_model=256, n_q=4, n_kv=2, head_dim=64, ffn=688, vocab=2048, eps=1e-6, rope_theta=1e4,
                              bits=4.0, name="tiny-llama"),
    # benchmark configuration 2: 27B-class dense GQA decoder
    "dense-27b": DenseConfig(n_layers=64, d_model=5120, n_q=40, n_kv=8, head_dim=128, ffn=17408, vocab=151936, eps=1e-6, rope_theta=1e6,
                             bits=4.0, name="dense-27b"),
    # small GPU test model with the production head geometry
    "test-hd128": DenseConfig(n_layers=2, d_model=512, n_q=8, n_kv=2, head_dim=128, ffn=1024, vocab=4096, bits=4.0, name="test-hd128"),
    "test-hd128-mtp": DenseConfig(n_layers=2, d_model=512, n_q=8, n_kv=2, head_dim=128, ffn=1024, vocab=4096, bits=4.0, name="test-hd128-mtp", mtp=True),
}


@dataclass
class HostLinear:
    trellis: np.ndarray
    suh: np.ndarray
    svh: np.ndarray
    bias: np.ndarray | None = None
    codebook: str = "3inst"

    def dense(self) -> np.ndarray:
        """Effective [K, N] float32 weight (native multi-threaded decoder; `exl3.decode_weight` is its numpy oracle)."""
        from ..native import host
        return host.decode_weight(self.trellis, self.codebook, self.suh.astype(np.float64), self.svh.astype(np.float64)).astype(np.float32)


@dataclass
class HostSplitLinear:
    """Projections that share their input but not their input rotation (a pack quantised one linear at a time: q / k / v, or gate / up,
    each with its own `suh`).  Served as separate GEMMs whose partial sums land side by side, so everything downstream sees one
    fused projection; packs written with one shared rotation take the fused single-GEMM path instead."""
    parts: list                  # HostLinear, in output-column order

    @property
    def svh(self) -> np.ndarray:
        return np.concatenate([p.svh for p in self.parts])

    @property
    def bias(self):
        return None if self.parts[0].bias is None else np.concatenate([p.bias for p in self.parts])

    @property
    def codebook(self) -> str:
        return self.parts[0].codebook

    def dense(self) -> np.ndarray:
        return np.concatenate([p.dense() for p in self.parts], axis=1)


class SplitWeight:
    """Device form of `HostSplitLinear`: the parts plus what the finish kernels read of a fused projection (svh, bias, N).  `suh` is None:
    producers that would fuse the next rotation into their epilogue only update the residual, and `DenseGPU._linear` rotates per part."""
    suh = None

    def __init__(self, parts, norm):
        self.parts, self.norm = parts, norm
        self.svh = torch.cat([p.svh for p in parts])
        self.bias = None if parts[0].bias is None else torch.cat([p.bias for p in parts])
        self.codebook = parts[0].codebook

    @property
    def K(self) -> int:
        return self.parts[0].K

    @property
    def N(self) -> int:
        return sum(p.N for p in self.parts)

    @property
    def twice(self) -> int:
        return self.parts[0].twice

    @property
    def nbytes(self) -> int:
        return sum(p.nbytes for p in self.parts)


@dataclass
class HostLayer:
    attn_norm: np.ndarray
    qkv: HostLinear
    o: HostLinear
    ffn_norm: np.ndarray
    gate_up: HostLinear
    down: HostLinear
    q_norm: np.ndarray | None = None
    k_norm: np.ndarray | None = None


@dataclass
class HostMtp:
    """The multi-token-prediction block of a config with `mtp`."""
    enorm: np.ndarray
    hnorm: np.ndarray
    e_proj: HostLinear           # d -> d: the embedding half of eh_proj
    h_proj: HostLinear           # d -> d: the hidden half
    layer: HostLayer
    final_norm: np.ndarray


@dataclass
class HostWeights:
    cfg: DenseConfig
    embed: np.ndarray            # float32 [vocab, d] (stored bf16 on device)
    layers: list = field(default_factory=list)
    final_norm: np.ndarray = None
    lm_head: HostLinear = None
    mtp: "HostMtp | None" = None


def _bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


def random_linear(K: int, N: int, bits: float, rng: np.random.Generator, codebook: str = "3inst", out_scale: float = 0.02,
                  zero_cols_from: int | None = None, zero_rows_from: int | None = None) -> HostLinear:
    """Random-init EXL3 layer: any random bit ring is a valid trellis; suh = +-1 signs, svh = +-out_scale."""
    b = exl3.Bits.of(bits)
    if not b.is_integer and codebook != "mul1":
        codebook = "mul1"
    trellis = rng.integers(-32768, 32768, size=(K // 16, N // 16, b.tile_words), dtype=np.int16)
    suh = np.where(rng.random(K) < 0.5, -1.0, 1.0).astype(np.float16)
    svh = (np.where(rng.random(N) < 0.5, -1.0, 1.0) * out_scale).astype(np.float16)
    if zero_cols_from is not None:
        svh[zero_cols_from:] = 0
    if zero_rows_from is not None:
        suh[zero_rows_from:] = 0
    return HostLinear(trellis, suh, svh, None, codebook)


def random_weights(cfg: DenseConfig, seed: int = 0, per_linear: bool = False) -> HostWeights:
    """Random-init weights of the architecture with valid random EXL3 tensors (benchmarks and kernel tests).  `per_linear`: q / k / v and
    gate / up keep their own input rotations (`HostSplitLinear`), the form of a pack that was quantised one linear at a time."""
    rng = np.random.default_rng(seed)
    d, F = cfg.d_model, cfg.ffn_padded
    s_in = 1.0 / math.sqrt(d)
    w = HostWeights(cfg, _bf16_round(rng.normal(0, 1.0, size=(cfg.vocab, d)).astype(np.float32)))
    for _ in range(cfg.n_layers + (1 if cfg.mtp else 0)):
        qkv = random_linear(d, cfg.qkv_width, cfg.bits, rng, cfg.codebook, s_in)
        o = random_linear(cfg.n_q * cfg.head_dim, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(cfg.n_q * cfg.head_dim))
        gu = random_linear(d, 2 * F, cfg.bits, rng, cfg.codebook, s_in)
        if F != cfg.ffn:  # padded FFN columns contribute exactly zero
            gu.svh[cfg.ffn:F] = 0
            gu.svh[F + cfg.ffn:] = 0
        down = random_linear(F, d, cfg.bits, rng, cfg.codebook, 0.5 / math.sqrt(F), zero_rows_from=cfg.ffn if F != cfg.ffn else None)
        if per_linear:
            def split(l, widths):
                parts, c0 = [], 0
                for wd in widths:
                    suh = np.where(rng.random(l.trellis.shape[0] * 16) < 0.5, -1.0, 1.0).astype(np.float16)
                    parts.append(HostLinear(np.ascontiguousarray(l.trellis[:, c0 // 16:(c0 + wd) // 16]), suh, l.svh[c0:c0 + wd].copy(), None, l.codebook))
                    c0 += wd
                return HostSplitLinear(parts)
            qkv = split(qkv, [cfg.n_q * cfg.head_dim, cfg.n_kv * cfg.head_dim, cfg.n_kv * cfg.head_dim])
            gu = split(gu, [F, F])
        lay = HostLayer(_bf16_round(1.0 + 0.1 * rng.normal(size=d)), qkv, o, _bf16_round(1.0 + 0.1 * rng.normal(size=d)), gu, down)
        if cfg.qk_norm:
            lay.q_norm = _bf16_round(1.0 + 0.1 * rng.normal(size=cfg.head_dim))
            lay.k_norm = _bf16_round(1.0 + 0.1 * rng.normal(size=cfg.head_dim))
        w.layers.append(lay)
    w.final_norm = _bf16_round(1.0 + 0.1 * rng.normal(size=d))
    hb = cfg.head_bits or cfg.bits
    w.lm_head = random_linear(d, cfg.vocab_padded, hb, rng, cfg.codebook, s_in, zero_cols_from=cfg.vocab if cfg.vocab_padded != cfg.vocab else None)
    if cfg.mtp:
        nrm = lambda: _bf16_round(1.0 + 0.1 * rng.normal(size=d))  # noqa: E731
        w.mtp = HostMtp(nrm(), nrm(), random_linear(d, d, cfg.bits, rng, cfg.codebook, 0.7 * s_in), random_linear(d, d, cfg.bits, rng, cfg.codebook, 0.7 * s_in),
                        w.layers.pop(), nrm())
    return w


def rope_inv_freq(cfg: DenseConfig) -> np.ndarray:
    i = np.arange(0, cfg.head_dim, 2, dtype=np.float32)
    return (1.0 / (np.float32(cfg.rope_theta) ** (i / np.float32(cfg.head_dim)))).astype(np.float32)


# ====================================================================================================== reference
class ReferenceDense:
    """fp32 PyTorch executor over the dequantized weights: the numerics oracle (CPU or any device).

    Keeps one contiguous KV list per sequence id; rows are (seq, position, token).
    """

    def __init__(self, w: HostWeights, device="cpu", dtype=torch.float32):
        self.cfg = cfg = w.cfg
        self.device, self.dtype = device, dtype
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=dtype)  # noqa: E731
        self.embed = t(w.embed)
        self.layers = []
        for lay in w.layers:
            self.layers.append(dict(attn_norm=t(lay.attn_norm), qkv=t(lay.qkv.dense()), o=t(lay.o.dense()), ffn_norm=t(lay.ffn_norm),
                                    gate_up=t(lay.gate_up.dense()), down=t(lay.down.dense()),
                                    q_norm=None if lay.q_norm is None else t(lay.q_norm), k_norm=None if lay.k_norm is None else t(lay.k_norm)))
        self.final_norm = t(w.final_norm)
        self.lm_head = t(w.lm_head.dense())[:, :cfg.vocab]
        self.inv_freq = torch.from_numpy(rope_inv_freq(cfg)).to(device)
        self.kv = {}  # seq -> list over layers of (k [T, n_kv, hd], v)
        self.mtp = None
        if w.mtp is not None:
            lay = w.mtp.layer
            self.mtp = dict(enorm=t(w.mtp.enorm), hnorm=t(w.mtp.hnorm), e_proj=t(w.mtp.e_proj.dense()), h_proj=t(w.mtp.h_proj.dense()), final_norm=t(w.mtp.final_norm),
                            layer=dict(attn_norm=t(lay.attn_norm), qkv=t(lay.qkv.dense()), o=t(lay.o.dense()), ffn_norm=t(lay.ffn_norm),
                                       gate_up=t(lay.gate_up.dense()), down=t(lay.down.dense()),
                                       q_norm=None if lay.q_norm is None else t(lay.q_norm), k_norm=None if lay.k_norm is None else t(lay.k_norm)))
        self.last_hidden = None     # the trunk's final residual rows of the last forward_seq (what an MTP block reads)

    def reset(self, seq=None):
        if seq is None:
            self.kv.clear()
        else:
            self.kv.pop(seq, None)

    def truncate(self, seq, length: int):
        if seq in self.kv:
            self.kv[seq] = [(k[:length], v[:length]) for k, v in self.kv[seq]]

    @staticmethod
    def _rms(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def _rope(self, x, pos):
        # x [T, H, hd]; rotate-half
        ang = pos.to(torch.float32)[:, None] * self.inv_freq[None, :]
        cos, sin = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
        h = x.shape[-1] // 2
        x1, x2 = x[..., :h], x[..., h:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    @torch.no_grad()
    def _ffn(self, li, L, h):
        cfg = self.cfg
        x = self._rms(h, L["ffn_norm"], cfg.eps)
        gu = x @ L["gate_up"]
        F = cfg.ffn_padded
        y = (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]) @ L["down"]
        ov = getattr(self, "interventions", {}).get(li)
        if ov is not None:                      # runtime overlay at the block's output (models/intervention.py)
            from .intervention import apply_reference
            y = apply_reference(y, ov)
        return h + y

    def _mix(self, li, L, h, pos, seq, start):
        """Token mixer of one layer on the residual stream `h` [T, d]: returns what is added to it (here: GQA attention + o_proj)."""
        cfg = self.cfg
        T = h.shape[0]
        x = self._rms(h, L["attn_norm"], cfg.eps)
        qkv = x @ L["qkv"]
        q = qkv[:, :cfg.n_q * cfg.head_dim].view(T, cfg.n_q, cfg.head_dim)
        k = qkv[:, cfg.n_q * cfg.head_dim:(cfg.n_q + cfg.n_kv) * cfg.head_dim].view(T, cfg.n_kv, cfg.head_dim)
        v = qkv[:, (cfg.n_q + cfg.n_kv) * cfg.head_dim:].view(T, cfg.n_kv, cfg.head_dim)
        if L["q_norm"] is not None:
            q, k = self._rms(q, L["q_norm"], cfg.eps), self._rms(k, L["k_norm"], cfg.eps)
        q, k = self._rope(q, pos), self._rope(k, pos)
        pk, pv = self.kv[seq][li]
        kk, vv = torch.cat([pk[:start], k]), torch.cat([pv[:start], v])
        self.kv[seq][li] = (kk, vv)
        g = cfg.n_q // cfg.n_kv
        kq, vq = kk.repeat_interleave(g, dim=1), vv.repeat_interleave(g, dim=1)
        s = torch.einsum("thd,shd->hts", q, kq) / math.sqrt(cfg.head_dim)
        kpos = torch.arange(kk.shape[0], device=self.device)
        mask = kpos[None, :] > pos[:, None]
        s = s.masked_fill(mask[None], float("-inf"))
        a = torch.einsum("hts,shd->thd", torch.softmax(s, dim=-1), vq).reshape(T, -1)
        return a @ L["o"]

    @torch.no_grad()
    def forward_seq(self, seq, tokens, start: int, n_layers: int | None = None) -> torch.Tensor:
        """Append `tokens` to sequence `seq` at positions start.. ; returns logits [T, vocab] (fp32).  `n_layers` runs only the
        first layers and applies the final norm and head to their output (the self-speculative draft)."""
        cfg = self.cfg
        ids = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        T = ids.shape[0]
        pos = torch.arange(start, start + T, device=self.device)
        h = self.embed[ids]
        if seq not in self.kv:
            self.kv[seq] = [(torch.zeros(0, cfg.n_kv, cfg.head_dim, device=self.device, dtype=self.dtype),) * 2 for _ in range(len(self.layers) + 1)]
        for li, L in enumerate(self.layers[:n_layers or len(self.layers)]):
            h = self._ffn(li, L, h + self._mix(li, L, h, pos, seq, start))
        self.last_hidden = h
        return (self._rms(h, self.final_norm, cfg.eps) @ self.lm_head).float()

    @torch.no_grad()
    def mtp_seq(self, seq, next_tokens, hidden, start: int):
        """The MTP block on rows at positions start..: row i reads the trunk (or previous MTP) hidden of position i and the token at i + 1.
        -> (logits [T, vocab] predicting the tokens at i + 2, the block's output hidden rows)."""
        cfg, m = self.cfg, self.mtp
        ids = torch.as_tensor(next_tokens, dtype=torch.long, device=self.device)
        T = ids.shape[0]
        pos = torch.arange(start, start + T, device=self.device)
        h = self._rms(self.embed[ids], m["enorm"], cfg.eps) @ m["e_proj"] + self._rms(hidden, m["hnorm"], cfg.eps) @ m["h_proj"]
        li = len(self.layers)
        h = self._ffn(li, m["layer"], h + self._mix(li, m["layer"], h, pos, seq, start))
        return (self._rms(h, m["final_norm"], cfg.eps) @ self.lm_head).float(), h


# ====================================================================================================== sm_100a executor
class DenseGPU:
    """The model on one B200: EXL3 weights as stored, paged bf16 KV cache, hand-written kernels only.

    ``rows`` API (what the engine backend drives): every call passes per-row token ids, absolute positions,
    the sequence slot of each row and the block table; rows may mix sequences freely (decode / verify windows) or be
    one or more prompt chunks (prefill).
    """

    def __init__(self, w: "HostWeights | DenseConfig", num_pages: int, max_rows: int = 256, max_seqs: int = 64, max_blocks_per_seq: int = 256,
                 device="cuda", max_prefill_rows: int = 8192, seed: int = 0, kv_dtype: str = "bf16"):
        """`w` is either host weights (uploaded as stored) or a bare config (random-init EXL3 weights are then generated on the
        device: any random bit ring is a valid trellis, which is how benchmark models of tens of GB are made in seconds)."""
        from ..ops import kernels as K
        self.K = K
        self.window_seq_rows = 1       # the most adjacent rows one sequence has in the next decode / verify window (set by the backend)
        self.attn_plan = None          # device plan of the current window for the attention kernel (allocated with the scratch)
        # int32 [rows, 3] (T, H, W positions) for the next forward of a model whose config has `mrope_sections`; None = text rows, where
        # the three axes equal `positions` and plain RoPE gives the same bits
        self.pos3 = None
        self.tree = None               # (tree_base, vbt, moves, n_moves) while a forward runs a verify window of draft trees
        self._kv_ptrs = None
        self._kv_scale_ptrs = None
        self.device = device
        self.mtp = None                # the multi-token-prediction block's tensors (config.mtp), set by the loaders of the dense family
        self.interventions = {}        # layer -> (alpha, orthonormal basis f32 [r, d]) runtime overlays (set_interventions)
        self._iv_y = None
        if isinstance(w, DenseConfig):
            self.cfg = cfg = w
            self._load_random(seed)
        else:
            self.cfg = cfg = w.cfg
            self._load_host(w)
        self.num_pages, self.max_seqs, self.max_blocks = num_pages, max_seqs, max_blocks_per_seq
        self.max_rows = max(max_rows, max_prefill_rows)
        self.inv_freq = torch.from_numpy(rope_inv_freq(cfg)).to(device)
        # paged KV: one K and one V tensor per layer, [pages, n_kv, 64, hd] bf16 (or E4M3 bytes with one scale per layer, K/V and head),
        # plus their TMA descriptors
        # (or int8 with one power-of-two scale per token and KV head, kept in k_tscale / v_tscale [pages, n_kv, 64] f32 beside each layer's cache)
        if kv_dtype not in ("bf16", "fp8", "int8", "q4"):
            raise ValueError(f"kv_dtype {kv_dtype!r}: bf16, fp8, int8 or q4")
        self.kv_fp8 = kv_dtype == "fp8"
        self.kv_i8 = kv_dtype == "int8"
        # q4: E2M1 nibbles with one E8M0 scale per 32 values (the MXFP4 element format on K / V rows), 68 bytes per 128-wide row instead of 256
        self.kv_q4 = kv_dtype == "q4"
        if self.kv_q4 and cfg.head_dim != 128:
            raise ValueError("the q4 KV cache is built for 128-wide heads")
        cdt = torch.uint8 if (self.kv_fp8 or self.kv_q4) else (torch.int8 if self.kv_i8 else torch.bfloat16)
        kw = cfg.head_dim // 2 if self.kv_q4 else cfg.head_dim          # stored width of a row
        kvl = set(self._kv_layers())
        nkv = cfg.n_layers + (1 if getattr(cfg, "mtp", False) else 0)      # the MTP block's attention owns cache index n_layers
        if nkv > cfg.n_layers:
            if self.mtp is None:
                raise ValueError(f"{type(self).__name__} has no multi-token-prediction block (config.mtp is a dense-family feature)")
            if kv_dtype != "bf16":
                raise ValueError("the multi-token-prediction block runs on a bf16 KV cache")
            kvl.add(cfg.n_layers)
        self.k_cache = [torch.zeros(num_pages, cfg.n_kv, PAGE, kw, dtype=cdt, device=device) if i in kvl else None for i in range(nkv)]
        self.v_cache = [torch.zeros(num_pages, cfg.n_kv, PAGE, kw, dtype=cdt, device=device) if i in kvl else None for i in range(nkv)]
        self.kv_scale = torch.ones(nkv, 2, cfg.n_kv, dtype=torch.float32, device=device) if self.kv_fp8 else None
        self.kv_amax = None        # set while calibrating
        mk_ts = (lambda: torch.full((num_pages, cfg.n_kv, PAGE, cfg.head_dim // 32), 127, dtype=torch.uint8, device=device)) if self.kv_q4 else \
            (lambda: torch.ones(num_pages, cfg.n_kv, PAGE, dtype=torch.float32, device=device))
        self.k_tscale = [mk_ts() if ((self.kv_i8 or self.kv_q4) and i in kvl) else None for i in range(nkv)]
        self.v_tscale = [mk_ts() if ((self.kv_i8 or self.kv_q4) and i in kvl) else None for i in range(nkv)]
        self.tk = [None if c is None else K.KvTensorMap(c) for c in self.k_cache]
        self.tv = [None if c is None else K.KvTensorMap(c) for c in self.v_cache]
        self.status = K.new_status(device)
        self._alloc_scratch(self.max_rows)

    def _load_host(self, w: HostWeights) -> None:
        from ..utils import loadstats
        with loadstats.stage("model", "upload"):
            self._upload_host(w)
            torch.cuda.synchronize()
        loadstats.add("model", "upload", 0.0, self.weight_bytes())

    def _upload_host(self, w: HostWeights) -> None:
        K, device = self.K, self.device
        dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=dt)  # noqa: E731
        up1 = lambda l: K.Exl3Weight.from_numpy(l.trellis, l.suh, l.svh, l.bias, l.codebook, device)  # noqa: E731

        def up(l, norm=None):
            return SplitWeight([up1(p) for p in l.parts], norm) if isinstance(l, HostSplitLinear) else up1(l)
        self.embed = dev(w.embed, torch.bfloat16)
        self.layers = []
        for lay in w.layers:
            an, fn = dev(lay.attn_norm, torch.bfloat16), dev(lay.ffn_norm, torch.bfloat16)
            self.layers.append(dict(attn_norm=an, qkv=up(lay.qkv, an), o=up(lay.o), ffn_norm=fn,
                                    gate_up=up(lay.gate_up, fn), down=up(lay.down),
                                    q_norm=None if lay.q_norm is None else dev(lay.q_norm, torch.bfloat16),
                                    k_norm=None if lay.k_norm is None else dev(lay.k_norm, torch.bfloat16)))
        self.final_norm = dev(w.final_norm, torch.bfloat16)
        self.lm_head = up(w.lm_head)
        if w.mtp is not None and type(self)._upload_host is DenseGPU._upload_host:
            lay = w.mtp.layer
            an, fn = dev(lay.attn_norm, torch.bfloat16), dev(lay.ffn_norm, torch.bfloat16)
            self.mtp = dict(enorm=dev(w.mtp.enorm, torch.bfloat16), hnorm=dev(w.mtp.hnorm, torch.bfloat16), e_proj=up1(w.mtp.e_proj), h_proj=up1(w.mtp.h_proj),
                            final_norm=dev(w.mtp.final_norm, torch.bfloat16),
                            layer=dict(attn_norm=an, qkv=up(lay.qkv, an), o=up(lay.o), ffn_norm=fn, gate_up=up(lay.gate_up, fn), down=up(lay.down),
                                       q_norm=None if lay.q_norm is None else dev(lay.q_norm, torch.bfloat16),
                                       k_norm=None if lay.k_norm is None else dev(lay.k_norm, torch.bfloat16)))

    def _load_random(self, seed: int) -> None:
        cfg, K, device = self.cfg, self.K, self.device
        g = torch.Generator(device=device).manual_seed(seed)
        tw = exl3.Bits.of(cfg.bits).tile_words
        cb = cfg.codebook if exl3.Bits.of(cfg.bits).is_integer else "mul1"

        def lin(k, n, scale, words=tw):
            tr = torch.randint(-32768, 32768, (k // 16, n // 16, words), dtype=torch.int16, device=device, generator=g)
            sg = lambda m: (torch.randint(0, 2, (m,), device=device, generator=g) * 2 - 1)  # noqa: E731
            return K.Exl3Weight(tr, sg(k).to(torch.float16), (sg(n) * scale).to(torch.float16), None, cb)

        norm = lambda: (1.0 + 0.1 * torch.randn(cfg.d_model, device=device, generator=g)).to(torch.bfloat16)  # noqa: E731
        d, F, HQ = cfg.d_model, cfg.ffn_padded, cfg.n_q * cfg.head_dim
        self.embed = torch.randn(cfg.vocab, d, device=device, generator=g).to(torch.bfloat16)
        self.layers = []
        for _ in range(cfg.n_layers + (1 if getattr(cfg, "mtp", False) else 0)):
            gu = lin(d, 2 * F, 1.0 / math.sqrt(d))
            dn = lin(F, d, 0.5 / math.sqrt(F))
            if F != cfg.ffn:
                gu.svh[cfg.ffn:F] = 0
                gu.svh[F + cfg.ffn:] = 0
                dn.suh[cfg.ffn:] = 0
            self.layers.append(dict(attn_norm=norm(), qkv=lin(d, cfg.qkv_width, 1.0 / math.sqrt(d)), o=lin(HQ, d, 0.5 / math.sqrt(HQ)),
                                    ffn_norm=norm(), gate_up=gu, down=dn, q_norm=None, k_norm=None))
        if getattr(cfg, "mtp", False):
            self.mtp = dict(enorm=norm(), hnorm=norm(), e_proj=lin(d, d, 0.7 / math.sqrt(d)), h_proj=lin(d, d, 0.7 / math.sqrt(d)), final_norm=norm(),
                            layer=self.layers.pop())
        self.final_norm = norm()
        hw = exl3.Bits.of(cfg.head_bits or cfg.bits).tile_words
        self.lm_head = lin(d, cfg.vocab_padded, 1.0 / math.sqrt(d), hw)
        if cfg.vocab_padded != cfg.vocab:
            self.lm_head.svh[cfg.vocab:] = 0

    # ------------------------------------------------------------------ buffers
    def _alloc_scratch(self, R: int):
        cfg, K, dev = self.cfg, self.K, self.device
        self.splits = {}
        part_elems = 0
        shapes = self._gemm_shapes()
        for cls, rows in (("decode", min(R, 256)), ("prefill", R)):
            for name, (k, n) in shapes.items():
                s = K.plan_splits(k, n, cls == "decode")
                self.splits[(cls, name)] = s
                r = rows if name != "lm_head" else min(rows, 256)
                part_elems = max(part_elems, s * r * n)
        from ..utils import canary
        g = lambda name, shape, dt: canary.guarded(f"{type(self).__name__}.{name}", shape, dt, dev)  # noqa: E731  (guard bands with REXL3_CANARY=1)
        self.part = g("part", part_elems, torch.float32)
        # split projections (per-linear input rotations) run one GEMM per part into this second buffer before the partials are placed
        split = any(isinstance(v, SplitWeight) for L in self.layers for v in L.values())
        self._part_split = torch.empty(part_elems, dtype=torch.float32, device=dev) if split else None
        kmax = max(k for k, _ in shapes.values())
        self.xr = g("xr", R * kmax, torch.float16)
        self.xr2 = g("xr2", R * cfg.ffn_padded, torch.float16)
        self.h = g("h", (R, cfg.d_model), torch.bfloat16)
        if self.mtp is not None:        # the block's own residual stream and the embedding rows of the next tokens
            self.h_mtp = torch.empty(R, cfg.d_model, dtype=torch.bfloat16, device=dev)
            self.e_mtp = torch.empty(R, cfg.d_model, dtype=torch.bfloat16, device=dev)
        self.q = g("q", (R, cfg.n_q * cfg.head_dim), torch.bfloat16)
        self.attn_out = g("attn_out", (R, cfg.n_q * cfg.head_dim), torch.bfloat16)
        self.logits = g("logits", (min(R, 256), cfg.vocab_padded), torch.float32)
        self.max_ctx_alloc = self.max_blocks * PAGE
        self.attn_scratch = K.attn_decode_scratch(min(R, 256), cfg.n_q, cfg.head_dim, self.max_ctx_alloc, dev)
        self.attn_plan = K.attn_plan_buffer(dev)
        self.topk_scratch = K.topk_scratch(min(R, 256), cfg.vocab_padded, 64, dev)
        self.cand_ids = torch.empty(min(R, 256), 64, dtype=torch.int32, device=dev)
        self.cand_vals = torch.empty(min(R, 256), 64, dtype=torch.float32, device=dev)

    def _gemm_shapes(self) -> dict:
        """name -> (K, N) of every EXL3 GEMM this executor launches through `_linear` (sizes the split plans and the scratch)."""
        cfg = self.cfg
        return dict(qkv=(cfg.d_model, cfg.qkv_width), o=(cfg.n_q * cfg.head_dim, cfg.d_model), gate_up=(cfg.d_model, 2 * cfg.ffn_padded),
                    down=(cfg.ffn_padded, cfg.d_model), lm_head=(cfg.d_model, cfg.vocab_padded), eh_proj=(cfg.d_model, cfg.d_model))

    def _kv_layers(self):
        """Indices of the layers that own a paged KV cache (all of them here; a hybrid has layers without one)."""
        return range(self.cfg.n_layers)

    def scale_tail(self, first_layer: int, eps: float) -> None:
        """Multiply the output scales of the residual writers (`o` and `down`, expert stacks included) of layers >= first_layer by eps.
        A synthetic-weight recipe for speculation benchmarks: with a small eps the layers above the draft depth barely move the residual
        stream, so a draft made of the first layers plus the shared head agrees with the target often; eps sets how often.  Random-init
        weights only have this knob: their acceptance is otherwise zero."""
        for L in self.layers[first_layer:]:
            for k in ("o", "down"):
                w = L.get(k)
                if w is not None and getattr(w, "svh", None) is not None:
                    w.svh.mul_(eps)

    def weight_bytes(self) -> int:
        n = self.embed.numel() * 2 + self.lm_head.nbytes
        for L in self.layers:
            n += sum(L[k].nbytes for k in ("qkv", "o", "gate_up", "down"))
        return n

    def calibrate_kv(self, tokens, passes: int = 2, headroom: float = 1.25) -> None:
        """FP8 cache: set the per-(layer, K/V, head) scales from the largest |K| and |V| seen while prefilling `tokens` (a list of token ids,
        at most one page table row long) into page 0..: scale = amax * headroom / 448.  Two passes, because the first one stores with
        scale 1.  A pack that ships calibrated scales sets `kv_scale` directly instead.  The pages used are scratch: call before serving."""
        if not self.kv_fp8:
            return
        T = len(tokens)
        dev = self.device
        nb = (T + PAGE - 1) // PAGE
        assert nb <= min(self.max_blocks, self.num_pages) and T <= self.max_rows
        bt = torch.zeros(self.max_seqs, self.max_blocks, dtype=torch.int32, device=dev)
        bt[0, :nb] = torch.arange(nb, dtype=torch.int32, device=dev)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
        pos = list(range(T))
        pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([T]), pos0=i32([0]), nseq=1, max_qlen=T)
        args = (i32(list(tokens)), i32(pos), i32(pos), i32([0] * T), i32([p + 1 for p in pos]), bt)
        for _ in range(passes):
            self.kv_amax = torch.zeros_like(self.kv_scale)
            self.forward_rows(*args, prefill=pf, want_logits=False)
            torch.cuda.synchronize()
            self.kv_scale.copy_(torch.clamp(self.kv_amax, min=1e-4) * (headroom / 448.0))
        self.kv_amax = None

    # ------------------------------------------------------------------ forward
    def _linear(self, xr, w, rows, cls, name):
        s = self.splits[(cls, name)]
        if isinstance(w, SplitWeight):
            # per-part input rotation of the normed residual rows, one GEMM per part, partial sums placed side by side
            K, N = self.K, w.N
            dst = self.part[:s * rows * N].view(s, rows, N)
            xr_p = self.xr2[:rows * w.K].view(rows, w.K)
            off = 0
            for p in w.parts:
                K.norm_rot_in(self.h[:rows], w.norm, self.cfg.eps, p.suh, xr_p)
                K.exl3_gemm(xr_p, p, self._part_split, s, self.status)
                dst[:, :, off:off + p.N].copy_(self._part_split[:s * rows * p.N].view(s, rows, p.N))
                off += p.N
            return s
        self.K.exl3_gemm(xr, w, self.part, s, self.status)
        return s

    def _mixer(self, li, L, M, cls, xr_d, xr_a, q, positions, slots, row_seq, ctx_len, block_table, prefill, max_ctx, scale):
        """The token mixer of layer `li` up to and including its output projection GEMM: leaves that GEMM's K-split partials in self.part
        and returns the split count.  Here: paged GQA attention."""
        cfg, K = self.cfg, self.K
        s = self._linear(xr_d, L["qkv"], M, cls, "qkv")
        ksc = self.kv_scale[li] if self.kv_fp8 else None
        kts = (self.k_tscale[li], self.v_tscale[li]) if (self.kv_i8 or self.kv_q4) else None
        q4 = self.kv_q4
        K.finish_qkv_rope(self.part, s, M, cfg.n_q, cfg.n_kv, cfg.head_dim, L["qkv"], L["q_norm"], L["k_norm"], cfg.eps, positions,
                          self.inv_freq, slots, q, self.k_cache[li], self.v_cache[li], ksc, None if self.kv_amax is None else self.kv_amax[li],
                          pos3=self.pos3, mrope_sections=getattr(cfg, "mrope_sections", None), kv_tscale=kts, q4=q4)
        if prefill is None:
            vbt = None
            if self.tree is not None:
                # this layer's K / V rows of the window are written: copy what each node's private pages must hold (the committed rows of the
                # page its path starts in, and its ancestors at their positions)
                vbt = self.tree[1]
                K.kv_move_rows(self._kv_ptr_table()[2 * li:2 * li + 2], self._kv_row_bytes(), cfg.n_kv, self.tree[2], self.tree[3])
                if kts is not None:
                    K.kv_move_rows(self._kv_scale_ptr_table()[2 * li:2 * li + 2], self._kv_scale_row_bytes(), cfg.n_kv, self.tree[2], self.tree[3])
            K.attn_decode(self.tk[li], self.tv[li], q, block_table, row_seq, ctx_len, self.attn_scratch, cfg.n_q, cfg.n_kv, cfg.head_dim,
                          max_ctx or self.max_ctx_alloc, scale, L["o"].suh, xr_a, None, self.status, ksc, max_seq_rows=self.window_seq_rows,
                          plan=self.attn_plan, kv_tscale=kts, q4=q4, vbt=vbt)
        else:
            ao = self.attn_out[:M]
            K.attn_prefill(self.tk[li], self.tv[li], q, block_table, prefill["seq_ids"], prefill["q_start"], prefill["q_len"], prefill["pos0"],
                           ao, prefill["nseq"], prefill["max_qlen"], cfg.n_q, cfg.n_kv, cfg.head_dim, scale, self.status, ksc, kv_tscale=kts, q4=q4)
            K.norm_rot_in(ao, None, cfg.eps, L["o"].suh, xr_a)
        s = self._linear(xr_a, L["o"], M, cls, "o")
        return s

    def _begin_forward(self) -> None:
        """Hook run once per forward before the first kernel (multi-rank executors bump their ticket epoch here)."""

    def _ffn(self, li, L, M, cls, s_o, h, xr_d, xr_f, next_norm, next_suh):
        """Everything between the o_proj GEMM (its partials are in self.part, `s_o` splits) and the next layer's rotated input."""
        cfg, K = self.cfg, self.K
        K.finish_add_norm_rot(self.part, s_o, M, L["o"], h, L["ffn_norm"], cfg.eps, L["gate_up"].suh, xr_d)
        s = self._linear(xr_d, L["gate_up"], M, cls, "gate_up")
        K.finish_swiglu_rot(self.part, s, M, L["gate_up"], L["down"].suh, xr_f)
        s = self._linear(xr_f, L["down"], M, cls, "down")
        ov = self.interventions.get(li) if self.interventions else None
        if ov is None:
            K.finish_add_norm_rot(self.part, s, M, L["down"], h, next_norm, cfg.eps, next_suh, xr_d)
            return
        # a runtime overlay on this layer's block output: finish the rows to f32, remove the overlay's directions, then residual, norm, rotation
        y = self._iv_y[:M]
        K.finish_store(self.part, s, M, L["down"], y)
        y.addmm_(y @ ov[1].T, ov[1], alpha=-ov[0])
        h.copy_(h.float() + y)
        if next_suh is not None:
            K.norm_rot_in(h, next_norm, cfg.eps, next_suh, xr_d)

    def set_interventions(self, overlays: dict) -> None:
        """overlays: {layer: models.intervention.LayerOverlay} (or {} to clear).  Applied at the output of the layer's feed-forward block."""
        if overlays and (type(self)._ffn is not DenseGPU._ffn or type(self)._ffn_phases is not DenseGPU._ffn_phases):
            raise ValueError(f"{type(self).__name__} replaces the feed-forward block: no overlay hook there (an overlay never applies silently in part)")
        for li in overlays:
            if not 0 <= li < self.cfg.n_layers:
                raise ValueError(f"intervention on layer {li}: the model has layers 0..{self.cfg.n_layers - 1}")
        self.interventions = {li: (float(o.alpha), torch.from_numpy(o.basis).to(self.device)) for li, o in overlays.items()}
        if overlays and getattr(self, "_iv_y", None) is None:
            self._iv_y = torch.empty(self.max_rows, self.cfg.d_model, dtype=torch.float32, device=self.device)

    def _ffn_phases(self, *a):
        """Generator form of `_ffn`: yields wherever the ranks of a multi-rank executor must all have launched the previous kernels
        before one of them may launch the next (a one-GPU loopback group steps its ranks there).  One rank: no such point."""
        self._ffn(*a)
        return
        yield

    def forward_rows(self, *a, **kw):
        g = self.forward_phases(*a, **kw)
        try:
            while True:
                next(g)
        except StopIteration as e:
            return e.value

    def forward_phases(self, ids, positions, slots, row_seq, ctx_len, block_table, *, prefill=None, logit_rows=None, max_ctx=None, want_logits=True,
                       n_layers=None, embed_rows=None, pos3=None, tree=None):
        """Run all layers over M rows.

        tree: (tree_base int32 [M], vbt int32 [M, attn_vbt_width()], moves int32 [n, 3], n) for a verify window of draft trees (decode path,
        bf16 cache).  A sequence's rows are its tree's nodes (the anchor first); row r stands at `positions[r]` = tree_base + depth, is written
        to `slots[r]` (its true slot when the node's path is the tree's first chain, else that position's row of a private page), and
        ctx_len = positions + 1.  vbt[r] lists the pages that hold the row's view of positions from chunk (tree_base + 1) // 256 on: the
        sequence's pages, with private pages where the row's own path lies; `moves` (see ops.kernels.kv_move_rows) fill those private pages in
        every layer once the layer's K / V rows are written.  Each row then attends to exactly the keys, at the positions, of a serial run
        over its path, so its logits are that run's bits.  `move_kv_rows` afterwards brings the accepted path's rows to their true slots.

        embed_rows: (int64 index tensor [n], bf16 [n, d_model]) - rows whose token embedding is replaced (image tokens encoded by a vision
        tower).  pos3: int32 [M, 3] (T, H, W positions) for a config with `mrope_sections`; None = text rows (all axes = positions).

        ids, positions, slots, row_seq, ctx_len: int32 device tensors [M] (slot = physical KV slot page*64+offset of the row's
        own token; ctx_len = number of keys the row attends to = position + 1).  block_table int32 [max_seqs, max_blocks].
        prefill: None for the decode/verify path, else dict(seq_ids, q_start, q_len, pos0, nseq, max_qlen) device tensors
        describing which rows form which prompt chunk.  logit_rows: index tensor of the rows whose logits are wanted
        (default: all rows).  Returns fp32 logits [len(logit_rows), vocab_padded] (a view of a reused buffer).
        """
        cfg, K = self.cfg, self.K
        M = ids.shape[0]
        cls = "decode" if prefill is None else "prefill"
        assert M <= self.max_rows and (prefill is not None or M <= 256)
        h = self.h[:M]
        d, F, HQ = cfg.d_model, cfg.ffn_padded, cfg.n_q * cfg.head_dim
        xr_d = self.xr[:M * d].view(M, d)
        xr_a = self.xr[:M * HQ].view(M, HQ)
        xr_f = self.xr2[:M * F].view(M, F)
        q = self.q[:M]
        scale = 1.0 / math.sqrt(cfg.head_dim)
        self._begin_forward()
        if tree is not None and (prefill is not None or not self.supports_trees() or self.attn_plan is None):
            raise ValueError("a tree window runs on the decode path of a model with a bf16 KV cache and attention in every layer")
        if prefill is None and self.attn_plan is not None:
            # one plan of the window (row blocks and work items of the persistent attention kernel) serves every layer
            K.attn_plan(row_seq, ctx_len, cfg.n_q, cfg.n_kv, self.window_seq_rows, self.attn_plan, tree_base=None if tree is None else tree[0])
        K.embed(ids, self.embed, h)
        if embed_rows is not None:
            h.index_copy_(0, embed_rows[0], embed_rows[1].to(h.dtype))
        self.pos3 = pos3
        self.tree = tree
        L0 = self.layers[0]
        if L0["qkv"].suh is not None:          # (split projections rotate per part inside _linear)
            K.norm_rot_in(h, L0["attn_norm"], cfg.eps, L0["qkv"].suh, xr_d)
        nl = n_layers or len(self.layers)      # n_layers < all: the self-speculative draft (first layers + shared final norm and head)
        for li in range(nl):
            L = self.layers[li]
            s = self._mixer(li, L, M, cls, xr_d, xr_a, q, positions, slots, row_seq, ctx_len, block_table, prefill, max_ctx, scale)
            nn_, ns_ = (self.layers[li + 1]["attn_norm"], self.layers[li + 1]["qkv"].suh) if li + 1 < nl else (self.final_norm, self.lm_head.suh)
            yield from self._ffn_phases(li, L, M, cls, s, h, xr_d, xr_f, nn_, ns_)
        self.tree = None
        if not want_logits:
            return None
        if logit_rows is not None:
            xl = xr_d.index_select(0, logit_rows).contiguous()
        else:
            xl = xr_d
        R = xl.shape[0]
        assert R <= self.logits.shape[0]
        s = self._linear(xl, self.lm_head, R, "decode", "lm_head")
        logits = self.logits[:R]
        K.finish_store(self.part, s, R, self.lm_head, logits)
        return logits

    def supports_trees(self) -> bool:
        """Tree windows need every layer's token mixer to be the paged attention of this class (a recurrent mixer has no per-node state).  bf16,
        fp8 and int8 caches work (the window's row copies also move the int8 cache's per-token scale planes); the q4 decode entry takes no
        private tables."""
        return type(self)._mixer is DenseGPU._mixer and not self.kv_q4 and all(c is not None for c in self.k_cache)

    def _kv_ptr_table(self):
        """int64 device tensor [2 * layers]: the K and V cache addresses, layer by layer."""
        if self._kv_ptrs is None:
            self._kv_ptrs = torch.tensor([c.data_ptr() for kv in zip(self.k_cache, self.v_cache) for c in kv], dtype=torch.int64, device=self.device)
        return self._kv_ptrs

    def _kv_row_bytes(self) -> int:
        return self.k_cache[0].shape[-1] * self.k_cache[0].element_size()

    def _kv_scale_ptr_table(self):
        """int64 device tensor [2 * layers]: the per-token scale planes of an int8 cache, layer by layer."""
        if self._kv_scale_ptrs is None:
            self._kv_scale_ptrs = torch.tensor([c.data_ptr() for kv in zip(self.k_tscale, self.v_tscale) for c in kv], dtype=torch.int64, device=self.device)
        return self._kv_scale_ptrs

    def _kv_scale_row_bytes(self) -> int:
        t = self.k_tscale[0]
        return (t.shape[3] if t.ndim == 4 else 1) * t.element_size()

    def move_kv_rows(self, moves, n_moves: int) -> None:
        """moves: int32 device tensor [>= n_moves, 3] of (source slot, destination slot, rows), applied to the K and V caches of every layer
        in one launch (and to the scale planes of an int8 cache in another): the accepted path of a tree window goes from its nodes' slots
        to its positions."""
        self.K.kv_move_rows(self._kv_ptr_table(), self._kv_row_bytes(), self.cfg.n_kv, moves, n_moves)
        if self.kv_i8:
            self.K.kv_move_rows(self._kv_scale_ptr_table(), self._kv_scale_row_bytes(), self.cfg.n_kv, moves, n_moves)

    def mtp_forward(self, ids_next, hidden, positions, slots, row_seq, ctx_len, block_table, *, prefill=None, max_ctx=None, want_logits=True,
                    logit_rows=None):
        """The multi-token-prediction block over M rows: row r reads `hidden[r]` (bf16 [M, d]: the trunk's final residual of a position, or this
        block's own output when drafts are chained) and `ids_next[r]`, the token AFTER that position; positions / slots / ctx_len are the
        position's own (the block's KV cache is indexed like the trunk's).  Returns (logits of the shared head or None, the block's output
        residual rows: a view of a reused buffer).  Same kernels and the same row rules as a trunk layer."""
        if self.mtp is None:
            raise ValueError("this model has no multi-token-prediction block")
        cfg, K, m = self.cfg, self.K, self.mtp
        M = ids_next.shape[0]
        cls = "decode" if prefill is None else "prefill"
        assert M <= self.max_rows and (prefill is not None or M <= 256) and hidden.shape == (M, cfg.d_model) and hidden.dtype == torch.bfloat16
        d, F, HQ = cfg.d_model, cfg.ffn_padded, cfg.n_q * cfg.head_dim
        h, e = self.h_mtp[:M], self.e_mtp[:M]
        xr_d = self.xr[:M * d].view(M, d)
        xr_a = self.xr[:M * HQ].view(M, HQ)
        xr_f = self.xr2[:M * F].view(M, F)
        q = self.q[:M]
        Lm = m["layer"]
        if prefill is None and self.attn_plan is not None:
            K.attn_plan(row_seq, ctx_len, cfg.n_q, cfg.n_kv, self.window_seq_rows, self.attn_plan)
        self.pos3 = None
        K.embed(ids_next, self.embed, e)
        K.norm_rot_in(e, m["enorm"], cfg.eps, m["e_proj"].suh, xr_d)
        s = self._linear(xr_d, m["e_proj"], M, cls, "eh_proj")
        K.finish_store(self.part, s, M, m["e_proj"], h)
        K.norm_rot_in(hidden, m["hnorm"], cfg.eps, m["h_proj"].suh, xr_d)
        s = self._linear(xr_d, m["h_proj"], M, cls, "eh_proj")
        K.finish_add_norm_rot(self.part, s, M, m["h_proj"], h, Lm["attn_norm"], cfg.eps, Lm["qkv"].suh, xr_d)
        s = self._mixer(cfg.n_layers, Lm, M, cls, xr_d, xr_a, q, positions, slots, row_seq, ctx_len, block_table, prefill, max_ctx, 1.0 / math.sqrt(cfg.head_dim))
        self._ffn(cfg.n_layers, Lm, M, cls, s, h, xr_d, xr_f, m["final_norm"], self.lm_head.suh)
        if not want_logits:
            return None, h
        xl = xr_d if logit_rows is None else xr_d.index_select(0, logit_rows).contiguous()
        R = xl.shape[0]
        assert R <= self.logits.shape[0]
        s = self._linear(xl, self.lm_head, R, "decode", "lm_head")
        logits = self.logits[:R]
        K.finish_store(self.part, s, R, self.lm_head, logits)
        return logits, h

    def candidates(self, logits: torch.Tensor, count: int):
        """Top `count` (value desc, id asc) of each row, padded vocabulary columns excluded by construction (their logit is 0 * svh = 0
        only when vocab is not a multiple of 128; callers mask them with `vocab`)."""
        R = logits.shape[0]
        if self.cfg.vocab_padded != self.cfg.vocab:
            logits[:, self.cfg.vocab:] = float("-inf")
        self.K.topk(logits, count, self.topk_scratch, self._ids_view(R, count), self._vals_view(R, count))
        return self._ids_view(R, count), self._vals_view(R, count)

    def _ids_view(self, R, count):
        return self.cand_ids.view(-1)[:R * count].view(R, count)

    def _vals_view(self, R, count):
        return self.cand_vals.view(-1)[:R * count].view(R, count)

    def check(self, what="forward"):
        self.K.check_status(self.status, what)
        from ..utils import canary
        if canary.enabled():
            canary.check_all()
