"""Torch-facing wrappers of the sm_100a launchers.  Every function enqueues on the current CUDA stream, allocates
nothing (callers pass outputs and scratch) and raises :class:`KernelError` on a launch error."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import lib as _lib

CB_ID = {"3inst": 0, "mcg": 1, "mul1": 2}


@dataclass
class Exl3Weight:
    """One EXL3 linear layer on the device."""

    trellis: torch.Tensor          # int16 [K/16, N/16, 16*bits]
    suh: torch.Tensor              # float16 [K]
    svh: torch.Tensor              # float16 [N]
    bias: torch.Tensor | None      # float32 [N]
    codebook: str = "3inst"

    @property
    def K(self) -> int:
        return self.trellis.shape[0] * 16

    @property
    def N(self) -> int:
        return self.trellis.shape[1] * 16

    @property
    def twice(self) -> int:
        return self.trellis.shape[2] // 8

    @property
    def nbytes(self) -> int:
        return self.trellis.numel() * 2 + self.suh.numel() * 2 + self.svh.numel() * 2

    @staticmethod
    def from_numpy(trellis, suh, svh, bias=None, codebook="3inst", device="cuda") -> "Exl3Weight":
        return Exl3Weight(torch.from_numpy(np.ascontiguousarray(trellis)).to(device),
                          torch.from_numpy(np.ascontiguousarray(suh, dtype=np.float16)).to(device),
                          torch.from_numpy(np.ascontiguousarray(svh, dtype=np.float16)).to(device),
                          None if bias is None else torch.from_numpy(np.ascontiguousarray(bias, dtype=np.float32)).to(device), codebook)


STATUS_WORDS = 8
ST_TIMEOUT, ST_BAD_ARG, ST_PEER_TIMEOUT, ST_ABORTED = 1, 2, 3, 4
STATUS_NAMES = {ST_TIMEOUT: "wait timed out", ST_BAD_ARG: "bad argument", ST_PEER_TIMEOUT: "peer timed out", ST_ABORTED: "aborted by the host"}


def new_status(device="cuda") -> torch.Tensor:
    """Eight int32 status words.  Kernels write [code, site, block, aux] into the first four when a bounded wait runs out; the host may set
    word 4 (wait limit in microseconds, 0 = the 2 s default) and word 5 (abort: every polling wait gives up) before a launch."""
    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)


def set_wait_limit(status: torch.Tensor, microseconds: int) -> None:
    status[4] = int(microseconds)


def set_abort(status: torch.Tensor, on: bool = True) -> None:
    status[5] = 1 if on else 0


def check_status(status: torch.Tensor, what: str = "kernel") -> None:
    s = status.tolist()
    if s[0] != 0:
        raise _lib.KernelError(f"{what}: device status code {s[0]} ({STATUS_NAMES.get(s[0], '?')}) at site {s[1]} (block {s[2]}, aux {s[3]})")


def plan_splits(K: int, N: int, decode_class: bool) -> int:
    return _lib.load().rx_exl3_plan_splits(K, N, 1 if decode_class else 0)


def tile_rows(rows: int) -> int:
    """MMA N (rows per tile) the GEMM uses for a window of `rows` rows: 16..256."""
    return _lib.load().rx_exl3_tile_rows(rows)


def exl3_gemm(xr: torch.Tensor, w: Exl3Weight, part: torch.Tensor, splits: int, status: torch.Tensor, force_generic: bool = False) -> None:
    """part[s, row, n] = partial sums of xr @ W_q over split s.  xr: fp16 [rows, K] contiguous; part: fp32 >= splits*rows*N."""
    rows, K = xr.shape
    assert xr.dtype == torch.float16 and xr.is_contiguous() and K == w.K
    assert part.dtype == torch.float32 and part.numel() >= splits * rows * w.N
    L = _lib.load()
    if w.twice == 8 and not force_generic:
        # 4.0 bpw: decoded weights go straight to tensor memory
        _lib.check(L.rx_exl3_gemm_b4(xr.data_ptr(), rows, K, w.trellis.data_ptr(), w.N, CB_ID[w.codebook], part.data_ptr(), splits,
                                     status.data_ptr(), _lib.stream_ptr()), "rx_exl3_gemm_b4")
    else:
        _lib.check(L.rx_exl3_gemm(xr.data_ptr(), rows, K, w.trellis.data_ptr(), w.N, w.twice, CB_ID[w.codebook], part.data_ptr(), splits,
                                  status.data_ptr(), _lib.stream_ptr()), "rx_exl3_gemm")
    _lib.count()


def exl3_unpack(w: Exl3Weight) -> torch.Tensor:
    out = torch.empty(w.K, w.N, dtype=torch.float16, device=w.trellis.device)
    L = _lib.load()
    _lib.check(L.rx_exl3_unpack(w.trellis.data_ptr(), w.K, w.N, w.twice, CB_ID[w.codebook], out.data_ptr(), _lib.stream_ptr()), "rx_exl3_unpack")
    _lib.count()
    return out


def embed(ids: torch.Tensor, table: torch.Tensor, h: torch.Tensor) -> None:
    L = _lib.load()
    _lib.check(L.rx_embed(ids.data_ptr(), table.data_ptr(), h.data_ptr(), ids.numel(), table.shape[1], table.shape[0], _lib.stream_ptr()), "rx_embed")
    _lib.count()


def norm_rot_in(x: torch.Tensor, norm_w, eps: float, suh: torch.Tensor, xr: torch.Tensor) -> None:
    rows, K = x.shape
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    L = _lib.load()
    _lib.check(L.rx_norm_rot_in(x.data_ptr(), _lib.ptr(norm_w), eps, suh.data_ptr(), xr.data_ptr(), rows, K, _lib.stream_ptr()), "rx_norm_rot_in")
    _lib.count()


# modes of the recurrent mixers (bit 0: write outputs, bit 1: write the pools)
SCAN_RECORD, SCAN_COMMIT, SCAN_FINAL = 1, 2, 3


def ssm_mixer(proj: torch.Tensor, M: int, H: int, P: int, G: int, N: int, row_seq, positions, seg_start, seg_len, nseg: int, conv_w, conv_b, dt_bias,
              a_neg, d_skip, norm_w, eps: float, conv_pool, ssm_pool, xbc, y, out, mode: int = SCAN_FINAL) -> None:
    """Mamba2 mixer between in_proj and out_proj: `proj` f32 [M, ldp] (z | x | B | C | dt | pad) -> `out` bf16 [M, H*P] (gated, normed);
    the conv and state pools of the rows' sequences advance.  seg_start / seg_len: device int32 segment table or None (found on the device).
    Three launches (conv, recurrence, gated norm).  mode: SCAN_FINAL = rows are final (outputs and pools written); SCAN_RECORD = a window
    whose rows may be rejected (pools only read; the caller keeps `proj` and `xbc` as the record); SCAN_COMMIT = the recurrence again over
    the recorded rows of the segments given (seg_len = rows kept), pools written, one launch."""
    L = _lib.load()
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and out.dtype == torch.bfloat16
    _lib.check(L.rx_ssm_mixer(proj.data_ptr(), proj.stride(0), M, H, P, G, N, row_seq.data_ptr(), positions.data_ptr(), _lib.ptr(seg_start),
                              _lib.ptr(seg_len), nseg, conv_w.data_ptr(), conv_b.data_ptr(), dt_bias.data_ptr(), a_neg.data_ptr(), d_skip.data_ptr(),
                              norm_w.data_ptr(), eps, conv_pool.data_ptr(), ssm_pool.data_ptr(), xbc.data_ptr(), y.data_ptr(), out.data_ptr(),
                              _lib.stream_ptr(), mode), "rx_ssm_mixer")
    _lib.count(1 if mode == SCAN_COMMIT else 3)


def gdn_mixer(proj: torch.Tensor, M: int, Hk: int, Hv: int, D: int, row_seq, positions, seg_start, seg_len, nseg: int, conv_w, conv_b, dt_bias, a_neg,
              norm_w, eps: float, conv_pool, s_pool, xbc, out, kda: bool = False, mode: int = SCAN_FINAL, y32=None) -> None:
    """Gated delta net mixer between in_proj and out_proj: `proj` f32 [M, ldp] (z | q | k | v | b | a | pad) -> `out` bf16 [M, Hv*D]
    (per-head normed and gated); the conv and state pools of the rows' sequences advance.  Two launches (conv; recurrence + norm).
    `kda`: per-key-channel decay (a and dt_bias have Hv*D entries) and a sigmoid output gate.  `mode` as in `ssm_mixer`.  `y32` (f32 scratch
    of M * Hv * D values) with a segment table: the recurrence runs split over a head's value columns and the norm as its own launch (same bits)."""
    L = _lib.load()
    assert proj.dtype == torch.float32 and proj.stride(-1) == 1 and out.dtype == torch.bfloat16
    _lib.check(L.rx_gdn_mixer(proj.data_ptr(), proj.stride(0), M, Hk, Hv, D, row_seq.data_ptr(), positions.data_ptr(), _lib.ptr(seg_start),
                              _lib.ptr(seg_len), nseg, conv_w.data_ptr(), conv_b.data_ptr(), dt_bias.data_ptr(), a_neg.data_ptr(), norm_w.data_ptr(),
                              eps, conv_pool.data_ptr(), s_pool.data_ptr(), xbc.data_ptr(), out.data_ptr(), _lib.stream_ptr(), 1 if kda else 0,
                              mode, _lib.ptr(y32)), "rx_gdn_mixer")
    split = seg_start is not None and y32 is not None
    _lib.count(1 if mode == SCAN_COMMIT else (3 if split else 2))


def finish_store(part, S, M, w: Exl3Weight, out: torch.Tensor) -> None:
    L = _lib.load()
    f32 = 1 if out.dtype == torch.float32 else 0
    assert out.dtype in (torch.float32, torch.bfloat16)
    _lib.check(L.rx_finish_store(part.data_ptr(), S, M, w.N, w.svh.data_ptr(), _lib.ptr(w.bias), out.data_ptr(), f32, _lib.stream_ptr()),
               "rx_finish_store")
    _lib.count()


def finish_add_norm_rot(part, S, M, w: Exl3Weight, h: torch.Tensor, norm_w, eps: float, suh_next, xr, xn_out=None) -> None:
    L = _lib.load()
    _lib.check(L.rx_finish_add_norm_rot(part.data_ptr(), S, M, w.N, w.svh.data_ptr(), _lib.ptr(w.bias), h.data_ptr(), _lib.ptr(norm_w), eps,
                                        _lib.ptr(suh_next), _lib.ptr(xr), _lib.stream_ptr(), _lib.ptr(xn_out)), "rx_finish_add_norm_rot")
    _lib.count()


def finish_swiglu_rot(part, S, M, w: Exl3Weight, suh_down: torch.Tensor, xr: torch.Tensor) -> None:
    L = _lib.load()
    _lib.check(L.rx_finish_swiglu_rot(part.data_ptr(), S, M, w.N // 2, w.svh.data_ptr(), _lib.ptr(w.bias), suh_down.data_ptr(), xr.data_ptr(),
                                      _lib.stream_ptr()), "rx_finish_swiglu_rot")
    _lib.count()


def finish_qkv_rope(part, S, M, n_q, n_kv, hd, w: Exl3Weight, q_norm, k_norm, eps, positions, inv_freq, slot, q_out, k_cache, v_cache,
                    kv_scale=None, kv_amax=None, pos3=None, mrope_sections=None, kv_tscale=None, q4: bool = False) -> None:
    """kv_scale (f32 [2, n_kv]) given: the caches are FP8 (E4M3) and K, V are stored divided by their head's scale.  kv_amax (f32 [2, n_kv])
    given: the largest |K| and |V| per head are recorded there.  pos3 (int32 [rows, 3]: T, H, W position of every row) with
    mrope_sections = (t, h, w) frequency-pair counts: interleaved M-RoPE instead of `positions` (pair i uses axis i % 3 inside its section)."""
    kts, vts = kv_tscale if kv_tscale is not None else (None, None)     # int8 caches: per-token scales are written there
    # q4: the caches are uint8 [pages, n_kv, 64, hd / 2] nibbles and kv_tscale holds the E8M0 scale bytes uint8 [pages, n_kv, 64, hd / 32]
    assert not q4 or (kts is not None and kts.dtype == torch.uint8 and k_cache.dtype == torch.uint8 and k_cache.shape[-1] == hd // 2)
    sec = mrope_sections or (0, 0, 0)
    assert pos3 is None or (pos3.dtype == torch.int32 and pos3.is_contiguous() and pos3.shape[1] == 3 and sum(sec) == hd // 2)
    L = _lib.load()
    _lib.check(L.rx_finish_qkv_rope(part.data_ptr(), S, M, n_q, n_kv, hd, w.svh.data_ptr(), _lib.ptr(w.bias), _lib.ptr(q_norm), _lib.ptr(k_norm),
                                    eps, positions.data_ptr(), inv_freq.data_ptr(), slot.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(),
                                    v_cache.data_ptr(), _lib.stream_ptr(), _lib.ptr(kv_scale), _lib.ptr(kv_amax), _lib.ptr(pos3), int(sec[1]), int(sec[2]),
                                    _lib.ptr(kts), _lib.ptr(vts), 1 if q4 else 0), "rx_finish_qkv_rope")
    _lib.count()


def hc_mix(x: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scales, norm_w: torch.Tensor, coef: torch.Tensor, out: torch.Tensor, *,
           rms_eps: float = 1e-6, hc_eps: float = 1e-6, norm_eps: float = 1e-6, iters: int = 20) -> None:
    """Hyper-connection mix of one site: x f32 [rows, 4, D] -> coef f32 [rows, 24] (pre 4 | post 4 | comb 4x4 after Sinkhorn) and
    out bf16 [rows, D] = RMSNorm(sum_h pre[h] x[h]) * norm_w, the sublayer's input.  fn f32 [24, 4 * D], base f32 [24], scales (s0, s1, s2)."""
    rows, ns, D = x.shape
    assert ns == 4 and x.dtype == torch.float32 and x.is_contiguous() and fn.shape == (24, 4 * D) and fn.dtype == torch.float32 and fn.is_contiguous()
    assert coef.shape == (rows, 24) and coef.dtype == torch.float32 and out.shape == (rows, D) and out.dtype == torch.bfloat16 and norm_w.dtype == torch.bfloat16
    L = _lib.load()
    _lib.check(L.rx_hc_mix(x.data_ptr(), fn.data_ptr(), base.data_ptr(), float(scales[0]), float(scales[1]), float(scales[2]), norm_w.data_ptr(),
                           rms_eps, hc_eps, norm_eps, iters, rows, D, coef.data_ptr(), out.data_ptr(), _lib.stream_ptr()), "rx_hc_mix")
    _lib.count()


def hc_apply(x: torch.Tensor, y: torch.Tensor, coef: torch.Tensor) -> None:
    """x[h] <- post[h] y + sum_g comb[g][h] x[g], in place: x f32 [rows, 4, D], y f32 [rows, D] (the sublayer's output), coef from `hc_mix`."""
    rows, ns, D = x.shape
    assert ns == 4 and x.dtype == torch.float32 and x.is_contiguous() and y.shape == (rows, D) and y.dtype == torch.float32 and y.is_contiguous()
    L = _lib.load()
    _lib.check(L.rx_hc_apply(x.data_ptr(), y.data_ptr(), coef.data_ptr(), rows, D, _lib.stream_ptr()), "rx_hc_apply")
    _lib.count()


class Fp8Weight:
    """An FP8 block-scaled linear on the device: `w` E4M3 bytes uint8 [N, K], `scales` E8M0 bytes uint8 [N / 32, K / 32] (one power of two per
    32 x 32 tile), optional f32 bias [N] (reference crates/cuda/csrc/fp8_linear.cu:1)."""

    def __init__(self, w: torch.Tensor, scales: torch.Tensor, bias: "torch.Tensor | None" = None):
        N, Kd = w.shape
        if w.dtype != torch.uint8 or scales.dtype != torch.uint8 or N % 128 or Kd % 64 or tuple(scales.shape) != (N // 32, Kd // 32):
            raise ValueError("fp8 weight: uint8 [N, K] with N % 128 == 0, K % 64 == 0 and uint8 scales [N / 32, K / 32]")
        self.w, self.scales, self.bias, self.N, self.K = w.contiguous(), scales.contiguous(), bias, N, Kd
        self._part = None

    @staticmethod
    def quantize(dense: torch.Tensor, bias=None) -> "Fp8Weight":
        """dense f32 [N, K] -> the smallest power-of-two scale per 32 x 32 tile that brings the tile into the E4M3 range, values rounded to E4M3."""
        N, Kd = dense.shape
        t = dense.float().view(N // 32, 32, Kd // 32, 32)
        amax = t.abs().amax(dim=(1, 3)).clamp_min(2.0 ** -120)
        e = torch.ceil(torch.log2(amax / 448.0)).clamp(-126, 127)
        q = (t / torch.exp2(e)[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
        return Fp8Weight(q.view(torch.uint8).view(N, Kd), (e + 127).to(torch.uint8), bias)

    def dense(self) -> torch.Tensor:
        """The f32 matrix the bytes stand for (oracle side)."""
        N, Kd = self.w.shape
        v = self.w.view(torch.float8_e4m3fn).float().view(N // 32, 32, Kd // 32, 32)
        return (v * torch.exp2(self.scales.float() - 127.0)[:, None, :, None]).view(N, Kd)


def fp8_linear(x: torch.Tensor, w: Fp8Weight, status: torch.Tensor, out: "torch.Tensor | None" = None, out_dtype=torch.bfloat16, splits: int = 0) -> torch.Tensor:
    """y = x @ W^T (+ bias) for an FP8 block-scaled weight on the tcgen05 kernel: x bf16 [rows, K] -> y [rows, N] (bf16, fp16 or fp32).  The
    block scales are powers of two, so the weights are exact in the bf16 operand tiles; accumulation is fp32 in a fixed order."""
    rows, Kd = x.shape
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and Kd == w.K
    if splits < 1:      # few rows: split K until the grid covers the SMs (weight streaming); many rows: one pass
        ctas = (w.N // 128) * ((rows + 255) // 256)
        splits = max(1, min(Kd // 64, 8, 296 // max(1, ctas))) if rows <= 256 else 1
    tr = 16
    while tr < rows and tr < 256:
        tr *= 2
    L = _lib.load()
    need = L.rx_fp8_linear_scratch_floats(rows, w.N, splits)
    if w._part is None or w._part.numel() < need:
        w._part = torch.empty(need, dtype=torch.float32, device=x.device)
    if out is None:
        out = torch.empty(rows, w.N, dtype=out_dtype, device=x.device)
    code = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[out.dtype]
    _lib.check(L.rx_fp8_linear(x.data_ptr(), rows, Kd, w.w.data_ptr(), w.scales.data_ptr(), w.N, w._part.data_ptr(), splits, tr, _lib.ptr(w.bias),
                               out.data_ptr(), code, status.data_ptr(), _lib.stream_ptr()), "rx_fp8_linear")
    _lib.count(2)
    return out


def bf16_linear(x: torch.Tensor, weight: torch.Tensor, bias: "torch.Tensor | None" = None) -> torch.Tensor:
    """Plain bf16 linear y = x @ W^T (+ bias), fp32 accumulate: a LIBRARY GEMM (cuBLASLt through torch), for the tensors a pack keeps unquantised
    (vision towers, routers, small projections; reference crates/cuda/csrc/dsv4_bf16.cu).  Reduced-precision accumulation is switched off."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    return torch.nn.functional.linear(x, weight, bias)


def state_digest(tensors, out: "torch.Tensor | None" = None) -> torch.Tensor:
    """Position-keyed 64-bit content digest of one tensor or of a list of tensors (each part into its own word, the words then folded on the
    host by `fold_digest`).  Returns the int64 device tensor of per-part digests; nothing synchronises here."""
    parts = tensors if isinstance(tensors, (list, tuple)) else [tensors]
    L = _lib.load()
    if out is None:
        out = torch.zeros(len(parts), dtype=torch.int64, device=parts[0].device)
    else:
        out.zero_()
    for i, t in enumerate(parts):
        assert t.is_contiguous()
        _lib.check(L.rx_state_digest(t.data_ptr(), t.numel() * t.element_size(), out[i:].data_ptr(), _lib.stream_ptr()), "rx_state_digest")
        _lib.count()
    return out


def state_digest_host(data: bytes) -> int:
    """The same digest of a byte string on the host (numpy, wrap-around uint64 arithmetic): the oracle of `state_digest`."""
    import numpy as np
    n = len(data)
    buf = np.frombuffer(data + b"\0" * ((-n) % 8), dtype="<u8")
    with np.errstate(over="ignore"):
        i = np.arange(1, len(buf) + 1, dtype=np.uint64)
        z = buf ^ (i * np.uint64(0x9E3779B97F4A7C15))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
        return int(z.sum(dtype=np.uint64))


def fold_digest(words) -> int:
    """Per-part digests -> one 64-bit value that depends on the order of the parts."""
    acc = 0
    for w in words:
        acc = ((acc * 0x100000001B3) ^ (int(w) & 0xFFFFFFFFFFFFFFFF)) & 0xFFFFFFFFFFFFFFFF
    return acc


def topk_scratch(rows: int, vocab: int, count: int, device="cuda") -> torch.Tensor:
    n = _lib.load().rx_topk_scratch_bytes(rows, vocab, count)
    return torch.empty(n // 8 + 1, dtype=torch.int64, device=device)


def topk(logits: torch.Tensor, count: int, scratch, ids: torch.Tensor, vals: torch.Tensor) -> None:
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    L = _lib.load()
    _lib.check(L.rx_topk(logits.data_ptr(), rows, vocab, count, scratch.data_ptr(), ids.data_ptr(), vals.data_ptr(), _lib.stream_ptr()), "rx_topk")
    _lib.count(2)


class KvTensorMap:
    """Host-side TMA descriptor of one layer's K or V cache (bf16 [pages, n_kv, 64, hd])."""

    def __init__(self, cache: torch.Tensor):
        pages, n_kv, page, hd = cache.shape
        assert page == 64 and cache.dtype in (torch.bfloat16, torch.uint8, torch.int8) and cache.is_contiguous()
        self.buf = np.zeros(128, dtype=np.uint8)
        self._keep = cache
        self.fp8 = cache.dtype == torch.uint8          # E4M3 bytes
        self.i8 = cache.dtype == torch.int8            # int8 with one scale per (token, KV head), kept beside the cache
        L = _lib.load()
        if self.fp8 or self.i8:
            _lib.check(L.rx_make_kv_tmap8(self.buf.ctypes.data, cache.data_ptr(), pages * n_kv * page, hd), "rx_make_kv_tmap8")
        else:
            _lib.check(L.rx_make_kv_tmap(self.buf.ctypes.data, cache.data_ptr(), pages * n_kv * page, hd), "rx_make_kv_tmap")

    @property
    def ptr(self) -> int:
        return self.buf.ctypes.data


def attn_decode_scratch(rows: int, n_q: int, hd: int, max_ctx: int, device="cuda") -> torch.Tensor:
    n = _lib.load().rx_attn_decode_scratch_floats(rows, n_q, hd, max_ctx)
    return torch.empty(n, dtype=torch.float32, device=device)


def attn_decode(tk: KvTensorMap, tv: KvTensorMap, q, block_table, row_seq, ctx_len, scratch, n_q, n_kv, hd, max_ctx, scale, suh, xr, out,
                status, kv_scale=None, max_seq_rows: int = 1, plan=None, kv_tscale=None, q4: bool = False, vbt=None) -> None:
    """Split-KV decode / verify-window attention.  `max_seq_rows`: the most adjacent rows one sequence has in this window (1 + drafts); it
    picks how many MMA tiles a CTA carries so that a sequence's rows share one pass over its K / V (results do not depend on it).
    `plan`: the window plan from `attn_plan` for these rows and this `max_seq_rows` (one plan serves every layer of a forward); None has
    the call compute it itself.  `kv_tscale`: (K scales, V scales), f32 [pages, n_kv, 64] each, of an int8 cache.
    `vbt`: the rows' private page tables, int32 [rows, attn_vbt_width()], of a tree window whose plan was made with `tree_base`."""
    kts, vts = kv_tscale if kv_tscale is not None else (None, None)
    rows = q.shape[0]
    L = _lib.load()
    assert vbt is None or (plan is not None and not q4 and vbt.dtype == torch.int32 and vbt.shape[0] >= rows)
    if q4:      # E2M1 nibble pages (the maps are 64 bytes wide) + E8M0 scale bytes uint8 [pages, n_kv, 64, hd / 32]
        assert hd == 128 and kts is not None and kts.dtype == torch.uint8
        _lib.check(L.rx_attn_decode_q4(tk.ptr, tv.ptr, q.data_ptr(), block_table.data_ptr(), block_table.shape[1], row_seq.data_ptr(), ctx_len.data_ptr(),
                                       scratch.data_ptr(), rows, n_q, n_kv, hd, max_ctx, scale, _lib.ptr(suh), _lib.ptr(xr), _lib.ptr(out), status.data_ptr(),
                                       _lib.stream_ptr(), int(max_seq_rows), _lib.ptr(plan), kts.data_ptr(), vts.data_ptr()), "rx_attn_decode_q4")
        _lib.count(2 if plan is not None else 3)
        return
    assert tk.fp8 == (kv_scale is not None), "an FP8 cache needs its per-head scales (and only an FP8 cache takes them)"
    assert tk.i8 == (kv_tscale is not None), "an int8 cache needs its per-token scales (and only an int8 cache takes them)"
    _lib.check(L.rx_attn_decode(tk.ptr, tv.ptr, q.data_ptr(), block_table.data_ptr(), block_table.shape[1], row_seq.data_ptr(), ctx_len.data_ptr(),
                                scratch.data_ptr(), rows, n_q, n_kv, hd, max_ctx, scale, _lib.ptr(suh), _lib.ptr(xr), _lib.ptr(out),
                                status.data_ptr(), _lib.stream_ptr(), _lib.ptr(kv_scale), int(max_seq_rows), _lib.ptr(plan), _lib.ptr(kts), _lib.ptr(vts), _lib.ptr(vbt)), "rx_attn_decode")
    _lib.count(2 if plan is not None else 3)


def kv_move_rows(tensor_ptrs, row_bytes: int, n_kv: int, moves, n_moves: int) -> None:
    """Copies runs of cache rows, moves[i] = (source slot, destination slot, rows), in every cache whose base address is in `tensor_ptrs`
    (int64 device tensor); caches are [pages, n_kv, 64, row_bytes]; a run stays inside one page; no destination row is a source or a
    destination of another move.  moves: int32 device tensor [>= n_moves, 3]."""
    if n_moves <= 0:
        return
    L = _lib.load()
    _lib.check(L.rx_kv_move_rows(tensor_ptrs.data_ptr(), tensor_ptrs.numel(), int(row_bytes), int(n_kv), moves.data_ptr(), int(n_moves), _lib.stream_ptr()),
               "rx_kv_move_rows")
    _lib.count()


def attn_plan_buffer(device) -> torch.Tensor:
    return torch.zeros(_lib.load().rx_attn_plan_ints(), dtype=torch.int32, device=device)


def attn_vbt_width() -> int:
    return _lib.load().rx_attn_vbt_width()


def attn_plan(row_seq, ctx_len, n_q: int, n_kv: int, max_seq_rows: int, plan: torch.Tensor, tree_base=None) -> None:
    """The work plan of a decode / verify window: which adjacent rows of a sequence share a CTA, and the flat (block, chunk, kv head) item
    list the persistent attention kernel walks.  A function of row_seq and ctx_len only: compute once per forward.
    tree_base (int32 [rows]): the window's rows are nodes of draft trees; row r stands at position ctx_len[r] - 1 = tree_base[r] + depth.
    The chunks that end at or before tree_base are planned over the sequence's block-table row and shared by its rows; the later ones are
    planned per row over the row's private table (the `vbt` of attn_decode), whose entry 0 stands for page index
    (tree_base + 1) // chunk * (chunk // 64)."""
    L = _lib.load()
    _lib.check(L.rx_attn_plan(row_seq.data_ptr(), ctx_len.data_ptr(), row_seq.shape[0], n_q, n_kv, int(max_seq_rows), plan.data_ptr(), _lib.stream_ptr(),
                              _lib.ptr(tree_base)), "rx_attn_plan")
    _lib.count()


def attn_prefill(tk: KvTensorMap, tv: KvTensorMap, q, block_table, seq_ids, q_start, q_len, pos0, out, nseq, max_qlen, n_q, n_kv, hd, scale,
                 status, kv_scale=None, kv_tscale=None, q4: bool = False) -> None:
    kts, vts = kv_tscale if kv_tscale is not None else (None, None)
    L = _lib.load()
    if q4:
        assert hd == 128 and kts is not None and kts.dtype == torch.uint8
        _lib.check(L.rx_attn_prefill_q4(tk.ptr, tv.ptr, q.data_ptr(), block_table.data_ptr(), block_table.shape[1], seq_ids.data_ptr(), q_start.data_ptr(),
                                        q_len.data_ptr(), pos0.data_ptr(), out.data_ptr(), nseq, max_qlen, n_q, n_kv, hd, scale, status.data_ptr(),
                                        _lib.stream_ptr(), kts.data_ptr(), vts.data_ptr()), "rx_attn_prefill_q4")
        _lib.count()
        return
    assert tk.fp8 == (kv_scale is not None), "an FP8 cache needs its per-head scales (and only an FP8 cache takes them)"
    assert tk.i8 == (kv_tscale is not None), "an int8 cache needs its per-token scales (and only an int8 cache takes them)"
    _lib.check(L.rx_attn_prefill(tk.ptr, tv.ptr, q.data_ptr(), block_table.data_ptr(), block_table.shape[1], seq_ids.data_ptr(), q_start.data_ptr(),
                                 q_len.data_ptr(), pos0.data_ptr(), out.data_ptr(), nseq, max_qlen, n_q, n_kv, hd, scale, status.data_ptr(),
                                 _lib.stream_ptr(), _lib.ptr(kv_scale), _lib.ptr(kts), _lib.ptr(vts)), "rx_attn_prefill")
    _lib.count()


def attn_prefill_tc(tk: KvTensorMap, tv: KvTensorMap, q, block_table, seq_ids, q_start, q_len, pos0, out, nseq, max_qlen, n_q, n_kv, hd, scale,
                    status, v_desc_variant: int = 0) -> None:
    """The tcgen05 / TMEM prefill attention (bf16 caches, head_dim 128)."""
    assert not tk.fp8 and hd == 128
    L = _lib.load()
    _lib.check(L.rx_attn_prefill_tc(tk.ptr, tv.ptr, q.data_ptr(), block_table.data_ptr(), block_table.shape[1], seq_ids.data_ptr(), q_start.data_ptr(),
                                    q_len.data_ptr(), pos0.data_ptr(), out.data_ptr(), nseq, max_qlen, n_q, n_kv, hd, scale, status.data_ptr(),
                                    _lib.stream_ptr(), v_desc_variant), "rx_attn_prefill_tc")
    _lib.count()


# ------------------------------------------------------------------------------------------------ device-side verify / accept
SEQ_SAMPLING = np.dtype([("seed", "<u8"), ("temperature", "<f8"), ("top_p", "<f8"), ("min_p", "<f8"), ("top_k", "<i4"), ("first_row", "<i4"),
                         ("n_rows", "<i4"), ("position", "<i4")], align=True)


def verify_accept(ids: torch.Tensor, vals: torch.Tensor, windows, device="cuda"):
    """Keyed samples and accepted-draft counts of one window, on the device.

    ids / vals: the window's candidates [rows, count] (value desc, id asc).  windows: per sequence (sampling, position of the first
    sample, fed tokens [last, d1 .. dk]).  Returns (samples int32 [rows], accepted int32 [n_seqs], error flag int32 [1]) device tensors.
    """
    L = _lib.load()
    if SEQ_SAMPLING.itemsize != L.rx_verify_desc_size():
        raise _lib.KernelError("sampling descriptor layout mismatch")
    rows, count = ids.shape
    desc = np.zeros(len(windows), dtype=SEQ_SAMPLING)
    row_seq, fed, r = [], [], 0
    for i, (s, position, tokens) in enumerate(windows):
        desc[i] = (s.seed, s.temperature, s.top_p, s.min_p, s.top_k, r, len(tokens), position)
        row_seq += [i] * len(tokens)
        fed += [int(t) for t in tokens]
        r += len(tokens)
    assert r == rows
    d_desc = torch.from_numpy(desc.view(np.uint8)).to(device)
    d_seq = torch.tensor(row_seq, dtype=torch.int32, device=device)
    d_fed = torch.tensor(fed, dtype=torch.int32, device=device)
    samples = torch.empty(rows, dtype=torch.int32, device=device)
    accepted = torch.empty(len(windows), dtype=torch.int32, device=device)
    err = torch.zeros(1, dtype=torch.int32, device=device)
    _lib.check(L.rx_verify_accept(ids.data_ptr(), vals.data_ptr(), rows, count, d_desc.data_ptr(), len(windows), d_seq.data_ptr(), d_fed.data_ptr(),
                                  samples.data_ptr(), accepted.data_ptr(), err.data_ptr(), _lib.stream_ptr()), "rx_verify_accept")
    _lib.count()
    return samples, accepted, err
