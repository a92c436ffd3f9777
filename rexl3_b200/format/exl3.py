"""EXL3 trellis format: bit-exact CPU codec and float64 reference layer.

Layer:   y = ((((x * suh) @ H_K) @ W_q) @ H_N) * svh + bias
         H = block-diagonal 128x128 Sylvester Hadamard / sqrt(128).
Storage: trellis int16 [K/16, N/16, 16*bits]; a 16x16 tile is a circular,
         MSB-first bit ring of 256*bits bits; value p is the 16-bit window
         that ENDS at bit E(p), mapped through a codebook to fp16.

Behaviour parity: reference crates/exl3/src/lib.rs:20-33 (constants),
:64-103 (widths, E(p)), :105-154 (codebooks, tile order, window read),
:193-260 (rotation + reference layer), crates/exl3/src/encode.rs:44-72
(packer).  Everything here is vectorised numpy; the C++ twin in
``rexl3_b200/native`` and the CUDA kernels are checked against it.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import numpy as np

HAD = 128
INST3_MUL = 89226354
INST3_ADD = 64248484
MCG_MUL = 0xCBAC1FED
MUL1_MUL = 0x83DCD12D
MASK = 0x8FFF8FFF
FLIP = 0x3B603B60
MUL1_SCALE = 0x1EEE  # fp16 bits
MUL1_BIAS = 0xC931  # fp16 bits
MARKER_MCG = 0xCBAC1FED
MARKER_MUL1 = 0x83DCD12D

CODEBOOKS = ("3inst", "mcg", "mul1")
#: every width the format allows, doubled so the half widths are exact
ALL_TWICE = (2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16)


@dataclass(frozen=True, order=True)
class Bits:
    """Bits per weight, stored doubled (3 == 1.5 bpw)."""

    twice: int

    def __post_init__(self):
        if self.twice not in ALL_TWICE:
            raise ValueError(f"unsupported EXL3 width {self.twice / 2}")

    @staticmethod
    def of(bpw: float) -> "Bits":
        t = int(round(bpw * 2))
        if abs(t - bpw * 2) > 1e-9:
            raise ValueError(f"EXL3 width {bpw} is not a multiple of 0.5")
        return Bits(t)

    @staticmethod
    def from_trellis_last(last: int) -> "Bits":
        if last % 8 != 0:
            raise ValueError(f"trellis last dim {last} is not 16*bits")
        return Bits(last // 8)

    @property
    def value(self) -> float:
        return self.twice / 2.0

    @property
    def is_integer(self) -> bool:
        return self.twice % 2 == 0

    @property
    def tile_words(self) -> int:
        """int16 words per 16x16 tile (= 16 * bits)."""
        return 8 * self.twice

    def stream_ends(self) -> np.ndarray:
        """E(p), p = 0..255: exclusive end bit of value p's 16-bit window."""
        p1 = np.arange(1, 257, dtype=np.int64)
        if self.is_integer:
            return p1 * (self.twice // 2)
        return (p1 * self.twice - (p1 % 2)) // 2


def fnv1a(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def fnv1a_u16(a: np.ndarray) -> int:
    return fnv1a(np.ascontiguousarray(a, dtype="<u2").tobytes())


@lru_cache(maxsize=None)
def codebook(name: str) -> np.ndarray:
    """fp16 bit pattern (uint16[65536]) of every 16-bit state."""
    s = np.arange(65536, dtype=np.uint64)
    if name == "mul1":
        x = (s * np.uint64(MUL1_MUL)) & np.uint64(0xFFFFFFFF)
        h = 1024 + (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + ((x >> 24) & 255)
        scale = np.array([MUL1_SCALE], dtype=np.uint16).view(np.float16).astype(np.float64)[0]
        bias = np.array([MUL1_BIAS], dtype=np.uint16).view(np.float16).astype(np.float64)[0]
        v = h.astype(np.float64) * scale + bias  # exact in f64 -> one rounding
        out = v.astype(np.float16).view(np.uint16)
    elif name in ("3inst", "mcg"):
        if name == "mcg":
            x = (s * np.uint64(MCG_MUL)) & np.uint64(0xFFFFFFFF)
        else:
            x = (s * np.uint64(INST3_MUL) + np.uint64(INST3_ADD)) & np.uint64(0xFFFFFFFF)
        x = (x & np.uint64(MASK)) ^ np.uint64(FLIP)
        lo = (x & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
        hi = (x >> 16).astype(np.uint16).view(np.float16).astype(np.float64)
        out = (lo + hi).astype(np.float16).view(np.uint16)
    else:
        raise ValueError(f"unknown codebook {name!r}")
    out.setflags(write=False)
    return out


def codebook_f32(name: str) -> np.ndarray:
    return codebook(name).view(np.float16).astype(np.float32)


@lru_cache(maxsize=None)
def tile_positions():
    """(row, col) inside the 16x16 tile of stream position p (k = row, n = col)."""
    p = np.arange(256)
    lane, j = p // 8, p % 8
    r = 2 * (lane % 4) + (j & 1) + 8 * ((j >> 1) & 1)
    c = lane // 4 + 8 * (j >> 2)
    return r.astype(np.int64), c.astype(np.int64)


def _words32(tiles: np.ndarray) -> np.ndarray:
    """int16 [..., 16*bits] -> uint64 32-bit words [..., 8*bits] (word i = u16[2i] | u16[2i+1] << 16)."""
    u = np.ascontiguousarray(tiles).view(np.uint16).astype(np.uint64)
    return u[..., 0::2] | (u[..., 1::2] << np.uint64(16))


def states(tiles: np.ndarray, bits: Bits) -> np.ndarray:
    """16-bit state of each of the 256 values of every tile. tiles: int16 [..., 16*bits] -> uint16 [..., 256]."""
    tiles = np.asarray(tiles)
    if tiles.shape[-1] != bits.tile_words:
        raise ValueError("tile must hold 16 * bits int16 words")
    words = _words32(tiles)
    nw = words.shape[-1]
    ring = 32 * nw
    first = bits.stream_ends() + ring - 16
    i0 = (first // 32) % nw
    off = (first % 32).astype(np.uint64)
    i1 = (i0 + 1) % nw
    pair = (words[..., i0] << np.uint64(32)) | words[..., i1]
    return ((pair >> (np.uint64(48) - off)) & np.uint64(0xFFFF)).astype(np.uint16)


def unpack(trellis: np.ndarray, table: np.ndarray | str = "3inst") -> np.ndarray:
    """W_q as fp16 bits, uint16 [K, N], from trellis int16 [K/16, N/16, 16*bits]."""
    trellis = np.asarray(trellis)
    kt, nt, last = trellis.shape
    bits = Bits.from_trellis_last(last)
    if isinstance(table, str):
        table = codebook(table)
    st = states(trellis, bits)  # [kt, nt, 256]
    vals = table[st]
    r, c = tile_positions()
    w = np.empty((kt, 16, nt, 16), dtype=np.uint16)
    w[:, r, :, c] = np.moveaxis(vals, 2, 0)
    return w.reshape(kt * 16, nt * 16)


def unpack_f32(trellis: np.ndarray, cb: str = "3inst") -> np.ndarray:
    return unpack(trellis, cb).view(np.float16).astype(np.float32)


def unpack_signs(packed: np.ndarray) -> np.ndarray:
    """su / sv packed signs int16 [n/16] -> +-1.0 float64 [n]; bit b of word w set => element 16w+b is -1."""
    w = np.asarray(packed).view(np.uint16).astype(np.int64)
    b = (w[:, None] >> np.arange(16)) & 1
    return np.where(b.reshape(-1) == 1, -1.0, 1.0)


@lru_cache(maxsize=None)
def hadamard128(dtype=np.float64) -> np.ndarray:
    """128x128 Sylvester Hadamard / sqrt(128): sign = (-1)^popcount(i & j)."""
    i = np.arange(HAD)
    a = i[:, None] & i[None, :]
    pc = np.zeros_like(a)
    for b in range(7):
        pc += (a >> b) & 1
    return (np.where(pc & 1, -1.0, 1.0) / np.sqrt(HAD)).astype(dtype)


def rotate(x: np.ndarray) -> np.ndarray:
    """Apply H/sqrt(128) to every 128-block of the last axis."""
    x = np.asarray(x)
    n = x.shape[-1]
    if n % HAD:
        raise ValueError("rotated dimension must be a multiple of 128")
    h = hadamard128(np.float64 if x.dtype == np.float64 else np.float32)
    y = x.reshape(*x.shape[:-1], n // HAD, HAD) @ h
    return y.reshape(x.shape)


def forward(x, trellis, cb="3inst", suh=None, svh=None, bias=None) -> np.ndarray:
    """Float64 reference layer. x [rows, K] -> [rows, N]."""
    x = np.asarray(x, dtype=np.float64)
    wq = unpack(trellis, cb).view(np.float16).astype(np.float64)
    k, n = wq.shape
    suh = np.ones(k) if suh is None else np.asarray(suh, dtype=np.float64)
    svh = np.ones(n) if svh is None else np.asarray(svh, dtype=np.float64)
    y = rotate(rotate(x * suh) @ wq) * svh
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)
    return y


def decode_weight(trellis, cb="3inst", suh=None, svh=None, dtype=np.float64) -> np.ndarray:
    """Effective dense weight [K, N] with forward(x) == x @ W."""
    wq = unpack(trellis, cb).view(np.float16).astype(np.float64)
    k, n = wq.shape
    suh = np.ones(k) if suh is None else np.asarray(suh, dtype=np.float64)
    svh = np.ones(n) if svh is None else np.asarray(svh, dtype=np.float64)
    # H_K W_q (per column, blocks of 128 rows); H symmetric so rotate the transpose's last axis
    w = rotate(wq.T.copy()).T
    w = w * suh[:, None]
    w = rotate(w) * svh[None, :]
    return w.astype(dtype)


def decode_strip(trellis, strip: int, cb="3inst", suh=None, svh=None) -> np.ndarray:
    """Columns [128*strip, 128*strip+128) of decode_weight, decoding only that strip's tiles."""
    trellis = np.asarray(trellis)
    sub = trellis[:, strip * 8:(strip + 1) * 8, :]
    sv = None if svh is None else np.asarray(svh)[strip * HAD:(strip + 1) * HAD]
    return decode_weight(sub, cb, suh, sv)


# ----------------------------------------------------------------------------- packer (inverse of states)

def pack_tile(st: np.ndarray, bits: Bits) -> np.ndarray:
    """Write 256 16-bit states into one tile's bit ring; raises if windows disagree on shared bits.

    st: uint16 [256] -> int16 [16*bits].
    """
    return pack_tiles(np.asarray(st)[None, :], bits)[0]


def pack_tiles(st: np.ndarray, bits: Bits, check: bool = True) -> np.ndarray:
    """Vectorised packer. st: uint16 [T, 256] -> int16 [T, 16*bits].

    Each value contributes its newest bits (the ones no earlier window ends on); the tail-biting
    consistency (shared bits agree) is verified by decoding the result when ``check``.
    """
    st = np.asarray(st, dtype=np.uint16)
    t = st.shape[0]
    nbits = 256 * bits.twice // 2
    ends = bits.stream_ends()
    starts = np.concatenate([[0], ends[:-1]])
    ring = np.zeros((t, nbits), dtype=np.uint8)
    for p in range(256):
        nb = int(ends[p] - starts[p])  # new bits this value brings (low nb bits of the state)
        v = st[:, p].astype(np.uint32)
        for b in range(nb):
            ring[:, starts[p] + b] = (v >> (nb - 1 - b)) & 1
    words = np.packbits(ring.reshape(t, nbits // 32, 32), axis=-1, bitorder="big")  # [T, nw, 4] big-endian bytes
    w32 = (words[..., 0].astype(np.uint32) << 24) | (words[..., 1].astype(np.uint32) << 16) | \
          (words[..., 2].astype(np.uint32) << 8) | words[..., 3].astype(np.uint32)
    out = np.empty((t, nbits // 16), dtype=np.uint16)
    out[:, 0::2] = w32 & 0xFFFF
    out[:, 1::2] = w32 >> 16
    out = out.view(np.int16)
    if check:
        back = states(out, bits)
        if not np.array_equal(back, st):
            bad = np.argwhere(back != st)[0]
            raise ValueError(f"states are not a valid trellis path (tile {bad[0]}, position {bad[1]})")
    return out


def random_trellis(kt: int, nt: int, bits: Bits, seed: int = 0) -> np.ndarray:
    """Any random bit ring is a valid tile: random-init EXL3 weights for tests and benches."""
    rng = np.random.default_rng(seed)
    return rng.integers(-32768, 32768, size=(kt, nt, bits.tile_words), dtype=np.int16)


def splitmix_stream(seed: int, n: int) -> np.ndarray:
    """n outputs of the splitmix64 generator the conformance fixtures use (uint64)."""
    out = np.empty(n, dtype=np.uint64)
    s = seed & 0xFFFFFFFFFFFFFFFF
    m = 0xFFFFFFFFFFFFFFFF
    for i in range(n):
        s = (s + 0x9E3779B97F4A7C15) & m
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        out[i] = z ^ (z >> 31)
    return out
