"""MXFP4 block-scaled weights: E2M1 nibbles with one E8M0 scale per 32 elements.

Layout (behaviour parity: reference crates/cuda/csrc/fp4_linear.cu:5-18,36-44): W int8 [n, k/2], element 2i in
the low nibble and 2i+1 in the high nibble, nibble = magnitude | sign << 3, magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6};
scales uint8 [n, k/32] meaning 2^(b-127), 0xFF = NaN.
"""
from __future__ import annotations

import numpy as np

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
BLOCK = 32


def e8m0_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    out = np.ldexp(np.float32(1.0), b.astype(np.int32) - 127).astype(np.float32)
    return np.where(b == 0xFF, np.float32(np.nan), out)


def dequant(w: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """int8/uint8 [n, k/2] + uint8 [n, k/32] -> float32 [n, k]."""
    w = np.asarray(w).view(np.uint8)
    n, k2 = w.shape
    nib = np.empty((n, k2 * 2), dtype=np.uint8)
    nib[:, 0::2] = w & 0xF
    nib[:, 1::2] = w >> 4
    v = E2M1[nib & 7] * np.where(nib & 8, np.float32(-1), np.float32(1))
    s = e8m0_to_f32(scales)
    return (v.reshape(n, -1, BLOCK) * s[:, :, None]).reshape(n, k2 * 2)


def quantize(w: np.ndarray):
    """float [n, k] -> (int8 [n, k/2], uint8 scales [n, k/32]); scale = 2^(floor(log2(amax)) - 2) as in the OCP MX spec."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    if k % BLOCK:
        raise ValueError(f"k={k} is not a multiple of {BLOCK}")
    blk = w.reshape(n, k // BLOCK, BLOCK)
    amax = np.abs(blk).max(axis=-1)
    e = np.where(amax > 0, np.floor(np.log2(np.maximum(amax, 1e-38))) - 2, -127).astype(np.int32)
    e = np.clip(e, -127, 127)
    scale = np.ldexp(np.float32(1.0), e)
    x = blk / scale[:, :, None]
    mag = np.abs(x)
    # round to nearest E2M1 magnitude (ties to the even mantissa = lower index on exact midpoints handled by argmin order)
    idx = np.abs(mag[..., None] - E2M1).argmin(axis=-1).astype(np.uint8)
    nib = (idx | np.where(x < 0, 8, 0).astype(np.uint8)).reshape(n, k)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return packed.view(np.int8), (e + 127).astype(np.uint8)
