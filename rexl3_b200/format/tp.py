"""Tensor-parallel width splitting of EXL3 layers at whole 128-column tiles.

Rules (behaviour parity: reference crates/exl3/src/tp.rs:39-123): ``floor`` gives rank r the tiles
[floor(B r / R), floor(B (r+1) / R)); ``uneven`` gives the extra tiles to the low ranks; ``uniform`` pads
with dummy zero tiles so every rank runs the same width.  Every tile lands on exactly one rank and the
skew between two ranks is at most one tile.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

TILE = 128


def tile_cut(tiles: int, rank: int, ranks: int):
    if ranks < 1 or not 0 <= rank < ranks:
        raise ValueError(f"rank {rank} out of {ranks}")
    return tiles * rank // ranks, tiles * (rank + 1) // ranks


@dataclass
class WidthSplit:
    tiles: list
    width: int
    dummy: int = 0

    def cols(self):
        real = len(self.tiles) - self.dummy
        lo = self.tiles[0] * TILE if self.tiles else 0
        return lo, lo + real * TILE


def split_width(n: int, r: int, ranks: int, mode: str = "floor") -> WidthSplit:
    if ranks < 1 or not 0 <= r < ranks:
        raise ValueError(f"rank {r} out of {ranks}")
    if n % TILE:
        raise ValueError(f"width {n} is not a multiple of the {TILE} tile")
    b = n // TILE
    if mode == "uneven":
        base, rem = divmod(b, ranks)
        start = r * base + min(r, rem)
        ln = base + (1 if r < rem else 0)
        return WidthSplit(list(range(start, start + ln)), ln * TILE, 0)
    if mode == "floor":
        lo, hi = tile_cut(b, r, ranks)
        return WidthSplit(list(range(lo, hi)), (hi - lo) * TILE, 0)
    if mode == "uniform":
        per = -(-b // ranks)
        lo, hi = r * per, (r + 1) * per
        return WidthSplit(list(range(lo, hi)), per * TILE, min(max(hi - b, 0), per))
    raise ValueError(f"unknown split mode {mode!r}")


def slice_columns(trellis: np.ndarray, svh: np.ndarray, bias, split: WidthSplit):
    """A rank's column (N) slice of a layer: trellis [K/16, n_r/16, w], svh [n_r], bias [n_r]; dummy tiles are zero."""
    lo, hi = split.cols()
    t = trellis[:, lo // 16:hi // 16, :]
    s = svh[lo:hi]
    b = None if bias is None else bias[lo:hi]
    pad = split.dummy * TILE
    if pad:
        t = np.concatenate([t, np.zeros((t.shape[0], pad // 16, t.shape[2]), t.dtype)], axis=1)
        s = np.concatenate([s, np.zeros(pad, s.dtype)])
        if b is not None:
            b = np.concatenate([b, np.zeros(pad, b.dtype)])
    return np.ascontiguousarray(t), np.ascontiguousarray(s), b


def slice_rows(trellis: np.ndarray, suh: np.ndarray, split: WidthSplit):
    """A rank's input (K) slice for row-parallel layers: whole 128-row Hadamard blocks, so the input rotation stays local."""
    lo, hi = split.cols()
    return np.ascontiguousarray(trellis[lo // 16:hi // 16]), np.ascontiguousarray(suh[lo:hi])
