"""Bindings of the native trellis encoder (tail-biting Viterbi over 65,536 states, ``native/csrc/trellis_encode.cpp``)."""
from __future__ import annotations

import ctypes
import os

import numpy as np

from ..format import exl3

_lib = None


def _load():
    global _lib
    if _lib is None:
        from ..native import build as nb
        path = nb.OUT if os.path.exists(nb.OUT) else nb.build()
        _lib = ctypes.CDLL(path)
        _lib.rx_trellis_encode.restype = ctypes.c_int
        _lib.rx_trellis_encode.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    return _lib


def encode_tiles(tiles: np.ndarray, bits: exl3.Bits, codebook: str, threads: int = 0):
    """tiles float32 [T, 256] in stream order -> (int16 [T, 16*bits], squared error per tile)."""
    tiles = np.ascontiguousarray(tiles, dtype=np.float32)
    t = tiles.shape[0]
    table = np.ascontiguousarray(exl3.codebook_f32(codebook), dtype=np.float32)
    out = np.zeros((t, bits.tile_words), dtype=np.int16)
    err = np.zeros(t, dtype=np.float32)
    rc = _load().rx_trellis_encode(tiles.ctypes.data, t, bits.twice, table.ctypes.data, out.ctypes.data, err.ctypes.data, threads)
    if rc != 0:
        raise ValueError("trellis encoder refused its arguments")
    return out, err


def encode_tiles_cuda(tiles, bits: exl3.Bits, codebook: str, ctas: int = 148, device="cuda"):
    """The same search on the GPU (one CTA per tile, bit-identical to `encode_tiles`).  tiles: float32 [T, 256] (array or device tensor)
    in stream order -> (int16 device tensor [T, 16*bits], squared error per tile)."""
    import torch
    from ..ops import lib as _oplib
    L = _oplib.load()
    t = torch.as_tensor(tiles, dtype=torch.float32).to(device).contiguous()
    T = t.shape[0]
    table = torch.from_numpy(np.ascontiguousarray(exl3.codebook_f32(codebook), dtype=np.float32)).to(device)
    out = torch.zeros(T, bits.tile_words, dtype=torch.int16, device=device)
    err = torch.zeros(T, dtype=torch.float32, device=device)
    ctas = max(1, min(ctas, T))
    scratch = torch.empty(L.rx_trellis_encode_scratch_bytes(ctas), dtype=torch.uint8, device=device)
    _oplib.check(L.rx_trellis_encode_cuda(t.data_ptr(), T, bits.twice, table.data_ptr(), out.data_ptr(), err.data_ptr(), scratch.data_ptr(), ctas,
                                          _oplib.stream_ptr()), "rx_trellis_encode_cuda")
    _oplib.count()
    return out, err
