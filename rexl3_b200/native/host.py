"""ctypes bindings of the host-side native library (``librexl3_host.so``): the EXL3 codec twin of `rexl3_b200.format.exl3`
(states / unpack / effective weight, multi-threaded) and the parallel file-range reader used when a pack is loaded."""
from __future__ import annotations

import ctypes
import os

import numpy as np

from ..format import exl3

_lib = None


def lib():
    global _lib
    if _lib is None:
        from . import build as nb
        path = nb.build()                 # rebuilds only when a source is newer than the library
        L = ctypes.CDLL(path)
        c_int, c_void = ctypes.c_int, ctypes.c_void_p
        L.rx_exl3_states_host.restype = c_int
        L.rx_exl3_states_host.argtypes = [c_void, c_int, c_int, c_int, c_void, c_int]
        L.rx_exl3_unpack_host.restype = c_int
        L.rx_exl3_unpack_host.argtypes = [c_void, c_int, c_int, c_int, c_void, c_void, c_int]
        L.rx_exl3_decode_weight_host.restype = c_int
        L.rx_exl3_decode_weight_host.argtypes = [c_void, c_int, c_int, c_int, c_void, c_void, c_void, c_void, c_int]
        L.rx_read_ranges.restype = c_int
        L.rx_read_ranges.argtypes = [ctypes.c_char_p, c_int, c_void, c_void, c_void, c_int, c_int, ctypes.POINTER(c_int)]
        L.rx_bpe_new.restype = c_void
        L.rx_bpe_new.argtypes = [c_void, c_void, c_int]
        L.rx_bpe_free.restype = None
        L.rx_bpe_free.argtypes = [c_void]
        L.rx_bpe_encode.restype = ctypes.c_int64
        L.rx_bpe_encode.argtypes = [c_void, c_void, c_void, c_int, c_void, ctypes.c_int64]
        L.rx_pretok_split.restype = ctypes.c_int64
        L.rx_pretok_split.argtypes = [c_int, c_void, ctypes.c_int64, c_void, ctypes.c_int64]
        L.rx_bpe_encode_text.restype = ctypes.c_int64
        L.rx_bpe_encode_text.argtypes = [c_void, c_int, c_void, ctypes.c_int64, c_void, ctypes.c_int64]
        _lib = L
    return _lib


def _trellis(trellis):
    t = np.ascontiguousarray(trellis, dtype=np.int16)
    if t.ndim != 3:
        raise ValueError("trellis is int16 [K/16, N/16, 16*bits]")
    return t, exl3.Bits.from_trellis_last(t.shape[2])


def states(trellis, threads: int = 0) -> np.ndarray:
    t, b = _trellis(trellis)
    out = np.empty(t.shape[:2] + (256,), dtype=np.uint16)
    if lib().rx_exl3_states_host(t.ctypes.data, t.shape[0], t.shape[1], b.twice, out.ctypes.data, threads) != 0:
        raise ValueError("native codec refused its arguments")
    return out


def unpack(trellis, codebook: str = "3inst", threads: int = 0) -> np.ndarray:
    """W_q as fp16 bit patterns, uint16 [K, N] (the twin of `exl3.unpack`)."""
    t, b = _trellis(trellis)
    table = np.ascontiguousarray(exl3.codebook(codebook))
    out = np.empty((t.shape[0] * 16, t.shape[1] * 16), dtype=np.uint16)
    if lib().rx_exl3_unpack_host(t.ctypes.data, t.shape[0], t.shape[1], b.twice, table.ctypes.data, out.ctypes.data, threads) != 0:
        raise ValueError("native codec refused its arguments")
    return out


def decode_weight(trellis, codebook: str = "3inst", suh=None, svh=None, threads: int = 0) -> np.ndarray:
    """Effective dense float64 weight [K, N] (the twin of `exl3.decode_weight`; equal to rounding, butterflies instead of matrix products)."""
    t, b = _trellis(trellis)
    table = np.ascontiguousarray(exl3.codebook(codebook))
    su = None if suh is None else np.ascontiguousarray(suh, dtype=np.float64)
    sv = None if svh is None else np.ascontiguousarray(svh, dtype=np.float64)
    out = np.empty((t.shape[0] * 16, t.shape[1] * 16), dtype=np.float64)
    rc = lib().rx_exl3_decode_weight_host(t.ctypes.data, t.shape[0], t.shape[1], b.twice, table.ctypes.data, None if su is None else su.ctypes.data,
                                          None if sv is None else sv.ctypes.data, out.ctypes.data, threads)
    if rc != 0:
        raise ValueError("native codec refused its arguments (K and N must be multiples of 128)")
    return out


def read_ranges(path: str, offsets, sizes, dst: np.ndarray, dst_offsets, threads: int = 8, direct: bool = False) -> bool:
    """Fill `dst` (a writable uint8 array, e.g. over pinned memory) at `dst_offsets` with the file ranges.  Returns whether O_DIRECT was used
    (a file system that refuses it falls back to buffered reads).  Raises OSError on any failure."""
    n = len(offsets)
    offs = np.ascontiguousarray(offsets, dtype=np.int64)
    szs = np.ascontiguousarray(sizes, dtype=np.int64)
    dofs = np.ascontiguousarray(dst_offsets, dtype=np.int64)
    if dst.dtype != np.uint8 or not dst.flags.c_contiguous or not dst.flags.writeable:
        raise ValueError("dst is a writable contiguous uint8 array")
    if n and int((dofs + szs).max()) > dst.nbytes:
        raise ValueError("a range does not fit the destination")
    ptrs = (dst.ctypes.data + dofs).astype(np.uint64)
    used = ctypes.c_int(0)
    rc = lib().rx_read_ranges(os.fsencode(path), n, offs.ctypes.data, szs.ctypes.data, ptrs.ctypes.data, threads, 1 if direct else 0, ctypes.byref(used))
    if rc != 0:
        raise OSError(rc, f"{os.strerror(rc)}: {path}")
    return bool(used.value)


# The split patterns the native pre-tokenizer implements (native/csrc/pretok.cpp), by the regular expression a tokenizer file spells them with.
_GPT2 = r"""'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
_GPT2_B = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
_CL100K = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
_QWEN2 = r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"""
PRETOK_KINDS = {_GPT2: 0, _GPT2_B: 0, _CL100K: 1, _QWEN2: 2}


def pretok_kind(pattern: str):
    """-> the native pattern id of a split regular expression, or None when the scanner does not implement it (the caller keeps `regex`)."""
    return PRETOK_KINDS.get(pattern)


def pretok_split(text: str, kind: int) -> list:
    """The pieces of `text` under native pattern `kind` (tests compare this with the `regex` oracle)."""
    raw = text.encode("utf-8")
    buf = np.frombuffer(raw, dtype=np.uint8) if raw else np.zeros(1, dtype=np.uint8)
    offs = np.empty(len(raw) + 2, dtype=np.int64)
    n = lib().rx_pretok_split(kind, buf.ctypes.data, len(raw), offs.ctypes.data, offs.size)
    if n < 1 or n > offs.size:
        raise ValueError("native pre-tokenizer refused its arguments")
    o = offs[:n].tolist()
    return [raw[a:b].decode("utf-8") for a, b in zip(o[:-1], o[1:])]


class BpeCore:
    """Ranked byte-level BPE merges on token ids (`native/csrc/bpe.cpp`).  byte_ids: the token id of each of the 256 bytes (-1: none);
    merges: (left id, right id, merged id) triples in rank order."""

    def __init__(self, byte_ids, merges):
        self._b = np.ascontiguousarray(byte_ids, dtype=np.int32)
        m = np.ascontiguousarray(merges, dtype=np.int32).reshape(-1, 3)
        if self._b.shape != (256,):
            raise ValueError("byte_ids has 256 entries")
        self._h = lib().rx_bpe_new(self._b.ctypes.data, m.ctypes.data, m.shape[0])
        self._free = lib().rx_bpe_free

    def encode_pieces(self, pieces) -> list:
        """pieces: iterable of bytes objects (the pre-tokenizer's output) -> token ids of their concatenation."""
        pieces = list(pieces)
        if not pieces:
            return []
        offs = np.zeros(len(pieces) + 1, dtype=np.int64)
        np.cumsum([len(p) for p in pieces], out=offs[1:])
        buf = np.frombuffer(b"".join(pieces), dtype=np.uint8)
        out = np.empty(max(int(offs[-1]), 1), dtype=np.int32)       # a piece never yields more tokens than it has bytes
        n = lib().rx_bpe_encode(self._h, buf.ctypes.data if buf.size else None, offs.ctypes.data, len(pieces), out.ctypes.data, out.size)
        if n < 0 or n > out.size:
            raise ValueError("native BPE refused its arguments")
        return out[:n].tolist()

    def encode_text(self, text: str, kind: int) -> list:
        """Pre-tokenizer split (pattern `kind`, see `pretok_kind`) + merges in one native call."""
        raw = text.encode("utf-8")
        if not raw:
            return []
        buf = np.frombuffer(raw, dtype=np.uint8)
        out = np.empty(len(raw), dtype=np.int32)
        n = lib().rx_bpe_encode_text(self._h, kind, buf.ctypes.data, len(raw), out.ctypes.data, out.size)
        if n < 0 or n > out.size:
            raise ValueError("native tokenizer refused its arguments")
        return out[:n].tolist()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._free(h)
