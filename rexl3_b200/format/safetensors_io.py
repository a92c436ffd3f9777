"""Minimal safetensors reader/writer with hostile-header checks.

The header of a ``*.safetensors`` file is untrusted input: every length, offset and
size is checked against the real file size and malformed entries are reported, never
silently dropped (behaviour parity: reference crates/exl3/src/checkpoint.rs:1-8,
:60-190, hardening tests crates/exl3/tests/hardening.rs).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field

import numpy as np

MAX_HEADER_BYTES = 100_000_000

_DTYPE_SIZE = {
    "BOOL": 1, "U8": 1, "I8": 1, "F8_E4M3": 1, "F8_E5M2": 1, "F8_E8M0": 1,
    "F16": 2, "BF16": 2, "I16": 2, "U16": 2,
    "F32": 4, "I32": 4, "U32": 4,
    "F64": 8, "I64": 8, "U64": 8,
}
_NP = {
    "BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "F8_E4M3": np.uint8, "F8_E5M2": np.uint8, "F8_E8M0": np.uint8,
    "F16": np.float16, "BF16": np.uint16, "I16": np.int16, "U16": np.uint16,
    "F32": np.float32, "I32": np.int32, "U32": np.uint32,
    "F64": np.float64, "I64": np.int64, "U64": np.uint64,
}
_FROM_NP = {np.dtype(np.float16): "F16", np.dtype(np.float32): "F32", np.dtype(np.float64): "F64",
            np.dtype(np.int8): "I8", np.dtype(np.uint8): "U8", np.dtype(np.int16): "I16", np.dtype(np.uint16): "U16",
            np.dtype(np.int32): "I32", np.dtype(np.uint32): "U32", np.dtype(np.int64): "I64", np.dtype(np.uint64): "U64",
            np.dtype(np.bool_): "BOOL"}


def dtype_size(dtype: str):
    return _DTYPE_SIZE.get(dtype)


@dataclass
class Entry:
    file: str
    dtype: str
    shape: tuple
    offsets: tuple  # (begin, end) relative to the data section
    header_size: int = 0

    @property
    def nbytes(self) -> int:
        return max(0, self.offsets[1] - self.offsets[0])

    @property
    def file_offset(self) -> int:
        return 8 + self.header_size + self.offsets[0]


@dataclass
class HeaderScan:
    entries: dict = field(default_factory=dict)
    issues: list = field(default_factory=list)
    metadata: dict = field(default_factory=dict)


def read_header(path: str) -> HeaderScan:
    """Parse one file's header. Never raises on malformed content: problems land in ``issues``."""
    out = HeaderScan()
    name = os.path.basename(path)
    try:
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            raw = f.read(8)
            if len(raw) < 8:
                out.issues.append(f"{name}: shorter than the 8-byte length prefix")
                return out
            (hlen,) = struct.unpack("<Q", raw)
            if hlen > MAX_HEADER_BYTES:
                out.issues.append(f"{name}: header of {hlen} bytes exceeds the {MAX_HEADER_BYTES}-byte cap")
                return out
            if 8 + hlen > size:
                out.issues.append(f"{name}: header of {hlen} bytes runs past the {size}-byte file")
                return out
            blob = f.read(hlen)
    except OSError as e:
        out.issues.append(f"{name}: {e}")
        return out
    try:
        hdr = json.loads(blob.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError, RecursionError) as e:
        out.issues.append(f"{name}: header is not JSON ({e.__class__.__name__})")
        return out
    if not isinstance(hdr, dict):
        out.issues.append(f"{name}: header is not a JSON object")
        return out
    data_len = size - 8 - hlen
    for key, v in hdr.items():
        if key == "__metadata__":
            if isinstance(v, dict):
                out.metadata = v
            continue
        if not isinstance(v, dict):
            out.issues.append(f"{name}: {key}: entry is not an object")
            continue
        dt, shape, offs = v.get("dtype"), v.get("shape"), v.get("data_offsets")
        if not isinstance(dt, str) or dt not in _DTYPE_SIZE:
            out.issues.append(f"{name}: {key}: unknown dtype {dt!r}")
            continue
        if not isinstance(shape, list) or any((not isinstance(d, int)) or isinstance(d, bool) or d < 0 for d in shape):
            out.issues.append(f"{name}: {key}: bad shape {shape!r}")
            continue
        if (not isinstance(offs, list) or len(offs) != 2
                or any((not isinstance(o, int)) or isinstance(o, bool) or o < 0 for o in offs)):
            out.issues.append(f"{name}: {key}: bad data_offsets {offs!r}")
            continue
        b, e = offs
        if e < b:
            out.issues.append(f"{name}: {key}: data ends ({e}) before it starts ({b})")
            continue
        if e > data_len:
            out.issues.append(f"{name}: {key}: data [{b}, {e}) runs past the {data_len}-byte data section")
            continue
        count = 1
        for d in shape:
            count *= d
        if count * _DTYPE_SIZE[dt] != e - b:
            out.issues.append(f"{name}: {key}: shape {shape} x {dt} is {count * _DTYPE_SIZE[dt]} bytes, offsets give {e - b}")
            continue
        out.entries[key] = Entry(name, dt, tuple(shape), (b, e), hlen)
    return out


_PREFETCHED = {}   # (absolute file path, file offset, nbytes) -> uint8 view of a staging buffer filled by `prefetch`


def prefetch(folder: str, entries, threads: int = 8, direct: bool = False, pinned: bool = False) -> int:
    """Read all `entries` (of any number of files) with the native parallel range reader into one staging buffer per file; later
    `read_tensor` calls for them are served from it (each once).  `pinned`: page-locked staging (host->device copies from the returned
    arrays can then be asynchronous).  Returns the bytes read."""
    from ..native import host
    by_file = {}
    for e in entries:
        by_file.setdefault(e.file, []).append(e)
    total = 0
    for fname, es in by_file.items():
        path = os.path.abspath(os.path.join(folder, fname))
        sizes = [e.nbytes for e in es]
        offs = [e.file_offset for e in es]
        starts, pos = [], 0
        for n in sizes:
            starts.append(pos)
            pos += (n + 63) // 64 * 64          # every tensor starts 64-byte aligned in the staging buffer
        if pinned:
            import torch
            stage = torch.empty(max(pos, 1), dtype=torch.uint8).pin_memory().numpy()
        else:
            stage = np.empty(max(pos, 1), dtype=np.uint8)
        from ..utils import loadstats
        with loadstats.stage("pack", "read", sum(sizes)):
            host.read_ranges(path, offs, sizes, stage, starts, threads=threads, direct=direct)
        for e, st, n in zip(es, starts, sizes):
            _PREFETCHED[(path, e.file_offset, n)] = stage[st:st + n]
        total += sum(sizes)
    return total


def drop_prefetched() -> None:
    _PREFETCHED.clear()


def read_tensor(folder: str, e: Entry) -> np.ndarray:
    """Read one tensor's bytes as numpy (BF16 / F8 come back as raw uint16 / uint8)."""
    hit = _PREFETCHED.pop((os.path.abspath(os.path.join(folder, e.file)), e.file_offset, e.nbytes), None)
    if hit is not None:
        return hit.view(_NP[e.dtype]).reshape(e.shape)
    with open(os.path.join(folder, e.file), "rb") as f:
        f.seek(e.file_offset)
        raw = f.read(e.nbytes)
    if len(raw) != e.nbytes:
        raise IOError(f"{e.file}: short read of {len(raw)} / {e.nbytes} bytes")
    return np.frombuffer(raw, dtype=_NP[e.dtype]).reshape(e.shape)


def write_file(path: str, tensors: dict, metadata: dict | None = None, dtypes: dict | None = None) -> None:
    """Write numpy tensors. ``dtypes`` overrides the safetensors dtype string (e.g. {'w': 'BF16'} for uint16 bits)."""
    hdr = {}
    if metadata:
        hdr["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        dt = (dtypes or {}).get(name) or _FROM_NP[a.dtype]
        if _DTYPE_SIZE[dt] != a.dtype.itemsize:
            raise ValueError(f"{name}: dtype {dt} does not match itemsize {a.dtype.itemsize}")
        b = a.tobytes()
        hdr[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    h = json.dumps(hdr, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)
