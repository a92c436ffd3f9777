"""Scan an EXL3 pack folder: headers only, tensors sorted into EXL3 groups, plain tensors and refused groups.

A group ``<prefix>`` is the set ``<prefix>.{trellis,suh|su,svh|sv,mcg|mul1,bias}``; it is refused for the
same reasons the reference refuses it (crates/exl3/src/checkpoint.rs:194-271): trellis not int16 rank 3,
unsupported width, both markers, half width without mul1, missing / doubled / mis-shaped scales, bad bias,
K or N not a multiple of 128.  ``model.safetensors.index.json`` is authoritative for tensor placement when
present (checkpoint.rs:403-414).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import numpy as np

from . import exl3
from .safetensors_io import Entry, read_header, read_tensor

PARTS = ("trellis", "suh", "su", "svh", "sv", "mcg", "mul1", "bias")


@dataclass
class Group:
    prefix: str
    bits: exl3.Bits
    codebook: str
    k: int
    n: int
    in_scales: str
    out_scales: str
    bias: bool
    files: list
    bytes: int
    parts: dict = field(default_factory=dict, repr=False)


@dataclass
class Checkpoint:
    folder: str
    groups: dict = field(default_factory=dict)   # prefix -> Group
    plain: dict = field(default_factory=dict)    # name -> Entry
    bad: dict = field(default_factory=dict)      # prefix -> reason
    issues: list = field(default_factory=list)

    def total_bytes(self) -> int:
        return sum(g.bytes for g in self.groups.values()) + sum(e.nbytes for e in self.plain.values())


SIDECAR_FILES = ("vision.safetensors",)

def parse_group(prefix: str, parts: dict) -> Group:
    """Raises ValueError(reason) for a group that must not load."""
    tr = parts.get("trellis")
    if tr is None:
        raise ValueError("no .trellis")
    if tr.dtype != "I16" or len(tr.shape) != 3:
        raise ValueError(f"trellis must be int16 [K/16, N/16, 16 * bits], got {tr.dtype} {list(tr.shape)}")
    if 0 in tr.shape:
        raise ValueError(f"trellis {list(tr.shape)} has an empty dimension")
    try:
        bits = exl3.Bits.from_trellis_last(tr.shape[2])
    except ValueError:
        raise ValueError(f"unsupported trellis width {tr.shape[2]}")
    has = [m for m in ("mcg", "mul1") if m in parts]
    if len(has) > 1:
        raise ValueError("both mcg and mul1 markers")
    for m in has:
        e = parts[m]
        if e.dtype != "I32" or e.nbytes != 4:
            raise ValueError(f".{m} marker must be one int32, got {e.dtype} {list(e.shape)}")
    cb = has[0] if has else "3inst"
    if not bits.is_integer and cb != "mul1":
        raise ValueError(f"{bits.value}-bit tiles need the mul1 codebook, found {cb}")
    k, n = 16 * tr.shape[0], 16 * tr.shape[1]
    if "suh" in parts and "su" in parts:
        raise ValueError("both .suh and .su input scales")
    if "svh" in parts and "sv" in parts:
        raise ValueError("both .svh and .sv output scales")
    if "suh" in parts:
        ins, want = "suh", ("F16", (k,))
    elif "su" in parts:
        ins, want = "su", ("I16", (k // 16,))
    else:
        raise ValueError("no input scales (.suh or .su)")
    e = parts[ins]
    if (e.dtype, tuple(e.shape)) != want:
        raise ValueError(f".{ins} must be {want[0]} {list(want[1])}, got {e.dtype} {list(e.shape)}")
    if "svh" in parts:
        outs, want = "svh", ("F16", (n,))
    elif "sv" in parts:
        outs, want = "sv", ("I16", (n // 16,))
    else:
        raise ValueError("no output scales (.svh or .sv)")
    e = parts[outs]
    if (e.dtype, tuple(e.shape)) != want:
        raise ValueError(f".{outs} must be {want[0]} {list(want[1])}, got {e.dtype} {list(e.shape)}")
    if "bias" in parts:
        b = parts["bias"]
        if b.dtype not in ("F16", "BF16", "F32") or tuple(b.shape) != (n,):
            raise ValueError(f".bias must be a float vector of {n}, got {b.dtype} {list(b.shape)}")
    if k % exl3.HAD or n % exl3.HAD:
        raise ValueError(f"K={k} and N={n} must be multiples of {exl3.HAD} (the Hadamard blocks)")
    return Group(prefix, bits, cb, k, n, ins, outs, "bias" in parts,
                 sorted({p.file for p in parts.values()}), sum(p.nbytes for p in parts.values()), dict(parts))


def scan(folder: str, verify_markers: bool = False) -> Checkpoint:
    """Header-only scan.  `verify_markers` also reads the 4 bytes of every codebook marker tensor: a marker that does not hold its
    codebook's multiplier refuses the group (reference crates/exl3/src/checkpoint.rs:203-220; its scan has the same switch)."""
    ck = Checkpoint(folder)
    # sidecar files hold tensors of another network (the vision tower): they are not shards of the language model's index
    files = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors") and f not in SIDECAR_FILES)
    placement = None
    idx = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(idx):
        try:
            wm = json.load(open(idx)).get("weight_map")
            if isinstance(wm, dict):
                placement = {str(k): str(v) for k, v in wm.items()}
            else:
                ck.issues.append("model.safetensors.index.json: no weight_map object")
        except (json.JSONDecodeError, OSError) as e:
            ck.issues.append(f"model.safetensors.index.json: {e}")
    entries: dict = {}
    for fn in files:
        hs = read_header(os.path.join(folder, fn))
        ck.issues.extend(hs.issues)
        for name, e in hs.entries.items():
            if placement is not None:
                want = placement.get(name)
                if want is None:
                    ck.issues.append(f"{fn}: {name}: not in the index")
                    continue
                if want != fn:
                    continue  # the index says another file owns this name
            if name in entries:
                ck.issues.append(f"{fn}: {name}: duplicate of the tensor in {entries[name].file}")
                continue
            entries[name] = e
    if placement is not None:
        for name, fn in placement.items():
            if name not in entries:
                ck.issues.append(f"index names {name} in {fn}, which does not hold it")
    by_prefix: dict = {}
    for name, e in entries.items():
        pre, _, part = name.rpartition(".")
        if part in PARTS and pre:
            by_prefix.setdefault(pre, {})[part] = e
    trellis_prefixes = {p for p, parts in by_prefix.items() if "trellis" in parts}
    for name, e in entries.items():
        pre, _, part = name.rpartition(".")
        if part in PARTS and pre in trellis_prefixes:
            continue
        ck.plain[name] = e
    for pre in sorted(trellis_prefixes):
        try:
            g = parse_group(pre, by_prefix[pre])
            if verify_markers:
                for part, want in (("mcg", exl3.MARKER_MCG), ("mul1", exl3.MARKER_MUL1)):
                    e = by_prefix[pre].get(part)
                    if e is not None:
                        got = int(np.frombuffer(read_tensor(folder, e).tobytes()[:4], dtype="<u4")[0])
                        if got != want:
                            raise ValueError(f".{part} marker holds 0x{got:08X}, not 0x{want:08X}")
            ck.groups[pre] = g
        except ValueError as err:
            ck.bad[pre] = str(err)
    return ck


@dataclass
class LoadedGroup:
    group: Group
    trellis: np.ndarray      # int16 [K/16, N/16, 16*bits]
    suh: np.ndarray          # float16 [K]
    svh: np.ndarray          # float16 [N]
    bias: np.ndarray | None  # float32 [N]


def _bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def load_group(folder: str, g: Group) -> LoadedGroup:
    p = g.parts
    trellis = read_tensor(folder, p["trellis"])
    if g.in_scales == "suh":
        suh = read_tensor(folder, p["suh"]).astype(np.float16)
    else:
        suh = exl3.unpack_signs(read_tensor(folder, p["su"])).astype(np.float16)
    if g.out_scales == "svh":
        svh = read_tensor(folder, p["svh"]).astype(np.float16)
    else:
        svh = exl3.unpack_signs(read_tensor(folder, p["sv"])).astype(np.float16)
    bias = None
    if g.bias:
        b = read_tensor(folder, p["bias"])
        bias = _bf16_to_f32(b) if p["bias"].dtype == "BF16" else b.astype(np.float32)
    return LoadedGroup(g, np.array(trellis), np.array(suh), np.array(svh), bias)


def load_plain(folder: str, e: Entry) -> np.ndarray:
    a = read_tensor(folder, e)
    if e.dtype == "BF16":
        return _bf16_to_f32(a)
    return np.array(a)
