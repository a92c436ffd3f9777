"""Pack identity and integrity: a fingerprint of what a pack IS (tensor inventory + quantization record, no payload bytes), per-tensor
CRC32 records (`crc32.txt`) and a per-file lock (`model.lock.json`, schema `rexl3.model-lock.v1`: sha256 and size of every file).

Roles: the reference's pack fingerprint (SHA-256 of a canonical description, crates/model/src/fingerprint.rs:1-15), optional CRC
verification (crates/model/src/verify.rs:1-21) and the recipe's `model.lock.json`.  The fingerprint is cheap (headers only) and is what
ranks of a tensor-parallel group compare at boot; the CRC and lock checks read every byte and are run on request.

    python -m rexl3_b200.format.verify PACK --write-crc --write-lock     # after quantizing
    python -m rexl3_b200.format.verify PACK --check                      # before serving; exit status 1 on any mismatch
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
import zlib

from . import safetensors_io

LOCK_SCHEMA = "rexl3.model-lock.v1"
_CHUNK = 8 << 20


def _tensor_files(folder: str) -> list:
    return sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))


def describe(folder: str) -> dict:
    """Canonical description: every tensor's name, dtype and shape (per file, in name order) and the config's model / quantization record."""
    tensors = {}
    for fname in _tensor_files(folder):
        scan = safetensors_io.read_header(os.path.join(folder, fname))
        if scan.issues:
            raise ValueError(f"{fname}: {scan.issues[0]}")
        for name, e in scan.entries.items():
            tensors[name] = [e.dtype, list(e.shape)]
    conf = {}
    cp = os.path.join(folder, "config.json")
    if os.path.exists(cp):
        c = json.load(open(cp))
        for k in ("architectures", "model_type", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                  "intermediate_size", "vocab_size", "quantization_config"):
            if k in c:
                conf[k] = c[k]
    return {"tensors": dict(sorted(tensors.items())), "config": conf}


def fingerprint(folder: str) -> str:
    blob = json.dumps(describe(folder), sort_keys=True, separators=(",", ":")).encode()
    return hashlib.sha256(blob).hexdigest()


# ---------------------------------------------------------------------------------------------------- per-tensor CRC32
def _crc_of_range(f, offset: int, nbytes: int) -> int:
    f.seek(offset)
    crc, left = 0, nbytes
    while left > 0:
        chunk = f.read(min(_CHUNK, left))
        if not chunk:
            raise IOError("short read")
        crc = zlib.crc32(chunk, crc)
        left -= len(chunk)
    return crc & 0xFFFFFFFF


def tensor_crcs(folder: str) -> dict:
    out = {}
    for fname in _tensor_files(folder):
        scan = safetensors_io.read_header(os.path.join(folder, fname))
        with open(os.path.join(folder, fname), "rb") as f:
            for name in sorted(scan.entries):
                e = scan.entries[name]
                out[name] = (_crc_of_range(f, e.file_offset, e.nbytes), e.nbytes)
    return out


def write_crc(folder: str) -> int:
    crcs = tensor_crcs(folder)
    with open(os.path.join(folder, "crc32.txt"), "w") as f:
        for name, (crc, n) in crcs.items():
            f.write(f"{crc:08x} {n} {name}\n")
    return len(crcs)


def verify_crc(folder: str) -> list:
    """Issues (empty = every recorded tensor matches and none is unrecorded)."""
    path = os.path.join(folder, "crc32.txt")
    if not os.path.exists(path):
        return ["crc32.txt is missing"]
    want = {}
    for ln in open(path):
        parts = ln.rstrip("\n").split(" ", 2)
        if len(parts) == 3:
            want[parts[2]] = (int(parts[0], 16), int(parts[1]))
    have = tensor_crcs(folder)
    issues = []
    for name, (crc, n) in have.items():
        w = want.get(name)
        if w is None:
            issues.append(f"{name}: not in crc32.txt")
        elif w != (crc, n):
            issues.append(f"{name}: crc {crc:08x} / {n} bytes, recorded {w[0]:08x} / {w[1]} bytes")
    issues += [f"{name}: recorded but not in the pack" for name in want if name not in have]
    return issues


# ---------------------------------------------------------------------------------------------------- per-file lock
def _sha256_file(path: str) -> tuple:
    h, n = hashlib.sha256(), 0
    with open(path, "rb") as f:
        while True:
            chunk = f.read(_CHUNK)
            if not chunk:
                break
            h.update(chunk)
            n += len(chunk)
    return h.hexdigest(), n


LOCKED_SUFFIXES = (".safetensors", ".json", ".txt", ".jinja", ".model")


def make_lock(folder: str) -> dict:
    files = {}
    for name in sorted(os.listdir(folder)):
        p = os.path.join(folder, name)
        if name == "model.lock.json" or not os.path.isfile(p) or not name.endswith(LOCKED_SUFFIXES):
            continue
        sha, n = _sha256_file(p)
        files[name] = {"sha256": sha, "bytes": n}
    return {"schema": LOCK_SCHEMA, "fingerprint": fingerprint(folder), "files": files}


def write_lock(folder: str) -> dict:
    lock = make_lock(folder)
    json.dump(lock, open(os.path.join(folder, "model.lock.json"), "w"), indent=1, sort_keys=True)
    return lock


def verify_lock(folder: str, lock: dict | None = None, sizes_only: bool = False) -> list:
    """Issues against `lock` (default: the pack's own model.lock.json).  `sizes_only` skips the hashes (a boot-time check that reads no payload)."""
    if lock is None:
        p = os.path.join(folder, "model.lock.json")
        if not os.path.exists(p):
            return ["model.lock.json is missing"]
        lock = json.load(open(p))
    if lock.get("schema") != LOCK_SCHEMA:
        return [f"lock schema {lock.get('schema')!r} is not {LOCK_SCHEMA}"]
    issues = []
    for name, want in sorted((lock.get("files") or {}).items()):
        p = os.path.join(folder, name)
        if not os.path.isfile(p):
            issues.append(f"{name}: missing")
            continue
        if sizes_only:
            n = os.path.getsize(p)
            if n != want.get("bytes"):
                issues.append(f"{name}: {n} bytes, locked {want.get('bytes')}")
            continue
        sha, n = _sha256_file(p)
        if n != want.get("bytes") or sha != want.get("sha256"):
            issues.append(f"{name}: sha256 {sha[:16]}... / {n} bytes does not match the lock")
    try:
        fp = fingerprint(folder)
        if lock.get("fingerprint") and fp != lock["fingerprint"]:
            issues.append(f"fingerprint {fp[:16]}... is not the locked {lock['fingerprint'][:16]}...")
    except (ValueError, OSError) as e:
        issues.append(f"fingerprint: {e}")
    return issues


def main(argv=None) -> int:
    import argparse
    p = argparse.ArgumentParser(prog="rexl3-verify", allow_abbrev=False)
    p.add_argument("pack")
    p.add_argument("--write-crc", action="store_true")
    p.add_argument("--write-lock", action="store_true")
    p.add_argument("--check", action="store_true", help="verify crc32.txt and model.lock.json (whichever exist)")
    a = p.parse_args(argv)
    print(f"fingerprint {fingerprint(a.pack)}")
    if a.write_crc:
        print(f"crc32.txt: {write_crc(a.pack)} tensors")
    if a.write_lock:
        print(f"model.lock.json: {len(write_lock(a.pack)['files'])} files")
    bad = []
    if a.check:
        if os.path.exists(os.path.join(a.pack, "crc32.txt")):
            bad += verify_crc(a.pack)
        if os.path.exists(os.path.join(a.pack, "model.lock.json")):
            bad += verify_lock(a.pack)
        for b in bad:
            print("MISMATCH", b)
        print("ok" if not bad else f"{len(bad)} mismatches")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
