"""Affinity keys: a 64-bit hash of the part of a request that shares a prefix cache on a backend - the system prompt(s) plus the
first user message of a chat completion, the prompt of a text completion - unless the client names a key itself.  FNV-1a 64
finished with a splitmix64 mix, so routers restarted or running side by side agree (not a security boundary).
Behaviour parity: reference crates/router/src/keying.rs:1-45.
"""
from __future__ import annotations

import json

MASK = (1 << 64) - 1
FNV_OFFSET, FNV_PRIME = 0xCBF29CE484222325, 0x100000001B3


def mix64(z: int) -> int:
    z &= MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def fnv64(data: bytes) -> int:
    h = FNV_OFFSET
    for b in data:
        h = ((h ^ b) * FNV_PRIME) & MASK
    return mix64(h)


def rendezvous(key: int, backend_hash: int) -> int:
    rot = ((backend_hash << 17) | (backend_hash >> 47)) & MASK
    return mix64(key ^ rot)


def _text(content) -> str:
    if isinstance(content, str):
        return content
    if isinstance(content, list):          # content parts: only the text takes part (no image bytes are hashed)
        return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") == "text")
    return ""


def affinity_key(headers, body: bytes, cap: int = 65536):
    """-> (key or None, source) with source in {"header", "prompt", "none"}."""
    h = headers.get("x-affinity-key")
    if h:
        return fnv64(h.encode()), "header"
    try:
        doc = json.loads(body)
    except (ValueError, UnicodeDecodeError):
        return None, "none"
    if not isinstance(doc, dict):
        return None, "none"
    if isinstance(doc.get("messages"), list):
        parts = []
        for m in doc["messages"]:
            if not isinstance(m, dict):
                continue
            role = m.get("role")
            if role in ("system", "developer"):
                parts.append("s:" + _text(m.get("content")))
            elif role == "user":
                parts.append("u:" + _text(m.get("content")))
                break
        if parts:
            return fnv64("\x1f".join(parts).encode()[:cap]), "prompt"
    p = doc.get("prompt")
    if isinstance(p, str) and p:
        return fnv64(p.encode()[:cap]), "prompt"
    if isinstance(p, list) and p and all(isinstance(t, int) for t in p):
        return fnv64(b"".join(int(t).to_bytes(4, "little", signed=False) for t in p[:cap // 4])), "prompt"
    return None, "none"
