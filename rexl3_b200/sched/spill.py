"""Second tier of the prefix cache: blocks evicted from device memory are written to a directory (an NVMe mount in production) and
read back when a later prompt walks the same chain, instead of being recomputed.  Role of the reference's prefix-snapshot spill
(crates/model/src/families/bailing_moe_v3/spill.rs:1-8) behind this engine's own block-chain index.

One file per block, named by the block's chain hash: `RXSP` magic, payload length, CRC32, payload.  Writes go to a temporary name and
are renamed, so a crash leaves whole files or none.  The store keeps an LRU over what it holds within a byte budget, drops files that
fail their checksum, and can adopt the files already in its directory (a restart keeps its warm prefixes).  A file is found again
only through its chain hash, which starts from the engine's cache namespace; the server derives that namespace from the pack
fingerprint, the KV dtype and the FP8 scale tensor (`server.main.cache_namespace`), so pages written by a different pack, a
re-quantised pack of the same name or a differently calibrated cache are never matched.
"""
from __future__ import annotations

import os
import struct
import zlib
from collections import OrderedDict

MAGIC = b"RXSP"
HEADER = struct.Struct("<4sQI")


class SpillStore:
    def __init__(self, directory: str, max_bytes: int, adopt: bool = True):
        self.dir, self.max_bytes = directory, int(max_bytes)
        os.makedirs(directory, exist_ok=True)
        self.index: "OrderedDict[bytes, int]" = OrderedDict()        # key -> file bytes, least recently used first
        self.bytes = 0
        self.stats = dict(puts=0, hits=0, misses=0, evictions=0, corrupt=0, bytes_written=0, bytes_read=0)
        if adopt:
            for name in sorted(os.listdir(directory)):
                if name.endswith(".blk"):
                    try:
                        key = bytes.fromhex(name[:-4])
                    except ValueError:
                        continue
                    n = os.path.getsize(os.path.join(directory, name))
                    self.index[key] = n
                    self.bytes += n
            self._trim()

    def _path(self, key: bytes) -> str:
        return os.path.join(self.dir, key.hex() + ".blk")

    def __contains__(self, key: bytes) -> bool:
        return key in self.index

    def __len__(self) -> int:
        return len(self.index)

    def put(self, key: bytes, payload: bytes) -> bool:
        """Store a block (a no-op for one already held).  False when the block alone exceeds the budget."""
        if key in self.index:
            self.index.move_to_end(key)
            return True
        n = HEADER.size + len(payload)
        if n > self.max_bytes:
            return False
        tmp = self._path(key) + ".tmp"
        with open(tmp, "wb") as f:
            f.write(HEADER.pack(MAGIC, len(payload), zlib.crc32(payload) & 0xFFFFFFFF))
            f.write(payload)
        os.replace(tmp, self._path(key))
        self.index[key] = n
        self.bytes += n
        self.stats["puts"] += 1
        self.stats["bytes_written"] += n
        self._trim(protect=key)
        return True

    def get(self, key: bytes):
        """The block's payload, or None (never stored, evicted, or failing its checksum: such a file is removed)."""
        if key not in self.index:
            self.stats["misses"] += 1
            return None
        try:
            with open(self._path(key), "rb") as f:
                head = f.read(HEADER.size)
                magic, n, crc = HEADER.unpack(head) if len(head) == HEADER.size else (b"", 0, 0)
                payload = f.read(n + 1) if magic == MAGIC else b""
        except OSError:
            magic, n, crc, payload = b"", 0, 0, b""
        if magic != MAGIC or len(payload) != n or (zlib.crc32(payload) & 0xFFFFFFFF) != crc:
            self.stats["corrupt"] += 1
            self.discard(key)
            return None
        self.index.move_to_end(key)
        self.stats["hits"] += 1
        self.stats["bytes_read"] += HEADER.size + n
        return payload

    def discard(self, key: bytes) -> None:
        n = self.index.pop(key, None)
        if n is not None:
            self.bytes -= n
            try:
                os.remove(self._path(key))
            except OSError:
                pass

    def _trim(self, protect: bytes | None = None) -> None:
        while self.bytes > self.max_bytes and self.index:
            key = next(iter(self.index))
            if key == protect:
                if len(self.index) == 1:
                    break
                self.index.move_to_end(key)
                continue
            self.discard(key)
            self.stats["evictions"] += 1
