"""Memory admission (fail closed), refcounted paged block pool, validated KV memory model.

Behaviour parity: reference crates/sched/src/lib.rs:79-236 (Admission), :244-297 (BlockPool),
crates/sched/src/memory.rs:36-130 (KvPlane / KvLayout::bytes_per_page).  A request is admitted only if its
whole reservation (prompt + max new tokens) fits; a config that can never fit is refused at boot, by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field


class AdmitError(Exception):
    def __init__(self, kind: str, **kw):
        self.kind, self.info = kind, kw
        super().__init__(f"{kind}: " + ", ".join(f"{k}={v}" for k, v in kw.items()))


class MemoryError_(ValueError):
    """A memory model that does not validate (zero-byte KV, negative sizes)."""


@dataclass
class ModelMemory:
    weights_bytes: int
    kv_bytes_per_token: int
    state_bytes_per_slot: int = 0
    activation_reserve: int = 0

    def validate(self) -> None:
        if self.kv_bytes_per_token <= 0:
            raise MemoryError_("kv_bytes_per_token must be positive (a zero-byte KV plan is refused)")
        if min(self.weights_bytes, self.state_bytes_per_slot, self.activation_reserve) < 0:
            raise MemoryError_("negative size in the memory model")


@dataclass
class KvPlane:
    """One cached plane of a layer class: elements per token and bytes per element (+ per-token scale bytes)."""
    name: str
    elems_per_token: int
    elem_bytes: float
    scale_bytes_per_token: int = 0

    def bytes_per_token(self) -> int:
        return int(self.elems_per_token * self.elem_bytes) + self.scale_bytes_per_token


@dataclass
class KvLayout:
    page_tokens: int
    planes: list = field(default_factory=list)   # list[(KvPlane, n_layers)]

    def bytes_per_token(self) -> int:
        return sum(p.bytes_per_token() * n for p, n in self.planes)

    def bytes_per_page(self) -> int:
        return self.bytes_per_token() * self.page_tokens

    @staticmethod
    def gqa(n_layers: int, n_kv: int, head_dim: int, dtype: str = "bf16", page_tokens: int = 64) -> "KvLayout":
        eb = {"bf16": 2, "fp16": 2, "fp8": 1, "int8": 1}[dtype]
        sc = 0 if eb == 2 else 4 * n_kv  # per-(token, head) fp32 scale for 8-bit KV
        return KvLayout(page_tokens, [(KvPlane("k", n_kv * head_dim, eb, sc), n_layers), (KvPlane("v", n_kv * head_dim, eb, sc), n_layers)])

    @staticmethod
    def mla(n_layers: int, kv_lora: int, rope_dim: int, dtype: str = "bf16", page_tokens: int = 64) -> "KvLayout":
        eb = {"bf16": 2, "fp16": 2, "fp8": 1}[dtype]
        return KvLayout(page_tokens, [(KvPlane("latent", kv_lora + rope_dim, eb), n_layers)])


class Admission:
    def __init__(self, allocatable_bytes: int, floor_bytes: int, model: ModelMemory, max_slots: int):
        model.validate()
        fixed = floor_bytes + model.weights_bytes + model.activation_reserve
        self.capacity = max(0, allocatable_bytes - fixed)
        self.used = 0
        self.pinned = 0
        self.max_context = None
        self.kv_tokens = None
        self.kv_in_use = 0
        self.model = model
        self.slots = [None] * max_slots

    def with_max_context(self, tokens: int) -> "Admission":
        self.max_context = tokens
        return self

    def with_kv_tokens(self, tokens: int) -> "Admission":
        self.kv_tokens = tokens
        return self

    def request_limit(self):
        lims = [x for x in (self.max_context, self.kv_tokens) if x is not None]
        return min(lims) if lims else None

    def available(self) -> int:
        return max(0, self.capacity - self.used - self.pinned)

    def cost(self, tokens: int) -> int:
        return tokens * self.model.kv_bytes_per_token + self.model.state_bytes_per_slot

    def check(self, tokens: int) -> None:
        """Could this request EVER run here?  Raises ContextTooLong / NeverFits."""
        lim = self.request_limit()
        if lim is not None and tokens > lim:
            raise AdmitError("ContextTooLong", tokens=tokens, max=lim)
        need = self.cost(tokens)
        if need > self.capacity:
            raise AdmitError("NeverFits", needed=need, capacity=self.capacity)

    def can_admit(self, tokens: int) -> int:
        lim = self.request_limit()
        if lim is not None and tokens > lim:
            raise AdmitError("ContextTooLong", tokens=tokens, max=lim)
        need = self.cost(tokens)
        if need > self.available():
            raise AdmitError("NoMemory", needed=need, available=self.available())
        if self.kv_tokens is not None:
            left = max(0, self.kv_tokens - self.kv_in_use)
            if tokens > left:
                per = self.model.kv_bytes_per_token
                raise AdmitError("NoMemory", needed=tokens * per, available=left * per)
        if None not in self.slots:
            raise AdmitError("NoSlot")
        return need

    def admit(self, tokens: int) -> int:
        need = self.can_admit(tokens)
        slot = self.slots.index(None)
        self.slots[slot] = (need, tokens)
        self.used += need
        self.kv_in_use += tokens
        return slot

    def release(self, slot: int) -> None:
        if 0 <= slot < len(self.slots) and self.slots[slot] is not None:
            b, t = self.slots[slot]
            self.slots[slot] = None
            self.used = max(0, self.used - b)
            self.kv_in_use = max(0, self.kv_in_use - t)

    def reserved(self):
        return [(i, s[1]) for i, s in enumerate(self.slots) if s is not None]

    def pin(self, nbytes: int) -> None:
        if nbytes > self.available():
            raise AdmitError("NoMemory", needed=nbytes, available=self.available())
        self.pinned += nbytes

    def unpin(self, nbytes: int) -> None:
        self.pinned = max(0, self.pinned - nbytes)

    def fits(self, tokens: int) -> int:
        return self.available() // max(1, self.cost(tokens))


class BlockPool:
    """Refcounted pool of fixed-size KV pages; a page returns to the free list when its last holder lets go."""

    def __init__(self, blocks: int, block_tokens: int = 64):
        self.free = list(range(blocks - 1, -1, -1))
        self.refs = [0] * blocks
        self.block_tokens = block_tokens

    def free_blocks(self) -> int:
        return len(self.free)

    def total_blocks(self) -> int:
        return len(self.refs)

    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.block_tokens)

    def alloc(self, n: int):
        if n > len(self.free):
            return None
        out = [self.free.pop() for _ in range(n)]
        for b in out:
            self.refs[b] = 1
        return out

    def retain(self, blocks) -> None:
        for b in blocks:
            if self.refs[b] <= 0:
                raise AssertionError(f"retain of a free block {b}")
            self.refs[b] += 1

    def release(self, blocks) -> None:
        for b in blocks:
            if self.refs[b] <= 0:
                raise AssertionError(f"double free of block {b}")
            self.refs[b] -= 1
            if self.refs[b] == 0:
                self.free.append(b)

    def refcount(self, b: int) -> int:
        return self.refs[b]
