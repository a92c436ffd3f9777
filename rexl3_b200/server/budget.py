"""Request budgets: admission before a request is retained or expanded (reference crates/server/src/budget.rs:1-30).  Limits are active by
default and derive from the context window: a body cap, a JSON node and depth cap checked while the body is walked (before any template
sees it), a cap on the rendered prompt (16 bytes per token of the window, at least 1 MiB), a bounded number of requests in preparation
(parse + render + tokenize) with a bounded queue behind them, and a tokenizer gate that prices a prompt by its size (tokenizing costs far
more memory than the text) so that the number of prompts tokenized at once follows their size, not a worker count.

Everything here is host-side and synchronous-safe: the HTTP layer calls `check_json`, `check_rendered` and takes a `TokenizerGate.charge`
around the tokenizer call; each refusal carries the HTTP status the reference answers with (413 too large, 429 busy).
"""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass

TOKENIZER_BYTES_PER_RENDERED_BYTE = 448      # priced memory of the tokenizer stage per byte of rendered text
RENDERED_BYTES_PER_WINDOW_TOKEN = 16
RENDERED_FLOOR_BYTES = 1 << 20
DEFAULT_WINDOW_TOKENS = 262_144
DEFAULT_PROCESSING_RESERVE_BYTES = 2 << 30
DEFAULT_TOKENIZER_WAIT_S = 60.0
TOKENIZER_SLACK_BYTES = 64


class BudgetRefused(Exception):
    def __init__(self, status: int, message: str, code: str, retry_after: "int | None" = None):
        super().__init__(message)
        self.status, self.code, self.retry_after = status, code, retry_after


def default_rendered_bytes(window_tokens: int) -> int:
    return max(window_tokens * RENDERED_BYTES_PER_WINDOW_TOKEN, RENDERED_FLOOR_BYTES)


@dataclass
class Limits:
    body_bytes: int = 64 << 20
    total_bytes: int = 128 << 20
    json_nodes: int = 300_000
    json_depth: int = 128
    rendered_bytes: int = default_rendered_bytes(DEFAULT_WINDOW_TOKENS)
    preparation_concurrency: int = 2
    preparation_queue: int = 64
    processing_reserve_bytes: int = DEFAULT_PROCESSING_RESERVE_BYTES
    tokenizer_wait_s: float = DEFAULT_TOKENIZER_WAIT_S

    @staticmethod
    def for_window(window_tokens: int) -> "Limits":
        """The defaults for a context window: the rendered cap follows the window, and the reserve is the default unless one prompt at
        that cap is priced higher."""
        lim = Limits(rendered_bytes=default_rendered_bytes(window_tokens))
        lim.processing_reserve_bytes = lim.derived_reserve()
        return lim

    def tokenizer_price(self) -> int:
        return (self.rendered_bytes + TOKENIZER_SLACK_BYTES) * TOKENIZER_BYTES_PER_RENDERED_BYTE

    def derived_reserve(self) -> int:
        return max(self.tokenizer_price(), DEFAULT_PROCESSING_RESERVE_BYTES)

    def validate(self) -> None:
        """Raises ValueError when the limits contradict each other (the reserve must hold the parse stage at full concurrency and the
        largest single prompt of the tokenizer stage)."""
        if 0 in (self.body_bytes, self.total_bytes, self.json_nodes, self.json_depth, self.rendered_bytes, self.preparation_concurrency):
            raise ValueError("request limits must be positive")
        if self.json_depth > 128:
            raise ValueError("max-json-depth must not exceed 128")
        raw = min(self.body_bytes, self.total_bytes) * 16
        nodes = self.json_nodes * 128
        required = max(max(raw, nodes) * self.preparation_concurrency, self.tokenizer_price())
        if self.processing_reserve_bytes < required:
            raise ValueError(f"processing reserve must be at least {required} bytes for these body/node/render/concurrency limits (the largest "
                             f"rendered prompt is priced at {self.tokenizer_price()} bytes: {TOKENIZER_BYTES_PER_RENDERED_BYTE} per rendered byte)")


def check_json(value, limits: Limits) -> int:
    """Walk a decoded JSON body; refuse (413) past the node or depth cap.  Returns the node count.  Iterative: a hostile depth cannot
    exhaust the interpreter's stack."""
    nodes, stack = 0, [(value, 1)]
    while stack:
        v, depth = stack.pop()
        nodes += 1
        if nodes > limits.json_nodes:
            raise BudgetRefused(413, f"the request body has more than {limits.json_nodes} JSON values (--max-json-nodes)", "json_too_large")
        if depth > limits.json_depth:
            raise BudgetRefused(413, f"the request body nests deeper than {limits.json_depth} levels (--max-json-depth)", "json_too_deep")
        if isinstance(v, dict):
            for k, x in v.items():
                nodes += 1            # the key is a value of its own in the count
                stack.append((x, depth + 1))
        elif isinstance(v, list):
            for x in v:
                stack.append((x, depth + 1))
    return nodes


def check_rendered(text: str, limits: Limits) -> int:
    n = len(text.encode("utf-8"))
    if n > limits.rendered_bytes:
        raise BudgetRefused(413, f"the rendered prompt has {n} bytes, the server admits {limits.rendered_bytes} (--max-rendered-prompt-mib)",
                            "prompt_too_large")
    return n


class PreparationGate:
    """At most `concurrency` requests in preparation, at most `queue` waiting behind them; a request beyond that is refused 429 at once
    (fail fast keeps the queue's memory bounded)."""

    def __init__(self, concurrency: int, queue: int):
        self.sem = threading.BoundedSemaphore(concurrency)
        self.lock = threading.Lock()
        self.waiting, self.queue = 0, queue
        self.refused = 0

    def __enter__(self):
        if self.sem.acquire(blocking=False):
            return self
        with self.lock:
            if self.waiting >= self.queue:
                self.refused += 1
                raise BudgetRefused(429, "too many requests are being prepared; retry shortly", "preparation_busy", retry_after=1)
            self.waiting += 1
        try:
            self.sem.acquire()
        finally:
            with self.lock:
                self.waiting -= 1
        return self

    def __exit__(self, *exc):
        self.sem.release()
        return False


class TokenizerGate:
    """The tokenizer stage's share of the processing reserve: a call takes its priced bytes before it allocates and gives them back when the
    encoding has been copied out.  A prompt that does not fit waits, first come first served (a large one is not starved by small ones);
    one that could never fit is refused 413; one that waited past `wait_s` is refused 429.  Reference crates/server/src/budget.rs:124-200."""

    def __init__(self, capacity: int, wait_s: float = DEFAULT_TOKENIZER_WAIT_S):
        self.capacity, self.wait_s = capacity, wait_s
        self.free = capacity
        self.queue: deque = deque()
        self.next = 0
        self.cv = threading.Condition()
        self.waited = self.refused = 0

    @staticmethod
    def price(text_bytes: int) -> int:
        return text_bytes * TOKENIZER_BYTES_PER_RENDERED_BYTE

    def in_use(self) -> int:
        with self.cv:
            return self.capacity - self.free

    def charge(self, text_bytes: int) -> "TokenizerCharge":
        price = self.price(text_bytes)
        if price > self.capacity:
            self.refused += 1
            raise BudgetRefused(413, f"the rendered prompt of {text_bytes} bytes is priced at {price} bytes of tokenizer memory "
                                     f"({TOKENIZER_BYTES_PER_RENDERED_BYTE} per byte), more than the processing reserve of {self.capacity} bytes "
                                     f"(--processing-reserve-mib)", "prompt_too_large")
        give_up = time.monotonic() + self.wait_s
        with self.cv:
            if not self.queue and self.free >= price:
                self.free -= price
                return TokenizerCharge(self, price)
            self.waited += 1
            ticket = self.next
            self.next += 1
            self.queue.append(ticket)
            while True:
                if self.queue[0] == ticket and self.free >= price:
                    self.queue.popleft()
                    self.free -= price
                    self.cv.notify_all()
                    return TokenizerCharge(self, price)
                left = give_up - time.monotonic()
                if left <= 0:
                    self.queue.remove(ticket)
                    self.refused += 1
                    self.cv.notify_all()
                    raise BudgetRefused(429, "the tokenizer stage is busy with other prompts; retry shortly", "tokenizer_busy",
                                        retry_after=max(1, int(self.wait_s // 4)))
                self.cv.wait(timeout=left)

    def _release(self, n: int) -> None:
        with self.cv:
            self.free += n
            self.cv.notify_all()


class TokenizerCharge:
    def __init__(self, gate: TokenizerGate, n: int):
        self.gate, self.n = gate, n

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()
        return False

    def release(self) -> None:
        if self.n:
            self.gate._release(self.n)
            self.n = 0
