"""Tokenizers: a byte-level BPE reader of HF ``tokenizer.json`` and a plain byte tokenizer, both with an incremental,
UTF-8-safe stream decoder.

The reference ships a C tokenizer with an HF fallback (crates/server/src/tokenizer.rs:1-60); here the BPE encoder is
written against the ``tokenizer.json`` format directly (byte-level pre-tokenizer, ranked merges, added/special tokens split
out before pre-tokenization), with the HF ``tokenizers`` wheel used only as the test oracle.  Synthetic-prompt benchmarks
pass token ids and never touch this module.
"""
from __future__ import annotations

import json
import os
from functools import lru_cache

import regex

GPT2_SPLIT = r"""'(?:[sdmt]|ll|ve|re)| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""


@lru_cache(maxsize=1)
def bytes_to_unicode() -> dict:
    """The GPT-2 byte <-> printable-codepoint table byte-level BPE vocabularies are written in."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


class StreamDecoder:
    """Incremental detokenizer: push token ids, get only the text that is complete UTF-8 (a multi-byte character split over
    tokens is held back until its last byte arrives)."""

    def __init__(self, tok: "Tok", skip_special: bool = True):
        self.tok, self.skip_special = tok, skip_special
        self.pending = b""

    def push(self, ids) -> str:
        self.pending += self.tok.decode_bytes(ids, self.skip_special)
        # longest prefix that decodes: cut at most 3 trailing bytes of an unfinished character
        for cut in range(0, min(4, len(self.pending) + 1)):
            head = self.pending[:len(self.pending) - cut]
            try:
                text = head.decode("utf-8")
            except UnicodeDecodeError:
                continue
            self.pending = self.pending[len(head):]
            return text
        text = self.pending.decode("utf-8", errors="replace")   # not UTF-8 at all: replace, never stall the stream
        self.pending = b""
        return text

    def flush(self) -> str:
        text = self.pending.decode("utf-8", errors="replace")
        self.pending = b""
        return text


class Tok:
    vocab_size: int = 0
    eos_ids: tuple = ()
    bos_id: int | None = None

    def encode(self, text: str, allow_special: bool = True) -> list:
        raise NotImplementedError

    def decode_bytes(self, ids, skip_special: bool = True) -> bytes:
        raise NotImplementedError

    def decode(self, ids, skip_special: bool = True) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")

    def stream(self, skip_special: bool = True) -> StreamDecoder:
        return StreamDecoder(self, skip_special)

    def special_id(self, text: str):
        return None


class ByteTokenizer(Tok):
    """ids 0..255 are bytes; specials follow.  For mock / synthetic models whose vocabulary has no text meaning."""

    SPECIALS = ("<|bos|>", "<|eos|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>")
    VISION_SPECIALS = ("<|vision_start|>", "<|image_pad|>", "<|vision_end|>")        # present when the vocabulary has room for them

    def __init__(self, vocab_size: int = 512):
        if vocab_size < 256 + len(self.SPECIALS):
            raise ValueError("byte tokenizer needs a vocabulary of at least 264")
        self.vocab_size = vocab_size
        if vocab_size >= 256 + len(self.SPECIALS) + len(self.VISION_SPECIALS):
            self.SPECIALS = self.SPECIALS + self.VISION_SPECIALS
        self.special = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self.special_rev = {v: k for k, v in self.special.items()}
        self.bos_id, self.eos_ids = self.special["<|bos|>"], (self.special["<|eos|>"], self.special["<|im_end|>"])
        self._split = regex.compile("(" + "|".join(regex.escape(s) for s in self.SPECIALS) + ")")

    def encode(self, text, allow_special=True):
        if not allow_special:
            return list(text.encode("utf-8"))
        out = []
        for part in self._split.split(text):
            if part in self.special:
                out.append(self.special[part])
            elif part:
                out.extend(part.encode("utf-8"))
        return out

    def decode_bytes(self, ids, skip_special=True):
        out = bytearray()
        for i in ids:
            if i < 256:
                out.append(i)
            elif i in self.special_rev:
                if not skip_special:
                    out += self.special_rev[i].encode()
            else:
                out += b"?"    # ids beyond the byte range have no text in this vocabulary; they are not specials, so they stay visible
        return bytes(out)

    def special_id(self, text):
        return self.special.get(text)


class BpeTokenizer(Tok):
    """Byte-level BPE from ``tokenizer.json`` (models of type BPE with a ByteLevel pre-tokenizer, optionally preceded by a regex Split)."""

    def __init__(self, spec: dict, eos_ids=(), bos_id=None):
        model = spec.get("model") or {}
        if model.get("type") != "BPE":
            raise ValueError(f"tokenizer.json model type {model.get('type')!r} is not supported (BPE only)")
        self.vocab = {str(k): int(v) for k, v in model["vocab"].items()}
        merges = model.get("merges") or []
        self.ranks = {}
        for r, m in enumerate(merges):
            a, b = (m.split(" ", 1) if isinstance(m, str) else m)
            self.ranks[(a, b)] = r
        self.added = {}
        self.special_set = set()
        for t in spec.get("added_tokens") or []:
            self.added[t["content"]] = int(t["id"])
            if t.get("special"):
                self.special_set.add(int(t["id"]))
        self.id_to_tok = {v: k for k, v in self.vocab.items()}
        self.id_to_tok.update({v: k for k, v in self.added.items()})
        self.vocab_size = max(self.id_to_tok) + 1
        self.pattern_text = self._split_pattern(spec.get("pre_tokenizer")) or GPT2_SPLIT
        self.pattern = regex.compile(self.pattern_text)
        self._added_split = regex.compile("(" + "|".join(regex.escape(s) for s in sorted(self.added, key=len, reverse=True)) + ")") if self.added else None
        self.b2u = bytes_to_unicode()
        self.u2b = {c: b for b, c in self.b2u.items()}
        self.eos_ids, self.bos_id = tuple(eos_ids), bos_id
        self._cache = {}
        self._native = self._make_native()
        self._native_kind = None        # the native scanner's id of this file's split pattern (None: `regex` does the split)
        if self._native is not None:
            from ..native import host
            self._native_kind = host.pretok_kind(self.pattern_text)

    def _make_native(self):
        """The merge loop in the host library, when every merge maps onto token ids (else the Python loop below runs)."""
        try:
            from ..native import host
            byte_ids = [self.vocab.get(self.b2u[b], -1) for b in range(256)]
            triples = []
            for (a, b), _r in sorted(self.ranks.items(), key=lambda kv: kv[1]):
                ia, ib, im = self.vocab.get(a), self.vocab.get(b), self.vocab.get(a + b)
                if ia is None or ib is None or im is None:
                    return None          # a merge whose pieces are not all tokens: the string-level loop handles such a file
                triples.append((ia, ib, im))
            return host.BpeCore(byte_ids, triples)
        except (OSError, RuntimeError):
            return None

    @staticmethod
    def _split_pattern(pre):
        if not pre:
            return None
        items = pre.get("pretokenizers") if pre.get("type") == "Sequence" else [pre]
        for it in items or []:
            if it.get("type") == "Split":
                p = it.get("pattern") or {}
                return p.get("Regex") or (regex.escape(p["String"]) if "String" in p else None)
        return None

    @staticmethod
    def from_dir(folder: str) -> "BpeTokenizer":
        spec = json.load(open(os.path.join(folder, "tokenizer.json"), encoding="utf-8"))
        eos, bos = [], None
        gp = os.path.join(folder, "generation_config.json")
        if os.path.exists(gp):
            g = json.load(open(gp))
            e = g.get("eos_token_id")
            eos = [e] if isinstance(e, int) else list(e or [])
            bos = g.get("bos_token_id")
        return BpeTokenizer(spec, eos, bos)

    def _bpe(self, word: str) -> list:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, bi = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            parts[bi:bi + 2] = [parts[bi] + parts[bi + 1]]
        ids = []
        for p in parts:
            if p in self.vocab:
                ids.append(self.vocab[p])
            else:                       # unknown piece: fall back to its bytes' own tokens
                ids.extend(self.vocab[c] for c in p if c in self.vocab)
        if len(self._cache) < 200_000:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str) -> list:
        if self._native is not None and self._native_kind is not None:
            return self._native.encode_text(text, self._native_kind)           # split + merges in one native call
        if self._native is not None:
            return self._native.encode_pieces(m.group(0).encode("utf-8") for m in self.pattern.finditer(text))
        out = []
        for m in self.pattern.finditer(text):
            out.extend(self._bpe("".join(self.b2u[b] for b in m.group(0).encode("utf-8"))))
        return out

    def encode(self, text, allow_special=True):
        if not allow_special or self._added_split is None:
            return self._encode_plain(text)
        out = []
        for part in self._added_split.split(text):
            if part in self.added:
                out.append(self.added[part])
            elif part:
                out.extend(self._encode_plain(part))
        return out

    def decode_bytes(self, ids, skip_special=True):
        out = bytearray()
        for i in ids:
            t = self.id_to_tok.get(int(i))
            if t is None:
                continue
            if int(i) in self.added.values():
                if not (skip_special and int(i) in self.special_set):
                    out += t.encode("utf-8")
                continue
            for c in t:
                b = self.u2b.get(c)
                if b is None:
                    out += c.encode("utf-8")
                else:
                    out.append(b)
        return bytes(out)

    def special_id(self, text):
        return self.added.get(text)


class _HfStream:
    """Incremental detokenizer over a tokenizer that only decodes whole id lists to text: decode the ids since the last rebase, emit what
    is new, hold back while the text ends in an unfinished character (the replacement mark)."""
    CONTEXT = 6          # ids kept as left context when the window is rebased (decoders may join a token to its predecessor)
    REBASE = 96          # ids after which the window is rebased, so a long stream does not re-decode its whole history every token

    def __init__(self, tok: "HfTokenizer", skip_special: bool):
        self.tok, self.skip = tok, skip_special
        self.ids, self.emitted = [], 0

    def push(self, ids) -> str:
        self.ids.extend(int(i) for i in ids)
        text = self.tok.decode(self.ids, self.skip)
        if text.endswith("\ufffd"):
            return ""
        out, self.emitted = text[self.emitted:], len(text)
        if len(self.ids) > self.REBASE:
            self.ids = self.ids[-self.CONTEXT:]
            self.emitted = len(self.tok.decode(self.ids, self.skip))
        return out

    def flush(self) -> str:
        text = self.tok.decode(self.ids, self.skip)
        out, self.ids, self.emitted = text[self.emitted:], [], 0
        return out


class HfTokenizer(Tok):
    """Any `tokenizer.json` the `tokenizers` library can load (Unigram / SentencePiece-style, WordPiece, BPE variants this module's own
    byte-level BPE does not cover).  The fallback path of `load_tokenizer`."""

    def __init__(self, path: str, eos_ids=(), bos_id=None):
        import tokenizers
        self.tk = tokenizers.Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        self.eos_ids, self.bos_id = tuple(eos_ids), bos_id

    def encode(self, text, allow_special=True):
        return list(self.tk.encode(text, add_special_tokens=False).ids)

    def decode(self, ids, skip_special=True):
        return self.tk.decode([int(i) for i in ids], skip_special_tokens=skip_special)

    def decode_bytes(self, ids, skip_special=True):
        return self.decode(ids, skip_special).encode("utf-8")

    def stream(self, skip_special=True):
        return _HfStream(self, skip_special)

    def special_id(self, text):
        return self.tk.token_to_id(text)


def load_tokenizer(folder: str | None, vocab_size: int) -> Tok:
    """The pack's tokenizer.json when there is one (this module's byte-level BPE, else whatever the `tokenizers` library can load), else
    the byte tokenizer over the model's vocabulary."""
    if folder and os.path.exists(os.path.join(folder, "tokenizer.json")):
        try:
            return BpeTokenizer.from_dir(folder)
        except (ValueError, KeyError) as own:
            eos, bos = [], None
            gp = os.path.join(folder, "generation_config.json")
            if os.path.exists(gp):
                g = json.load(open(gp))
                e = g.get("eos_token_id")
                eos = [e] if isinstance(e, int) else list(e or [])
                bos = g.get("bos_token_id")
            try:
                return HfTokenizer(os.path.join(folder, "tokenizer.json"), eos, bos)
            except Exception as hf:  # noqa: BLE001  (neither path can read the file: say both reasons)
                raise ValueError(f"tokenizer.json: not byte-level BPE ({own}) and the tokenizers library refused it ({hf})") from hf
    return ByteTokenizer(max(vocab_size, 264))
