"""The native pre-tokenizer against the `regex` oracle: the three split patterns on hostile and multilingual text; the one-call encode path."""
import random

import pytest
import regex

from rexl3_b200.native import host

PATTERNS = {0: host._GPT2, 1: host._CL100K, 2: host._QWEN2}
SAMPLES = [
    "", " ", "  ", "\n", " \n ", "a", "Hello, world!  It's 12345 o'clock; we'll see... I'D say they'RE fine, aren't they?",
    "tabs\tand\r\nCRLF\r\n\r\n  indented\n\n\n   three", "trailing spaces   ", "   leading", "x  y   z    w", "a\n b\n  c",
    "price: $1,234,567.89 (approx.) #hash @user 100% a_b-c+d=e", "def f(x):\n    return x ** 2  # comment\n\n\nclass A:\n\tpass\n",
    "Grüße aus München, naïve café, Ångström, ſtraße's", "Привет, мир! Это тест 123 и ещё.", "你好，世界！这是一个测试。１２３ 四五六",
    "مرحبا بالعالم ١٢٣", "नमस्ते दुनिया १२३", "日本語のテキストとカタカナ、ひらがな。", "emoji 😀😃 👨‍👩‍👧‍👦 flags 🇩🇪🇫🇷 ok", "zero\u200bwidth\u00a0nbsp\u2003emspace\u3000ideographic",
    "'s 't 're 've 'm 'll 'd 'S 'T 'RE 'Ve 'x '' ' 's", "it's John's; they've, I'm, we'll, he'd, y'all'd've", "１２３４５６７ 1234567890 ①②③ ½ Ⅷ", "a1b2c3 4d5e 6.7.8",
    "....!!!???\n\n", "--- \n*** \r\n=== ", "\x00\x01\x1c\x1d\x1e\x1f\x7f control", "mixed\u2028line\u2029para\x0b\x0csep\x85nel",
]


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_split_equals_the_regex_oracle(kind):
    pat = regex.compile(PATTERNS[kind])
    rng = random.Random(kind)
    alphabet = list(" \n\r\t'.,!?-_$%()[]{}0123456789abcXYZäßЖя中日한あア١२😀\u00a0\u3000\u200b") + ["'s", "'ll", "'RE", "  ", "\n\n", "12345"]
    texts = SAMPLES + ["".join(rng.choice(alphabet) for _ in range(rng.randint(1, 60))) for _ in range(400)]
    for t in texts:
        want = [m.group(0) for m in pat.finditer(t)]
        got = host.pretok_split(t, kind)
        assert got == want, (kind, t, got, want)
        assert "".join(got) == t


def test_every_code_point_class_agrees_with_the_oracle():
    """One string per plane slice: a letter, number or space misclassified anywhere shows up as a different split."""
    pat = regex.compile(host._CL100K)
    for base in range(0, 0x30000, 0x400):
        t = " ".join("a" + chr(cp) + "1" for cp in range(base, base + 0x400) if not 0xD800 <= cp <= 0xDFFF)
        assert host.pretok_split(t, 1) == [m.group(0) for m in pat.finditer(t)], hex(base)


def test_one_call_encode_equals_split_then_merge():
    from rexl3_b200.server.tokenizer import BpeTokenizer, bytes_to_unicode
    b2u = bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    merges = []
    for a, b in [("t", "h"), ("th", "e"), ("Ġ", "the"), ("i", "n"), ("Ġ", "a"), ("1", "2"), ("e", "r"), ("Ġ", "w")]:
        vocab[a + b] = len(vocab)
        merges.append(f"{a} {b}")
    for kind, pat in PATTERNS.items():
        spec = {"model": {"type": "BPE", "vocab": vocab, "merges": merges}, "added_tokens": [{"content": "<|eot|>", "id": len(vocab), "special": True}],
                "pre_tokenizer": {"type": "Sequence", "pretokenizers": [{"type": "Split", "pattern": {"Regex": pat}, "behavior": "Isolated"}, {"type": "ByteLevel"}]}}
        tok = BpeTokenizer(spec, [len(vocab)], None)
        assert tok._native is not None and tok._native_kind == kind
        for t in SAMPLES:
            fast = tok.encode(t + "<|eot|>")
            tok._native_kind = None                 # the regex split feeding the same native merges
            slow = tok.encode(t + "<|eot|>")
            tok._native_kind = kind
            assert fast == slow, (kind, t)
            assert tok.decode_bytes(fast, skip_special=False).decode("utf-8") == t + "<|eot|>"
