"""The host library's EXL3 codec against the numpy oracle, and the parallel range reader."""
import os

import numpy as np
import pytest

from rexl3_b200.format import exl3, safetensors_io
from rexl3_b200.native import host


@pytest.mark.parametrize("twice", exl3.ALL_TWICE)
def test_states_and_unpack_are_bit_exact(twice):
    rng = np.random.default_rng(twice)
    b = exl3.Bits(twice)
    tr = rng.integers(-32768, 32768, size=(8, 16, b.tile_words), dtype=np.int16)
    assert np.array_equal(host.states(tr), exl3.states(tr, b))
    for cb in exl3.CODEBOOKS:
        assert np.array_equal(host.unpack(tr, cb), exl3.unpack(tr, cb))
    assert np.array_equal(host.unpack(tr, "3inst", threads=1), host.unpack(tr, "3inst", threads=5))


def test_decode_weight_matches_the_matrix_form():
    rng = np.random.default_rng(0)
    tr = rng.integers(-32768, 32768, size=(16, 8, exl3.Bits.of(3.0).tile_words), dtype=np.int16)
    suh = np.where(rng.random(256) < 0.5, -1.0, 1.0)
    svh = rng.normal(size=128) * 0.02
    want = exl3.decode_weight(tr, "mcg", suh, svh)
    got = host.decode_weight(tr, "mcg", suh, svh)
    assert got.shape == want.shape and np.allclose(got, want, rtol=1e-12, atol=1e-12 * np.abs(want).max())
    assert np.allclose(host.decode_weight(tr, "mcg"), exl3.decode_weight(tr, "mcg"), rtol=1e-12, atol=1e-12)
    with pytest.raises(ValueError):
        host.decode_weight(tr[:3], "mcg")


@pytest.mark.parametrize("direct", [False, True])
def test_read_ranges(tmp_path, direct):
    rng = np.random.default_rng(1)
    blob = rng.integers(0, 256, size=(20 << 20) + 12345, dtype=np.uint8)
    path = tmp_path / "blob.bin"
    blob.tofile(path)
    offs = [0, 5, 4097, (9 << 20) + 3, blob.size - 100]
    sizes = [4, 70000, (9 << 20) + 11, 1, 100]
    starts, pos = [], 0
    for n in sizes:
        starts.append(pos)
        pos += n + 7
    dst = np.zeros(pos, dtype=np.uint8)
    host.read_ranges(str(path), offs, sizes, dst, starts, threads=4, direct=direct)     # a file system without O_DIRECT falls back
    for o, n, s in zip(offs, sizes, starts):
        assert np.array_equal(dst[s:s + n], blob[o:o + n])
    with pytest.raises(OSError):
        host.read_ranges(str(path), [blob.size - 10], [11], dst, [0])
    with pytest.raises(OSError):
        host.read_ranges(str(tmp_path / "missing"), [0], [1], dst, [0])
    with pytest.raises(ValueError):
        host.read_ranges(str(path), [0], [dst.size + 1], dst, [0])


def test_pack_loads_through_the_prefetcher(tmp_path):
    import dataclasses

    from rexl3_b200.models import dense
    from rexl3_b200.quant import quantize
    cfg = dataclasses.replace(dense.CONFIGS["tiny-llama"], n_layers=1, vocab=256, ffn=128)
    w = dense.random_weights(cfg, seed=3)
    folder = str(tmp_path / "pack")
    quantize.write_pack(folder, w)
    a = quantize.load_pack(folder, threads=0)        # plain per-tensor reads
    b = quantize.load_pack(folder, threads=3)
    assert not safetensors_io._PREFETCHED
    for la, lb in zip(a.layers, b.layers):
        for name in ("qkv", "o", "gate_up", "down"):
            x, y = getattr(la, name), getattr(lb, name)
            assert np.array_equal(x.trellis, y.trellis) and np.array_equal(x.suh, y.suh) and np.array_equal(x.svh, y.svh)
        assert np.array_equal(la.attn_norm, lb.attn_norm)
    assert np.array_equal(a.embed, b.embed) and np.array_equal(a.lm_head.trellis, b.lm_head.trellis)
    assert os.path.exists(os.path.join(folder, "model.safetensors"))


def test_native_bpe_equals_the_python_merge_loop():
    from rexl3_b200.server import tokenizer
    b2u = tokenizer.bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    merges = []
    def add(a, b):
        merges.append(f"{a} {b}")
        vocab.setdefault(a + b, len(vocab))
    sp = b2u[ord(" ")]
    for a, b in [("t", "h"), ("th", "e"), (sp, "the"), ("a", "a"), ("aa", "a"), ("aa", "aa"), ("i", "n"), ("in", "g"), (sp, "a"), ("e", "r"), ("1", "2")]:
        add(a, b)
    spec = {"model": {"type": "BPE", "vocab": vocab, "merges": merges}, "added_tokens": [{"content": "<|x|>", "id": len(vocab), "special": True}]}
    tk = tokenizer.BpeTokenizer(spec)
    assert tk._native is not None
    py = tokenizer.BpeTokenizer(spec)
    py._native = None
    rng = np.random.default_rng(0)
    texts = ["the theme of the thing", "aaaaaaa aaaa aaaaa", "", " ", "bathing in the aaa<|x|>12 1212", "héllo ✓ 你好 the"]
    texts += ["".join(rng.choice(list("the aing12r\n"), size=int(rng.integers(1, 60)))) for _ in range(50)]
    for t in texts:
        assert tk.encode(t) == py.encode(t), t
        assert tk.decode(tk.encode(t), skip_special=False) == t
