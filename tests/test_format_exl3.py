"""EXL3 codec: conformance vectors, pack/unpack round trips for all 11 widths, strips, signs."""
import json
import os

import numpy as np
import pytest

from rexl3_b200.format import exl3


def _trellis(seed, kt, nt, bits):
    return (exl3.splitmix_stream(seed, kt * nt * bits.tile_words) & 0xFFFF).astype(np.uint16).view(np.int16).reshape(kt, nt, -1)


def _f64s(seed, n, lo, hi):
    return lo + (hi - lo) * ((exl3.splitmix_stream(seed, n) >> np.uint64(11)).astype(np.float64) * 2.0 ** -53)


def _combos():
    return [(cb, t) for cb in exl3.CODEBOOKS for t in exl3.ALL_TWICE if t % 2 == 0 or cb == "mul1"]


def test_codebooks_match_conformance_hashes(reference_fixtures):
    f = json.load(open(os.path.join(reference_fixtures, "exl3.json")))
    for cb in exl3.CODEBOOKS:
        assert exl3.fnv1a_u16(exl3.codebook(cb)) == f["codebook_fnv"][cb]


def test_unpack_bit_exact_all_27_combinations(reference_fixtures):
    f = json.load(open(os.path.join(reference_fixtures, "exl3.json")))
    combos = _combos()
    assert len(combos) == 27
    for idx, (cb, t) in enumerate(combos):
        b = exl3.Bits(t)
        w = exl3.unpack(_trellis(5000 + idx, 4, 3, b), cb)
        key = f"{cb}:{t // 2}" if t % 2 == 0 else f"{cb}:{t / 2:.1f}"
        assert exl3.fnv1a_u16(w) == f["unpack_kt4_nt3"][key], key


def test_forward_matches_float64_reference(reference_fixtures):
    f = json.load(open(os.path.join(reference_fixtures, "exl3.json")))
    q = lambda v: v.astype(np.float16).astype(np.float64)  # noqa: E731
    for idx, e in enumerate(f["forward_k128_n256_rows2"]):
        b = exl3.Bits.of(e["bits"])
        kt, nt, rows = 8, 16, 2
        tr = _trellis(9000 + idx, kt, nt, b)
        x = _f64s(9100 + idx, rows * kt * 16, -1, 1).reshape(rows, -1)
        suh, svh = q(_f64s(9200 + idx, kt * 16, 0.5, 1.5)), q(_f64s(9300 + idx, nt * 16, 0.001, 0.05))
        bias = q(_f64s(9400 + idx, nt * 16, -0.1, 0.1)) if e["bias"] else None
        want = np.array(e["y"]).reshape(rows, -1)
        y = exl3.forward(x, tr, e["codebook"], suh, svh, bias)
        assert np.abs(y - want).max() <= 1e-12 * np.abs(want).max()
        w = exl3.decode_weight(tr, e["codebook"], suh, svh)
        y2 = x @ w + (0 if bias is None else bias)
        assert np.abs(y2 - want).max() <= 1e-11 * np.abs(want).max()


@pytest.mark.parametrize("twice", exl3.ALL_TWICE)
def test_pack_is_inverse_of_states_for_every_width(twice):
    b = exl3.Bits(twice)
    tr = exl3.random_trellis(3, 2, b, seed=twice)
    st = exl3.states(tr.reshape(6, -1), b)
    assert np.array_equal(exl3.pack_tiles(st, b), tr.reshape(6, -1))


def test_pack_refuses_inconsistent_windows():
    b = exl3.Bits.of(4)
    st = exl3.states(exl3.random_trellis(1, 1, b, 3).reshape(1, -1), b).copy()
    st[0, 10] ^= 0x8000  # top bit is shared with earlier windows
    with pytest.raises(ValueError):
        exl3.pack_tiles(st, b)


def test_stream_ends_integer_and_half_widths():
    assert exl3.Bits.of(4).stream_ends()[0] == 4 and exl3.Bits.of(4).stream_ends()[255] == 1024
    e = exl3.Bits.of(2.5).stream_ends()
    assert e[0] == 2 and e[1] == 5 and e[255] == 640
    assert np.all(np.diff(e) >= 2) and np.all(np.diff(e) <= 3)


def test_strip_equals_dense_columns():
    b = exl3.Bits.of(3)
    tr = exl3.random_trellis(8, 24, b, 1)
    rng = np.random.default_rng(0)
    suh = rng.uniform(0.5, 1.5, 128).astype(np.float16)
    svh = rng.uniform(0.01, 0.05, 384).astype(np.float16)
    w = exl3.decode_weight(tr, "3inst", suh, svh)
    for s in range(3):
        np.testing.assert_allclose(exl3.decode_strip(tr, s, "3inst", suh, svh), w[:, 128 * s:128 * s + 128], rtol=1e-12, atol=1e-15)


def test_unpack_signs():
    s = exl3.unpack_signs(np.array([0b101, -32768], dtype=np.int16))
    assert s[0] == -1 and s[1] == 1 and s[2] == -1 and s[3] == 1 and s[31] == -1 and s[30] == 1


def test_width_validation():
    with pytest.raises(ValueError):
        exl3.Bits.of(4.5)
    with pytest.raises(ValueError):
        exl3.Bits.from_trellis_last(20)
