"""Quantizer-side conformance data of the reference tree (read as data when mounted): the trellis round trip (packed bits -> states ->
fp16 values) through both decoders and the packer, and the encoder's search quality on the reference's eight fixed tiles."""
import json
import os

import numpy as np

from rexl3_b200.format import exl3
from rexl3_b200.native import host
from rexl3_b200.quant.trellis import encode_tiles


def test_trellis_roundtrip_vectors(reference_fixtures):
    d = json.load(open(os.path.join(reference_fixtures, "quant_trellis_roundtrip.json")))
    for name, want in d["codebook_fnv"].items():
        assert exl3.fnv1a_u16(exl3.codebook(name)) == int(want, 16)
    assert [w["twice"] for w in d["widths"]] == list(exl3.ALL_TWICE)
    for w in d["widths"]:
        b = exl3.Bits(w["twice"])
        assert w["words"] == b.tile_words
        tr = np.frombuffer(bytes.fromhex(w["trellis_hex"]), dtype="<i2").reshape(d["kt"], d["nt"], b.tile_words)
        st = np.frombuffer(bytes.fromhex(w["states_hex"]), dtype="<u2").reshape(d["kt"], d["nt"], 256)
        wq = np.frombuffer(bytes.fromhex(w["wq_hex"]), dtype="<u2").reshape(d["kt"] * 16, d["nt"] * 16)
        assert np.array_equal(exl3.states(tr, b), st) and np.array_equal(host.states(tr), st)
        assert np.array_equal(exl3.unpack(tr, "mul1"), wq) and np.array_equal(host.unpack(tr, "mul1"), wq)
        assert exl3.fnv1a_u16(wq) == int(w["wq_fnv"], 16)
        assert np.array_equal(exl3.pack_tiles(st.reshape(-1, 256), b).reshape(tr.shape), tr)      # the packer is the decoder's inverse


def _encode_cases(path):
    lines = open(path).read().splitlines()
    x = np.frombuffer(bytes.fromhex(lines[3].split()[1]), dtype="<f4").reshape(int(lines[2].split()[1]), 256)
    cases, i = [], 4
    while i < len(lines):
        if lines[i].startswith("case"):
            hdr, d = lines[i].split(), {}
            i += 1
            while lines[i] != "end":
                k, v = lines[i].split(None, 1)
                d[k] = v
                i += 1
            cases.append((hdr, d))
        i += 1
    return x, cases


def test_encoder_matches_the_reference_search_quality(reference_fixtures):
    """Same tiles, same codebook (mul1), every width: this encoder's squared error per tile is within half a percent of the error the
    reference's encoder recorded (both are tail-biting searches over the same trellis; their states need not be identical)."""
    x, cases = _encode_cases(os.path.join(reference_fixtures, "exl3_trellis_encode.txt"))
    seen = 0
    for hdr, d in cases:
        if "states" not in d or hdr[2] != "fp32":
            continue
        b = exl3.Bits(int(hdr[1]))
        st = np.frombuffer(bytes.fromhex(d["states"]), dtype="<u2").reshape(-1, 256)
        theirs = ((x - exl3.codebook_f32("mul1")[st]) ** 2).sum(1)
        packed, mine = encode_tiles(x, b, "mul1")
        # the cost this encoder reports is the cost of what it packed
        dec = exl3.codebook_f32("mul1")[exl3.states(packed, b)]
        assert np.allclose(((x - dec) ** 2).sum(1), mine, rtol=1e-4, atol=1e-6)
        assert np.all(mine <= theirs * 1.005 + 1e-6), (hdr, mine, theirs)
        seen += 1
    assert seen == len(exl3.ALL_TWICE)
