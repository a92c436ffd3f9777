"""Pack fingerprint, per-tensor CRC records and the per-file lock."""
import dataclasses
import json
import os

from rexl3_b200.format import verify
from rexl3_b200.models import dense
from rexl3_b200.quant import quantize


def _pack(tmp_path, seed=1, name="p"):
    cfg = dataclasses.replace(dense.CONFIGS["tiny-llama"], n_layers=1, vocab=256, ffn=128)
    folder = str(tmp_path / name)
    quantize.write_pack(folder, dense.random_weights(cfg, seed=seed))
    return folder


def test_fingerprint_is_about_structure_not_payload(tmp_path):
    a, b = _pack(tmp_path, 1, "a"), _pack(tmp_path, 2, "b")
    assert verify.fingerprint(a) == verify.fingerprint(b)            # same inventory and quantization record, different weights
    c = json.load(open(os.path.join(b, "config.json")))
    c["quantization_config"]["bits"] = 3.0
    json.dump(c, open(os.path.join(b, "config.json"), "w"))
    assert verify.fingerprint(a) != verify.fingerprint(b)


def test_crc_and_lock_catch_a_flipped_byte(tmp_path):
    folder = _pack(tmp_path)
    assert verify.write_crc(folder) > 5
    lock = verify.write_lock(folder)
    assert lock["schema"] == verify.LOCK_SCHEMA and "model.safetensors" in lock["files"] and "crc32.txt" in lock["files"]
    assert verify.verify_crc(folder) == [] and verify.verify_lock(folder) == [] and verify.main([folder, "--check"]) == 0
    path = os.path.join(folder, "model.safetensors")
    raw = bytearray(open(path, "rb").read())
    raw[-3] ^= 0x40                                                   # inside the last tensor's payload
    open(path, "wb").write(raw)
    bad = verify.verify_crc(folder)
    assert len(bad) == 1 and "crc" in bad[0]
    assert any("model.safetensors" in b for b in verify.verify_lock(folder))
    assert verify.verify_lock(folder, sizes_only=True) == []         # same size: the cheap check cannot see it
    assert verify.main([folder, "--check"]) == 1
    os.remove(os.path.join(folder, "crc32.txt"))
    assert verify.verify_crc(folder) == ["crc32.txt is missing"]
    assert any("crc32.txt: missing" in b for b in verify.verify_lock(folder))


def test_server_refuses_a_pack_that_fails_verification(tmp_path):
    import pytest

    from rexl3_b200.server import main
    folder = _pack(tmp_path)
    verify.write_crc(folder)
    verify.write_lock(folder)
    base = ["--backend", "cpu", "--model", folder, "--slots", "2", "--max-model-len", "128"]
    for mode in ("sizes", "crc", "lock"):
        make, _tok, _fmt, name, info = main.build(main.parser().parse_args(base + ["--verify-pack", mode]))
        assert len(info["pack_fingerprint"]) == 64
    path = os.path.join(folder, "model.safetensors")
    raw = bytearray(open(path, "rb").read())
    raw[-5] ^= 0x01
    open(path, "wb").write(raw)
    main.build(main.parser().parse_args(base + ["--verify-pack", "sizes"]))          # same size: passes the cheap check
    for mode in ("crc", "lock"):
        with pytest.raises(SystemExit, match="pack refused"):
            main.build(main.parser().parse_args(base + ["--verify-pack", mode]))
