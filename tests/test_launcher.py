"""Lifecycle verbs of a runtime recipe on a throw-away tree with a mock-backend profile: setup refuses a changed tree and a pack that is
not the locked one, start / status / verify / logs / stop / reset-state drive a real server process by its recorded pid."""
import io
import json
import os
import socket
import time

import pytest

from rexl3_b200 import launcher, recipes


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tree(tmp_path, lock=None):
    vdir = tmp_path / "runtimes" / "fam" / "tiny" / "v1"
    vdir.mkdir(parents=True)
    (vdir.parent / "MODEL.json").write_text(json.dumps({"schema": "rexl3.prod-model.v1", "family": "fam", "model": "tiny", "runtime_id": "tiny-mock"}))
    (vdir.parent / "LATEST").write_text("v1\n")
    prof = {"schema": "rexl3.runtime-profile.v1", "state": "final", "runtime_id": "tiny-mock", "default_profile": "mock", "profiles": {"mock": {
        "kind": "single", "site_fields": ["http_port"], "http_host": "127.0.0.1", "readiness_timeout_s": 60,
        "argv": ["--backend", "mock", "--mock", "vocab=512", "--slots", "2", "--max-model-len", "256", "--host", "@HTTP_HOST@", "--port", "@HTTP_PORT@",
                 "--served-model-name", "tiny"],
        "smoke_request": {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}}}}
    (vdir / "profile.json").write_text(json.dumps(prof))
    (vdir / "model.lock.json").write_text(json.dumps(lock or {"schema": launcher.LOCK_SCHEMA, "packs": {"target": {"source": "random-init", "config": "tiny"}}}))
    recipes.seal(str(vdir))
    return vdir


def _run(argv):
    out = io.StringIO()
    rc = launcher.main(argv, out=out)
    return rc, out.getvalue()


def test_setup_refuses_a_changed_tree_and_a_foreign_pack(tmp_path, capsys):
    pack = tmp_path / "pack"
    pack.mkdir()
    (pack / "config.json").write_text("{}")
    (pack / "model.safetensors").write_bytes(b"x" * 100)
    lock = launcher.write_lock_for_folder(str(pack), repo="someone/pack", revision="abc")
    assert set(lock["packs"]["target"]["files"]) == {"config.json", "model.safetensors"}
    vdir = _tree(tmp_path, lock)
    site = tmp_path / "site.json"
    site.write_text(json.dumps({"http_port": _free_port(), "model_dir": str(pack)}))
    assert _run(["setup", "--recipe", str(vdir), "--site", str(site), "--crc"])[0] == 0
    (pack / "model.safetensors").write_bytes(b"y" * 100)                      # same size, other bytes: only --crc sees it
    assert _run(["setup", "--recipe", str(vdir), "--site", str(site)])[0] == 0
    assert _run(["setup", "--recipe", str(vdir), "--site", str(site), "--crc"])[0] == 2
    assert "PACK_MISMATCH" in capsys.readouterr().err
    (pack / "model.safetensors").write_bytes(b"y" * 99)
    assert _run(["setup", "--recipe", str(vdir), "--site", str(site)])[0] == 2
    (vdir / "profile.json").write_text((vdir / "profile.json").read_text() + " ")
    assert _run(["setup", "--recipe", str(vdir), "--site", str(site)])[0] == 2
    assert "TREE_CHANGED" in capsys.readouterr().err
    assert _run(["install-deps", "--recipe", str(vdir)])[0] == 2


def test_doctor_reads_a_fake_probe_and_changes_nothing(tmp_path):
    vdir = _tree(tmp_path)
    site = tmp_path / "site.json"
    site.write_text(json.dumps({"http_port": _free_port()}))
    out = io.StringIO()
    assert launcher.main(["doctor", "--recipe", str(vdir), "--site", str(site)], out=out) in (0, 1)
    text = out.getvalue()
    assert "python" in text and "port" in text and "is free" in text
    r = recipes.resolve(str(tmp_path / "runtimes"), "fam", "tiny", {"http_port": 1}, "v1")
    r.argv[r.argv.index("mock")] = "cuda"
    r.kind, r.ranks = "tp", 2
    rep = launcher.doctor(r, nvml=lambda i: {"total_mib": 1000, "free_mib": 990, "compute_pids": []} if i == 0 else (_ for _ in ()).throw(RuntimeError("no gpu")))
    gp = next(c for c in rep["checks"] if c["name"] == "gpus")
    assert not gp["ok"] and "1 answered" in gp["detail"] and not rep["ok"]


def test_start_status_verify_logs_stop_reset(tmp_path):
    vdir = _tree(tmp_path)
    port = _free_port()
    site = tmp_path / "site.json"
    site.write_text(json.dumps({"http_port": port}))
    sd = str(tmp_path / "state")
    common = ["--recipe", str(vdir), "--state-dir", sd]
    rc, text = _run(["print-command", "--site", str(site)] + common)
    assert rc == 0 and "rexl3_b200.server" in text and f"--port {port}" in text
    assert _run(["status"] + common)[0] == 3
    rc, text = _run(["start", "--site", str(site), "--no-wait"] + common)
    assert rc == 0 and "started pid" in text
    try:
        for _ in range(240):
            if launcher.health("127.0.0.1", port)[0] == 200:
                break
            time.sleep(0.25)
        rc, text = _run(["status"] + common)
        st = json.loads(text)
        assert rc == 0 and st["running"] and st["health"] == 200 and st["profile"] == "mock"
        assert _run(["start", "--site", str(site), "--no-wait"] + common)[0] == 2          # a second start is refused while the first is alive
        rc, text = _run(["verify", "--site", str(site)] + common)
        assert rc == 0 and "smoke request answered (4 tokens)" in text
        assert _run(["reset-state"] + common)[0] == 2
        rc, text = _run(["diagnostics", "--site", str(site)] + common)
        doc = json.loads(text)
        assert doc["running"] and doc["tree_problems"] == [] and "command" in doc
    finally:
        rc, text = _run(["stop"] + common)
    assert rc == 0 and "stopped pid" in text
    for _ in range(100):
        if _run(["status"] + common)[0] == 3:
            break
        time.sleep(0.1)
    assert _run(["status"] + common)[0] == 3
    assert _run(["logs"] + common)[0] == 0
    assert _run(["reset-state"] + common)[0] == 0 and not os.path.exists(os.path.join(sd, "state.json"))
