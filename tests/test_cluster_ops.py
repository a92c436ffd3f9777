"""Cluster group operations: pre-flight with a fake GPU probe, GPU locks, state / status / down on plain child processes."""
import json
import os
import subprocess
import sys
import time

from rexl3_b200.cluster import ops
from rexl3_b200.cluster.schema import validate

DOC = {"schema_version": 1, "name": "box", "nodes": [{"name": "g0", "gpu": 0}, {"name": "g1", "gpu": 1}], "random_init": "tiny-llama",
       "groups": [{"name": "tp2", "ranks": ["g0", "g1"], "tp_port": 29611, "http_port": 8611}]}


def test_preflight_reports_each_fact(tmp_path):
    c = validate(DOC)
    lib = tmp_path / "lib.so"
    lib.write_bytes(b"x" * 100)
    locks = ops.GpuLocks(str(tmp_path / "locks"))
    probe = lambda i: {"total_mib": 183000, "free_mib": 180000 if i == 0 else 4000, "compute_pids": [] if i == 0 else [4242]}  # noqa: E731
    checks = ops.preflight(c, "tp2", need_mib=100000, gpu_probe=probe, port_free=lambda p: p != 8611, locks=locks,
                           libraries=[str(lib), str(tmp_path / "absent.so")])
    by = {ch.name: ch for ch in checks}
    assert by["binary:lib.so"].ok and len(by["binary:lib.so"].detail) == 16 and not by["binary:absent.so"].ok
    assert by["pack"].ok and "tiny-llama" in by["pack"].detail
    assert by["tp_port"].ok and not by["http_port"].ok
    assert by["gpu0:idle"].ok and by["gpu0:memory"].ok and not by["gpu1:idle"].ok and not by["gpu1:memory"].ok
    assert by["lock:gpu0"].ok and by["lock:gpu1"].ok

    def broken(i):
        raise RuntimeError("no NVML here")
    assert not any(ch.ok for ch in ops.preflight(c, "tp2", gpu_probe=broken, port_free=lambda p: True, libraries=[]) if ch.name.startswith("gpu"))


def test_gpu_locks_are_all_or_nothing_and_stale_locks_are_taken(tmp_path):
    locks = ops.GpuLocks(str(tmp_path))
    assert locks.acquire([0, 1], "a")
    assert not locks.acquire([1, 2], "b") and locks.holder(2) is None           # nothing taken on failure
    assert locks.acquire([0, 1], "a")                                           # the holder may re-acquire
    locks.release([0, 1], "b")                                                  # not the holder: no effect
    assert locks.holder(0)["group"] == "a"
    locks.release([0, 1], "a")
    assert locks.holder(0) is None
    dead = subprocess.Popen([sys.executable, "-c", "pass"])
    dead.wait()
    json.dump({"group": "ghost", "pid": dead.pid, "time": 0}, open(os.path.join(str(tmp_path), "gpu3.lock"), "w"))
    assert locks.holder(3) is None and locks.acquire([3], "b")


def test_status_and_down_touch_only_recorded_processes_of_this_package(tmp_path):
    sd = str(tmp_path / "state")
    assert ops.status(sd, "tp2")["state"] == "down" and ops.down(sd, "tp2") == []
    mine = [subprocess.Popen([sys.executable, "-c", "import time; time.sleep(60)  # rexl3_b200 rank"]) for _ in range(2)]
    other = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(60)"])
    try:
        ops.write_state(sd, "tp2", -1, [p.pid for p in mine] + [other.pid], 8611, str(tmp_path))
        st = ops.status(sd, "tp2", ready_probe=lambda port: port == 8611)
        assert st["state"] == "up" and st["ready"] is True and [r["alive"] for r in st["ranks"]] == [True] * 3
        hit = ops.down(sd, "tp2", grace_s=5.0)
        assert sorted(hit) == sorted(p.pid for p in mine)                       # the foreign process was not signalled
        for p in mine:
            assert p.wait(timeout=10) != 0
        assert other.poll() is None
        assert ops.status(sd, "tp2")["state"] == "down"
    finally:
        for p in mine + [other]:
            if p.poll() is None:
                p.kill()
                p.wait()


def test_tail_logs(tmp_path):
    (tmp_path / "rank0.log").write_text("\n".join(f"line {i}" for i in range(100)))
    out = ops.tail_logs(str(tmp_path), 2, lines=3)
    assert out[0] == ["line 97", "line 98", "line 99"] and out[1] is None


def test_cli_check_and_status(tmp_path, capsys):
    from rexl3_b200.cluster.__main__ import main
    f = tmp_path / "c.json"
    f.write_text(json.dumps(DOC))
    rc = main(["check", "--cluster", str(f), "--state-dir", str(tmp_path / "s"), "--no-gpu-probe"])
    out = capsys.readouterr().out
    assert "pack: random-init tiny-llama" in out and "tp_port" in out and rc in (0, 1)
    assert main(["status", "--cluster", str(f), "--state-dir", str(tmp_path / "s")]) == 0
    assert json.loads(capsys.readouterr().out)["state"] == "down"
    assert main(["logs", "--cluster", str(f), "--state-dir", str(tmp_path / "s")]) == 2


def test_check_derives_the_memory_need_from_the_plan():
    from rexl3_b200.cluster.__main__ import _planned_mib
    doc = dict(DOC, random_init="dense-27b", serve={"flags": ["--slots", "64", "--max-model-len", "8704"]})
    c = validate(doc)
    need = _planned_mib(c, c.groups["tp2"])
    # half of the weights (about 6 GB) + half of 64 x 8704 tokens of KV (about 68 GB) + the reserve
    assert 70_000 < need < 85_000
    assert _planned_mib(validate(dict(DOC, random_init="unknown-model")), c.groups["tp2"]) == 0
