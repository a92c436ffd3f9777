"""Ranks on other hosts through an ssh client: command wrapping, a stand-in client that runs on this host, the remote pre-flight facts."""
import json
import os
import stat
import subprocess
import sys

from rexl3_b200.cluster import ops, remote
from rexl3_b200.cluster.schema import rank_commands, validate
from rexl3_b200.cluster.supervise import LocalRunner

DOC = {"schema_version": 1, "name": "two-hosts", "random_init": "test-hd128",
       "nodes": [{"name": "a0", "gpu": 0}, {"name": "b0", "gpu": 1, "address": "node-b.example.invalid"}],
       "groups": [{"name": "tp2", "ranks": ["a0", "b0"], "tp_port": 29750, "http_port": 18750}]}


def fake_ssh(tmp_path):
    """A stand-in ssh client: drops its options and the host, runs the command through sh on this host, records what it was asked."""
    path = tmp_path / "fake_ssh"
    path.write_text("#!/bin/sh\nwhile [ \"$1\" != \"--\" ]; do echo \"$1\" >> \"%s\"; shift; done\nshift\nexec sh -c \"$1\"\n" % (tmp_path / "ssh_args.log"))
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    return str(path)


def test_remote_rank_is_wrapped_and_local_rank_is_not(tmp_path):
    c = validate(DOC)
    cmds = rank_commands(c, "tp2", sys.executable, ssh="/usr/bin/ssh", workdir="/srv/rexl3")
    (env0, argv0), (env1, argv1) = cmds
    assert argv0[0] == sys.executable and env0["RANK"] == "0" and "ssh" not in argv0[0]
    assert argv1[:2] == ["/usr/bin/ssh", "-tt"] and "node-b.example.invalid" in argv1 and env1 == {}
    remote_cmd = argv1[-1]
    assert remote_cmd.startswith("cd /srv/rexl3 && exec env ") and "RANK=1" in remote_cmd and "WORLD_SIZE=2" in remote_cmd and "MASTER_PORT=29750" in remote_cmd
    assert "python3 -m rexl3_b200.server" in remote_cmd and sys.executable not in remote_cmd
    assert remote.is_local(None) and remote.is_local("127.0.0.1") and not remote.is_local("node-b.example.invalid")


def test_runner_drives_a_remote_rank_through_the_client_and_ends_it_by_pid(tmp_path):
    ssh = fake_ssh(tmp_path)
    marker = tmp_path / "ran.txt"
    env, argv = remote.wrap({"RANK": "1", "GREETING": "hello there"}, ["sh", "-c", f"echo $RANK:$GREETING > {marker}; sleep 30"], "host-x", str(tmp_path), ssh)
    local = ({}, [sys.executable, "-c", "import time; time.sleep(0.8)"])
    att = LocalRunner([local, (env, argv)], max_runtime_s=0)()
    assert marker.read_text().strip() == "1:hello there"
    assert att.codes[0] == 0 and att.runtime_s < 20                      # the first exit took the other rank down with it (by pid), not after 30 s
    assert "host-x" in (tmp_path / "ssh_args.log").read_text()


def test_remote_preflight_compares_the_build_and_reads_ports_and_gpus(tmp_path):
    c = validate(DOC)
    from rexl3_b200.ops import lib as oplib
    here = ops._sha256(oplib.LIB_PATH)[:16] if os.path.exists(oplib.LIB_PATH) else None

    def prober(host, workdir, python, ports, gpus, libs, ssh):
        assert host == "node-b.example.invalid" and gpus == [1] and ports == []        # the group's ports live on the first rank's host
        return {"libs": {"librexl3_kernels.so": here}, "ports": {}, "gpus": {"1": {"total_mib": 1000, "free_mib": 400, "compute_pids": [7]}}}
    checks = {ch.name: ch for ch in ops.preflight_remote(c, "tp2", need_mib=500, prober=prober)}
    assert checks["node-b.example.invalid:reachable"].ok and checks["node-b.example.invalid:binary"].ok == (here is not None)
    assert not checks["node-b.example.invalid:gpu1:idle"].ok and not checks["node-b.example.invalid:gpu1:memory"].ok

    def other_build(*a):
        return {"libs": {"librexl3_kernels.so": "0" * 16}, "ports": {}, "gpus": {}}
    assert not {ch.name: ch for ch in ops.preflight_remote(c, "tp2", prober=other_build)}["node-b.example.invalid:binary"].ok

    def down(*a):
        raise RuntimeError("connection refused")
    bad = ops.preflight_remote(c, "tp2", prober=down)
    assert len(bad) == 1 and not bad[0].ok and "refused" in bad[0].detail
    # the real probe through the stand-in client: this host answers about itself
    facts = remote.probe("host-y", os.getcwd(), sys.executable, [18751], [], ["rexl3_b200/ops/librexl3_kernels.so"], fake_ssh(tmp_path))
    assert facts["ports"] == {"18751": True} and "librexl3_kernels.so" in facts["libs"]
    assert ops.preflight_remote(validate({**DOC, "nodes": [{"name": "a0", "gpu": 0}, {"name": "b0", "gpu": 1}]}), "tp2") == []
