"""Ranks on other hosts: how a group's per-rank command is carried over ssh, and the facts a pre-flight check reads there.

A node with an `address` that is not this host is driven through an ssh client: the rank's command becomes
`ssh -tt -o BatchMode=yes ADDRESS -- cd WORKDIR && exec env K=V ... ARGV`.  `-tt` gives the remote process a terminal that goes away with the
client, so ending the local ssh child (which the runner does by recorded pid, as for local ranks) hangs up the remote rank; nothing is ever
looked up by name on the remote side.  The client binary is a parameter (`--ssh`, `REXL3_SSH`): the tests pass a stand-in that runs the
command on this host.  Role of the reference's multi-node launch in `crates/cluster` (`rexl3-cluster up` over its node list).
"""
from __future__ import annotations

import json
import os
import shlex
import socket
import subprocess

LOCAL = {"", "127.0.0.1", "localhost", "::1"}


def is_local(address) -> bool:
    if address is None or address in LOCAL:
        return True
    try:
        return address in (socket.gethostname(), socket.getfqdn())
    except OSError:
        return False


def ssh_binary(override: str = "") -> str:
    return override or os.environ.get("REXL3_SSH", "ssh")


def wrap(env: dict, argv: list, address: str, workdir: str, ssh: str = "", options=("-o", "BatchMode=yes", "-o", "ConnectTimeout=10")) -> tuple:
    """(env for the local child, argv of the ssh client) that runs `argv` under `env` in `workdir` on `address`."""
    assign = " ".join(f"{k}={shlex.quote(str(v))}" for k, v in sorted(env.items()))
    remote = f"cd {shlex.quote(workdir)} && exec env {assign} " + " ".join(shlex.quote(a) for a in argv)
    return {}, [ssh_binary(ssh), "-tt", *options, address, "--", remote]


def probe_command(python: str, ports: list, gpus: list, libraries: list) -> list:
    """argv (to run on the remote host) that prints one JSON line of facts: library hashes, free ports, read-only GPU facts."""
    code = ("import json,sys;from rexl3_b200.cluster import ops;"
            "a=json.loads(sys.argv[1]);out={'ports':{str(p):ops.port_is_free(p) for p in a['ports']},'libs':{},'gpus':{}}\n"
            "import os\n"
            "for l in a['libs']:\n out['libs'][os.path.basename(l)]=ops._sha256(l)[:16] if os.path.exists(l) else None\n"
            "for g in a['gpus']:\n"
            " try: out['gpus'][str(g)]=ops.nvml_probe(g)\n"
            " except Exception as e: out['gpus'][str(g)]={'error':str(e)}\n"
            "print(json.dumps(out))")
    return [python, "-c", code, json.dumps({"ports": ports, "gpus": gpus, "libs": libraries})]


def probe(address: str, workdir: str, python: str, ports: list, gpus: list, libraries: list, ssh: str = "", timeout_s: float = 60.0) -> dict:
    """Facts of a remote node for the pre-flight check; raises RuntimeError when the host cannot be reached or answers garbage."""
    _, argv = wrap({}, probe_command(python, ports, gpus, libraries), address, workdir, ssh)
    argv = [a for a in argv if a != "-tt"]                         # no terminal for a one-shot command: its output must stay clean
    r = subprocess.run(argv, capture_output=True, text=True, timeout=timeout_s)
    if r.returncode != 0:
        raise RuntimeError(f"{address}: exit status {r.returncode}: {r.stderr.strip()[-200:]}")
    try:
        return json.loads(r.stdout.strip().splitlines()[-1])
    except (ValueError, IndexError):
        raise RuntimeError(f"{address}: the probe did not answer with JSON: {r.stdout[-200:]!r}")
