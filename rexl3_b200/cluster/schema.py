"""The cluster file: nodes (here: GPUs of one NVLink box, or hosts), the serve flags, and groups of ranks.  Validation is offline and
strict (unknown keys, ranks naming unknown nodes, a node in two groups, port clashes are errors), as in the reference's
`rexl3-cluster validate` (crates/cluster/src/schema.rs, main.rs:17-45; example docs/examples/cluster.dp-fleet.json).

{
  "schema_version": 1, "name": "b200-box",
  "nodes": [{"name": "g0", "gpu": 0}, ...],                     # "address": the rank runs on that host through an ssh client
  "pack": "/models/x", "serve": {"flags": ["--slots", "64"]},
  "groups": [{"name": "tp8", "ranks": ["g0", ..., "g7"], "tp_port": 29600, "http_port": 8080}],
  "supervisor": {"backoff_s": [1, 2, 5, 15], "window_s": 600, "max_failures": 5}
}
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

TOP = {"schema_version", "name", "nodes", "pack", "serve", "groups", "supervisor", "user", "binary", "nccl", "memory", "_comment", "random_init"}
NODE = {"name", "gpu", "address", "number"}
GROUP = {"name", "ranks", "tp_port", "http_port", "flags", "_comment"}
SUP = {"backoff_s", "window_s", "max_failures", "ready_timeout_s"}


class ClusterError(ValueError):
    pass


@dataclass
class Group:
    name: str
    ranks: list
    tp_port: int
    http_port: int
    flags: list = field(default_factory=list)


@dataclass
class Cluster:
    name: str
    nodes: dict
    groups: dict
    pack: str = ""
    random_init: str = ""
    flags: list = field(default_factory=list)
    supervisor: dict = field(default_factory=dict)


def validate(doc: dict) -> Cluster:
    if not isinstance(doc, dict):
        raise ClusterError("the cluster file must be a JSON object")
    unknown = set(doc) - TOP
    if unknown:
        raise ClusterError(f"unknown keys: {sorted(unknown)}")
    if doc.get("schema_version") != 1:
        raise ClusterError("schema_version must be 1")
    nodes = {}
    for n in doc.get("nodes") or []:
        if set(n) - NODE or "name" not in n:
            raise ClusterError(f"bad node entry {n!r}")
        if n["name"] in nodes:
            raise ClusterError(f"node {n['name']!r} is listed twice")
        nodes[n["name"]] = n
    if not nodes:
        raise ClusterError("no nodes")
    groups, used, ports = {}, {}, set()
    for g in doc.get("groups") or []:
        if set(g) - GROUP or not {"name", "ranks", "tp_port", "http_port"} <= set(g):
            raise ClusterError(f"bad group entry {g!r}")
        if g["name"] in groups:
            raise ClusterError(f"group {g['name']!r} is listed twice")
        if not g["ranks"] or len(g["ranks"]) not in (1, 2, 4, 8):
            raise ClusterError(f"group {g['name']!r}: 1, 2, 4 or 8 ranks")
        for r in g["ranks"]:
            if r not in nodes:
                raise ClusterError(f"group {g['name']!r} names unknown node {r!r}")
            if r in used:
                raise ClusterError(f"node {r!r} is in groups {used[r]!r} and {g['name']!r}: one model per node")
            used[r] = g["name"]
        for p in (g["tp_port"], g["http_port"]):
            if not isinstance(p, int) or not 1024 <= p <= 65535:
                raise ClusterError(f"group {g['name']!r}: port {p!r} out of range")
        host = nodes[g["ranks"][0]].get("address", "127.0.0.1")
        for p in (g["tp_port"], g["http_port"]):
            if (host, p) in ports:
                raise ClusterError(f"port {p} on {host} is used twice")
            ports.add((host, p))
        groups[g["name"]] = Group(g["name"], list(g["ranks"]), g["tp_port"], g["http_port"], list(g.get("flags", [])))
    if not groups:
        raise ClusterError("no groups")
    sup = doc.get("supervisor") or {}
    if set(sup) - SUP:
        raise ClusterError(f"unknown supervisor keys: {sorted(set(sup) - SUP)}")
    if not doc.get("pack") and not doc.get("random_init"):
        raise ClusterError("pack (or random_init) is required")
    flags = list((doc.get("serve") or {}).get("flags", []))
    return Cluster(doc.get("name", "cluster"), nodes, groups, doc.get("pack", ""), doc.get("random_init", ""), flags, sup)


def load_cluster(path: str) -> Cluster:
    with open(path) as f:
        try:
            return validate(json.load(f))
        except json.JSONDecodeError as e:
            raise ClusterError(f"{path}: {e}") from e


def rank_commands(c: Cluster, group: str, python: str = "python", ssh: str = "", workdir: str = "") -> list:
    """One (env, argv) per rank: the serving binary under the lockstep environment of the group.  A rank whose node has an `address` that is
    not this host is wrapped into an ssh client command (`cluster.remote.wrap`; `workdir` = the repository's path on that host, default: the
    same path as here)."""
    g = c.groups[group]
    out = []
    R = len(g.ranks)
    for r, node in enumerate(g.ranks):
        n = c.nodes[node]
        env = {"RANK": str(r), "WORLD_SIZE": str(R), "LOCAL_RANK": str(n.get("gpu", r)), "MASTER_ADDR": c.nodes[g.ranks[0]].get("address", "127.0.0.1"),
               "MASTER_PORT": str(g.tp_port), "NCCL_NVLS_ENABLE": "0"}
        if R == 1:
            # a replica of its own: the process sees only its GPU (the serving binary uses the current device when it is not part of a group)
            env["CUDA_VISIBLE_DEVICES"] = str(n.get("gpu", 0))
            env["LOCAL_RANK"] = "0"
        argv = [python, "-m", "rexl3_b200.server", "--backend", "cuda", "--port", str(g.http_port)]
        argv += ["--model", c.pack] if c.pack else ["--random-init", c.random_init]
        argv += c.flags + g.flags
        from . import remote
        if not remote.is_local(n.get("address")):
            import os
            rpy = python if python != os.sys.executable else "python3"      # this host's interpreter path means nothing over there
            env, argv = remote.wrap(env, [rpy] + argv[1:], n["address"], workdir or os.getcwd(), ssh)
        out.append((env, argv))
    return out
