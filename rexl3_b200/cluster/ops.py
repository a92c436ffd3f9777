"""Group operations around the supervisor: pre-flight checks, GPU lock files, the state file of a running group, status, down, logs.
Parity: the reference's `rexl3-cluster` check / up / down / status / logs (crates/cluster/src/check.rs, ops.rs), for the GPUs of one
NVLink box, or several hosts (ranks on this host are child processes; ranks on other hosts are ssh client children, `cluster.remote`).

Pre-flight facts per group: the kernel and host libraries exist and every rank would load the same bytes (sha256), the pack is present
and has one identity (structure fingerprint), the group's ports are free, each GPU has the memory the plan needs and runs no other
compute process, no other group holds a GPU's lock.  GPU facts come from a probe (NVML, read-only) that tests replace with a fake.
"""
from __future__ import annotations

import hashlib
import json
import os
import signal
import socket
import time
from dataclasses import dataclass

from .schema import Cluster


@dataclass
class Check:
    name: str
    ok: bool
    detail: str = ""


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(8 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def port_is_free(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return True
        except OSError:
            return False


def nvml_probe(index: int) -> dict:
    """Read-only facts of one GPU: {"total_mib", "free_mib", "compute_pids"} (raises when NVML is not available)."""
    import pynvml
    pynvml.nvmlInit()
    try:
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        mem = pynvml.nvmlDeviceGetMemoryInfo(h)
        pids = [p.pid for p in pynvml.nvmlDeviceGetComputeRunningProcesses(h)]
        return {"total_mib": mem.total >> 20, "free_mib": mem.free >> 20, "compute_pids": pids}
    finally:
        pynvml.nvmlShutdown()


def preflight(c: Cluster, group: str, *, need_mib: int = 0, gpu_probe=None, port_free=port_is_free, locks: "GpuLocks | None" = None,
              libraries=None) -> list:
    g = c.groups[group]
    out = []
    if libraries is None:
        from ..native import build as nbuild
        from ..ops import lib as oplib
        libraries = [oplib.LIB_PATH, nbuild.OUT]
    for path in libraries:
        if os.path.exists(path):
            out.append(Check(f"binary:{os.path.basename(path)}", True, _sha256(path)[:16]))
        else:
            out.append(Check(f"binary:{os.path.basename(path)}", False, "missing: build it first"))
    if c.pack:
        try:
            from ..format import verify
            out.append(Check("pack", True, f"fingerprint {verify.fingerprint(c.pack)[:16]}"))
        except (OSError, ValueError) as e:
            out.append(Check("pack", False, str(e)))
    else:
        out.append(Check("pack", True, f"random-init {c.random_init}"))
    for what, port in (("tp_port", g.tp_port), ("http_port", g.http_port)):
        free = port_free(port)
        out.append(Check(what, free, f"{port} " + ("free" if free else "in use")))
    for node in g.ranks:
        idx = c.nodes[node].get("gpu", g.ranks.index(node))
        if locks is not None:
            holder = locks.holder(idx)
            out.append(Check(f"lock:gpu{idx}", holder is None or holder.get("group") == group, "free" if holder is None else f"held by {holder}"))
        if gpu_probe is None:
            continue
        try:
            f = gpu_probe(idx)
        except Exception as e:  # noqa: BLE001  (any probe failure is a failed check, not a crash)
            out.append(Check(f"gpu{idx}", False, f"probe failed: {e}"))
            continue
        idle = not f.get("compute_pids")
        out.append(Check(f"gpu{idx}:idle", idle, "no compute process" if idle else f"busy: pids {f['compute_pids']}"))
        if need_mib:
            out.append(Check(f"gpu{idx}:memory", f["free_mib"] >= need_mib, f"{f['free_mib']} MiB free, {need_mib} needed"))
    return out


def preflight_remote(c: Cluster, group: str, *, need_mib: int = 0, ssh: str = "", workdir: str = "", probe_gpus: bool = True, python: str = "python3",
                     prober=None) -> list:
    """The same facts for the ranks of the group that live on other hosts, read through one ssh command per host (`cluster.remote.probe`):
    the kernel library there must have the hash of the one here (ranks of one group must run one build), the group's ports must be free on
    the first rank's host, every GPU idle with `need_mib` free.  `prober`: stand-in for `remote.probe` in tests."""
    from . import remote
    g = c.groups[group]
    out, by_host = [], {}
    for i, node in enumerate(g.ranks):
        n = c.nodes[node]
        if not remote.is_local(n.get("address")):
            by_host.setdefault(n["address"], []).append((i, n.get("gpu", i)))
    if not by_host:
        return out
    from ..ops import lib as oplib
    here = _sha256(oplib.LIB_PATH)[:16] if os.path.exists(oplib.LIB_PATH) else None
    rel = os.path.relpath(oplib.LIB_PATH, os.getcwd()) if os.path.exists(oplib.LIB_PATH) else "rexl3_b200/ops/librexl3_kernels.so"
    first_host = c.nodes[g.ranks[0]].get("address")
    for host, ranks in sorted(by_host.items()):
        ports = [g.tp_port, g.http_port] if host == first_host else []
        try:
            facts = (prober or remote.probe)(host, workdir, python, ports, [gpu for _, gpu in ranks] if probe_gpus else [], [rel], ssh)
        except Exception as e:  # noqa: BLE001
            out.append(Check(f"{host}:reachable", False, str(e)))
            continue
        out.append(Check(f"{host}:reachable", True, "answered the probe"))
        there = next(iter(facts.get("libs", {}).values()), None)
        out.append(Check(f"{host}:binary", there is not None and there == here, f"{there} there, {here} here"))
        for port, free in facts.get("ports", {}).items():
            out.append(Check(f"{host}:port{port}", bool(free), "free" if free else "in use"))
        for gpu, f in facts.get("gpus", {}).items():
            if "error" in f:
                out.append(Check(f"{host}:gpu{gpu}", False, f"probe failed: {f['error']}"))
                continue
            idle = not f.get("compute_pids")
            out.append(Check(f"{host}:gpu{gpu}:idle", idle, "no compute process" if idle else f"busy: pids {f['compute_pids']}"))
            if need_mib:
                out.append(Check(f"{host}:gpu{gpu}:memory", f["free_mib"] >= need_mib, f"{f['free_mib']} MiB free, {need_mib} needed"))
    return out


class GpuLocks:
    """One lock file per GPU index: {"group", "pid", "time"}.  A lock whose pid is gone is stale and may be taken."""

    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)

    def _path(self, idx: int) -> str:
        return os.path.join(self.dir, f"gpu{idx}.lock")

    def holder(self, idx: int):
        try:
            h = json.load(open(self._path(idx)))
        except (OSError, ValueError):
            return None
        return h if _alive(h.get("pid", -1)) else None

    def acquire(self, indices, group: str, pid: int | None = None) -> bool:
        """All or nothing.  False when another live group holds one of the GPUs."""
        pid = pid or os.getpid()
        for i in indices:
            h = self.holder(i)
            if h is not None and (h.get("group") != group or h.get("pid") != pid):
                return False
        for i in indices:
            tmp = self._path(i) + f".{pid}.tmp"
            json.dump({"group": group, "pid": pid, "time": time.time()}, open(tmp, "w"))
            os.replace(tmp, self._path(i))
        return True

    def release(self, indices, group: str) -> None:
        for i in indices:
            try:
                h = json.load(open(self._path(i)))
            except (OSError, ValueError):
                continue
            if h.get("group") == group:
                try:
                    os.remove(self._path(i))
                except OSError:
                    pass


def _alive(pid: int) -> bool:
    if pid <= 0:
        return False
    try:
        os.kill(pid, 0)
        return True
    except ProcessLookupError:
        return False
    except PermissionError:
        return True


def _is_ours(pid: int, marker: str = "rexl3_b200") -> bool:
    """The process is alive and its command line names this package (a recycled pid of something else is never signalled)."""
    try:
        with open(f"/proc/{pid}/cmdline", "rb") as f:
            return marker.encode() in f.read()
    except OSError:
        return False


def state_path(state_dir: str, group: str) -> str:
    return os.path.join(state_dir, f"{group}.state.json")


def write_state(state_dir: str, group: str, supervisor_pid: int, rank_pids: list, http_port: int, log_dir: str = "") -> None:
    os.makedirs(state_dir, exist_ok=True)
    tmp = state_path(state_dir, group) + ".tmp"
    json.dump({"group": group, "supervisor_pid": supervisor_pid, "rank_pids": list(rank_pids), "http_port": http_port, "log_dir": log_dir,
               "time": time.time()}, open(tmp, "w"))
    os.replace(tmp, state_path(state_dir, group))


def read_state(state_dir: str, group: str):
    try:
        return json.load(open(state_path(state_dir, group)))
    except (OSError, ValueError):
        return None


def status(state_dir: str, group: str, ready_probe=None) -> dict:
    st = read_state(state_dir, group)
    if st is None:
        return {"group": group, "state": "down"}
    ranks = [{"rank": r, "pid": pid, "alive": _alive(pid)} for r, pid in enumerate(st.get("rank_pids", []))]
    up = all(r["alive"] for r in ranks) and bool(ranks)
    ready = bool(ready_probe(st["http_port"])) if (up and ready_probe is not None) else None
    return {"group": group, "state": "up" if up else ("partial" if any(r["alive"] for r in ranks) else "down"), "ready": ready,
            "supervisor_alive": _alive(st.get("supervisor_pid", -1)), "ranks": ranks, "http_port": st["http_port"]}


def down(state_dir: str, group: str, locks: GpuLocks | None = None, gpu_indices=(), grace_s: float = 15.0, marker: str = "rexl3_b200") -> list:
    """Stop the group recorded in the state file: the supervisor first (so it does not restart the ranks), then rank 0, then the rest, each
    by its recorded pid and only while that pid still runs this package.  Returns the pids that were signalled."""
    st = read_state(state_dir, group)
    hit = []
    if st is not None:
        order = [st.get("supervisor_pid", -1)] + list(st.get("rank_pids", []))
        for pid in order:
            if pid > 0 and pid != os.getpid() and _alive(pid) and _is_ours(pid, marker):
                os.kill(pid, signal.SIGTERM)
                hit.append(pid)
        t = time.monotonic() + grace_s
        while time.monotonic() < t and any(_alive(p) and _is_ours(p, marker) for p in hit):
            time.sleep(0.1)
        for pid in hit:
            if _alive(pid) and _is_ours(pid, marker):
                os.kill(pid, signal.SIGKILL)
        try:
            os.remove(state_path(state_dir, group))
        except OSError:
            pass
    if locks is not None:
        locks.release(gpu_indices, group)
    return hit


def tail_logs(log_dir: str, ranks: int, lines: int = 40) -> dict:
    out = {}
    for r in range(ranks):
        p = os.path.join(log_dir, f"rank{r}.log")
        try:
            with open(p, "rb") as f:
                f.seek(0, os.SEEK_END)
                n = f.tell()
                f.seek(max(0, n - 64 * 1024))
                out[r] = f.read().decode("utf-8", "replace").splitlines()[-lines:]
        except OSError:
            out[r] = None
    return out
