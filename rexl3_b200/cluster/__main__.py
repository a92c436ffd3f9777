"""python -m rexl3_b200.cluster COMMAND --cluster FILE [--group NAME]
   validate | plan | check | up | supervise | status | down | logs          (--dry-run prints the plan instead of starting anything)"""
import argparse
import json
import os
import shlex
import sys
import urllib.request

from . import ops
from .schema import ClusterError, load_cluster, rank_commands
from .supervise import LocalRunner, Policy, supervise


def _ready(port: int) -> bool:
    try:
        return urllib.request.urlopen(f"http://127.0.0.1:{port}/health/ready", timeout=1).status == 200
    except Exception:  # noqa: BLE001
        return False


def _planned_mib(c, g) -> int:
    """Memory each GPU of the group needs according to the memory plan of the cluster file's model and serve flags (0: unknown model)."""
    from .. import plan
    flags = list(c.flags) + list(g.flags)

    def opt(name, default):
        return int(flags[flags.index(name) + 1]) if name in flags and flags.index(name) + 1 < len(flags) else default
    try:
        if c.random_init:
            cfg = plan.find_config(c.random_init)
        else:
            from ..quant import quantize
            cfg = quantize.config_from_pack(c.pack)
    except (KeyError, OSError, ValueError):
        return 0
    d = plan.plan(cfg, gpus=len(g.ranks), slots=opt("--slots", 16), max_model_len=opt("--max-model-len", 8192),
                  kv_dtype="fp8" if "fp8" in flags else "bf16")
    per = d["per_gpu"]
    kv = per["kv_for_all_slots"]
    if "--kv-tokens" in flags:
        kv = opt("--kv-tokens", 0) * max(1, d["kv_bytes_per_token"] // len(g.ranks))
    return int((per["weights"] + per["recurrent_state"] + per["reserve"] + kv) >> 20)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="rexl3-cluster", allow_abbrev=False)
    p.add_argument("command", choices=["validate", "plan", "check", "up", "supervise", "status", "down", "logs"])
    p.add_argument("--cluster", required=True)
    p.add_argument("--group", default="")
    p.add_argument("--dry-run", action="store_true")
    p.add_argument("--log-dir", default="")
    p.add_argument("--state-dir", default=".rexl3-cluster", help="state files and GPU locks of the groups started from here")
    p.add_argument("--need-mib", type=int, default=0, help="check: free memory every GPU of the group must have")
    p.add_argument("--no-gpu-probe", action="store_true", help="check: skip the NVML facts (memory, idle)")
    p.add_argument("--lines", type=int, default=40)
    p.add_argument("--max-runtime", type=float, default=0.0)
    p.add_argument("--ssh", default="", help="ssh client for ranks on other hosts (default: $REXL3_SSH or ssh)")
    p.add_argument("--remote-workdir", default="", help="path of this repository on the other hosts (default: the same path as here)")
    a = p.parse_args(argv)
    try:
        c = load_cluster(a.cluster)
    except (ClusterError, OSError) as e:
        print(f"rexl3-cluster: {e}", file=sys.stderr)
        return 2
    if a.command == "validate":
        print(json.dumps({"name": c.name, "groups": {g.name: g.ranks for g in c.groups.values()}}))
        return 0
    group = a.group or (next(iter(c.groups)) if len(c.groups) == 1 else "")
    if group not in c.groups:
        print("rexl3-cluster: --group NAME is required (the file has several groups)", file=sys.stderr)
        return 2
    g = c.groups[group]
    gpus = [c.nodes[n].get("gpu", i) for i, n in enumerate(g.ranks)]
    locks = ops.GpuLocks(os.path.join(a.state_dir, "locks"))
    if a.command == "status":
        print(json.dumps(ops.status(a.state_dir, group, _ready)))
        return 0
    if a.command == "down":
        hit = ops.down(a.state_dir, group, locks, gpus)
        print(json.dumps({"group": group, "signalled": hit}))
        return 0
    if a.command == "logs":
        st = ops.read_state(a.state_dir, group) or {}
        log_dir = a.log_dir or st.get("log_dir", "")
        if not log_dir:
            print("rexl3-cluster: no log directory is known for this group (--log-dir)", file=sys.stderr)
            return 2
        for r, lines in ops.tail_logs(log_dir, len(g.ranks), a.lines).items():
            print(f"==> rank {r} <==")
            print("\n".join(lines) if lines is not None else "(no log)")
        return 0
    if a.command == "check":
        need = a.need_mib or _planned_mib(c, g)
        checks = ops.preflight(c, group, need_mib=need, gpu_probe=None if a.no_gpu_probe else ops.nvml_probe, locks=locks)
        checks += ops.preflight_remote(c, group, need_mib=need, ssh=a.ssh, workdir=a.remote_workdir or os.getcwd(), probe_gpus=not a.no_gpu_probe)
        for ch in checks:
            print(f"{'ok  ' if ch.ok else 'FAIL'} {ch.name}: {ch.detail}")
        return 0 if all(ch.ok for ch in checks) else 1
    cmds = rank_commands(c, group, sys.executable, a.ssh, a.remote_workdir)
    if a.command == "plan" or a.dry_run:
        for r, (env, argv_) in enumerate(cmds):
            print(f"rank {r}: " + " ".join(f"{k}={shlex.quote(v)}" for k, v in env.items()) + " " + " ".join(shlex.quote(x) for x in argv_))
        return 0
    if not locks.acquire(gpus, group):
        print(f"rexl3-cluster: a GPU of group {group} is locked by another group (see {locks.dir})", file=sys.stderr)
        return 75
    if a.log_dir:
        os.makedirs(a.log_dir, exist_ok=True)
    runner = LocalRunner(cmds, lambda: _ready(g.http_port), a.log_dir, a.max_runtime,
                         on_start=lambda pids: ops.write_state(a.state_dir, group, os.getpid(), pids, g.http_port, a.log_dir))
    try:
        if a.command == "up":
            att = runner()
            return 0 if all(c_ == 0 for c_ in att.codes if c_ is not None) else 1
        sup = c.supervisor
        return supervise(runner, Policy(sup.get("backoff_s", Policy().backoff_s), sup.get("window_s", 600.0), sup.get("max_failures", 5)))
    finally:
        locks.release(gpus, group)
        try:
            os.remove(ops.state_path(a.state_dir, group))
        except OSError:
            pass


if __name__ == "__main__":
    sys.exit(main())
