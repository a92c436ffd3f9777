"""python -m rexl3_b200.cluster COMMAND --cluster FILE [--group NAME] [--dry-run]      (validate | plan | up | supervise)"""
import argparse
import json
import shlex
import sys
import urllib.request

from .schema import ClusterError, load_cluster, rank_commands
from .supervise import LocalRunner, Policy, supervise


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="rexl3-cluster", allow_abbrev=False)
    p.add_argument("command", choices=["validate", "plan", "up", "supervise"])
    p.add_argument("--cluster", required=True)
    p.add_argument("--group", default="")
    p.add_argument("--dry-run", action="store_true")
    p.add_argument("--log-dir", default="")
    p.add_argument("--max-runtime", type=float, default=0.0)
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
    cmds = rank_commands(c, group, sys.executable)
    if a.command == "plan" or a.dry_run:
        for r, (env, argv_) in enumerate(cmds):
            print(f"rank {r}: " + " ".join(f"{k}={shlex.quote(v)}" for k, v in env.items()) + " " + " ".join(shlex.quote(x) for x in argv_))
        return 0
    port = c.groups[group].http_port

    def ready():
        try:
            return urllib.request.urlopen(f"http://127.0.0.1:{port}/health/ready", timeout=1).status == 200
        except Exception:
            return False
    runner = LocalRunner(cmds, ready, a.log_dir, a.max_runtime)
    if a.command == "up":
        att = runner()
        return 0 if all(c_ == 0 for c_ in att.codes if c_ is not None) else 1
    sup = c.supervisor
    return supervise(runner, Policy(sup.get("backoff_s", Policy().backoff_s), sup.get("window_s", 600.0), sup.get("max_failures", 5)))


if __name__ == "__main__":
    sys.exit(main())
