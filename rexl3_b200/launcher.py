"""Lifecycle verbs of a runtime recipe (what a recipe's `launch.sh` runs): one entry point per sealed version directory, the model identity
and the tuning coming only from the reviewed files in it (`profile.json`, `model.lock.json`) plus the operator's site file.  Role of the
reference's per-recipe `launch.sh` + `scripts/runtime.py` (runtimes/qwen3.8/qwen3.8-27b/v4/launch.sh: doctor, install-deps, setup,
print-command, start, status, stop, logs, verify, diagnostics, reset-state).

    python -m rexl3_b200.launcher VERB --recipe runtimes/dense/dense-27b/v1 [--site site.json] [--profile NAME] [--state-dir DIR]

    doctor         what this host offers against what the profile needs (python, torch, CUDA device count and memory through a read-only NVML
                   probe, the kernel library, free port); exits 1 when something required is missing, changes nothing
    install-deps   refused: this runtime installs nothing (no package index is assumed); prints what `doctor` found missing
    setup          verifies the sealed tree, then the model folder against `model.lock.json` (sizes; `--crc` also the checksums); a lock whose
                   source is "random-init" needs no folder
    print-command  the resolved server command and environment, nothing started
    start          setup, then the server in the foreground as a child in its own process group, pid and log path recorded in the state
                   directory, readiness polled on /health/ready; Ctrl-C stops only that process group
    status         recorded pid alive? health of the port
    stop           SIGTERM to the recorded process group (never a pattern match), then SIGKILL after a grace period
    logs           tail of the recorded log
    verify         sealed tree + lock + a live smoke request when the server is up
    diagnostics    a JSON bundle: doctor report, resolved command, state, tail of the log (no secrets: the site file's values are not copied)
    reset-state    removes the state directory's files (refused while the recorded process is alive)
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import signal
import socket
import subprocess
import sys
import time
import urllib.request

from . import recipes

VERBS = ("doctor", "install-deps", "setup", "print-command", "start", "status", "stop", "logs", "verify", "diagnostics", "reset-state")
LOCK_SCHEMA = "rexl3.model-lock.v1"


class LaunchError(RuntimeError):
    def __init__(self, code: str, message: str, exit_status: int = 2):
        super().__init__(f"{code}: {message}")
        self.code, self.exit_status = code, exit_status


# ------------------------------------------------------------------------------------------------ recipe directory
def split_recipe(vdir: str) -> tuple:
    """<root>/<family>/<model>/<version> -> (root, family, model, version)."""
    vdir = os.path.abspath(vdir)
    model_dir, version = os.path.split(vdir)
    family_dir, model = os.path.split(model_dir)
    root, family = os.path.split(family_dir)
    if not os.path.isfile(os.path.join(vdir, "profile.json")):
        raise LaunchError("NOT_A_RECIPE", f"{vdir} holds no profile.json")
    return root, family, model, version


def read_lock(vdir: str) -> dict:
    path = os.path.join(vdir, "model.lock.json")
    if not os.path.isfile(path):
        raise LaunchError("LOCK_MISSING", f"{vdir} holds no model.lock.json")
    with open(path, encoding="utf-8") as f:
        doc = json.load(f)
    if doc.get("schema") != LOCK_SCHEMA or not isinstance(doc.get("packs"), dict) or "target" not in doc["packs"]:
        raise LaunchError("LOCK_INVALID", f"{path}: not a {LOCK_SCHEMA} document with a target pack")
    return doc


def check_lock(lock: dict, model_dir: "str | None", crc: bool = False) -> list:
    """Problems of the model folder against the lock (empty: it is the reviewed pack).  A "random-init" source has no folder to check."""
    import hashlib
    problems = []
    for role, pack in lock["packs"].items():
        if pack.get("source") == "random-init":
            continue
        if not model_dir:
            problems.append(f"{role}: the lock names a pack but the site file gives no model_dir")
            continue
        folder = model_dir if role == "target" else os.path.join(model_dir, role)
        for rel, want in sorted((pack.get("files") or {}).items()):
            path = os.path.join(folder, rel)
            if not os.path.isfile(path):
                problems.append(f"{role}: missing {rel}")
                continue
            if os.path.getsize(path) != want.get("bytes"):
                problems.append(f"{role}: {rel} has {os.path.getsize(path)} bytes, the lock says {want.get('bytes')}")
                continue
            if crc:
                h = hashlib.sha256()
                with open(path, "rb") as f:
                    for chunk in iter(lambda: f.read(1 << 22), b""):
                        h.update(chunk)
                if h.hexdigest() != want.get("sha256"):
                    problems.append(f"{role}: {rel} does not have the locked sha256")
    return problems


def write_lock_for_folder(folder: str, repo: str = "", revision: str = "", license_: str = "") -> dict:
    """A lock document for an existing pack folder (sizes and sha256 of every file): what a recipe author commits after review."""
    import hashlib
    files = {}
    for name in sorted(os.listdir(folder)):
        path = os.path.join(folder, name)
        if not os.path.isfile(path):
            continue
        h = hashlib.sha256()
        with open(path, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 22), b""):
                h.update(chunk)
        files[name] = {"sha256": h.hexdigest(), "bytes": os.path.getsize(path)}
    from .format import verify as pack_verify
    try:
        fp = pack_verify.fingerprint(folder)
    except Exception:
        fp = ""
    return {"schema": LOCK_SCHEMA, "packs": {"target": {"repo": repo, "revision": revision, "fingerprint": fp, "license": license_, "files": files}}}


# ------------------------------------------------------------------------------------------------ state directory
class State:
    def __init__(self, path: str):
        self.dir = path
        self.file = os.path.join(path, "state.json")
        self.log = os.path.join(path, "server.log")

    def read(self) -> dict:
        try:
            with open(self.file, encoding="utf-8") as f:
                return json.load(f)
        except (OSError, ValueError):
            return {}

    def write(self, doc: dict) -> None:
        os.makedirs(self.dir, exist_ok=True)
        tmp = self.file + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(doc, f, indent=1, sort_keys=True)
        os.replace(tmp, self.file)

    def alive(self) -> bool:
        pid = self.read().get("pid")
        if not pid:
            return False
        try:
            os.kill(int(pid), 0)
        except (OSError, ValueError):
            return False
        # the pid may have been reused: the recorded start time of the process must match
        want = self.read().get("proc_start")
        return want is None or want == _proc_start(int(pid))


def _proc_start(pid: int):
    try:
        with open(f"/proc/{pid}/stat") as f:
            return f.read().rsplit(")", 1)[1].split()[19]
    except (OSError, IndexError):
        return None


def default_state_dir(vdir: str) -> str:
    root, family, model, version = split_recipe(vdir)
    base = os.environ.get("REXL3_STATE_DIR") or os.path.join(os.path.expanduser("~"), ".local", "state", "rexl3")
    return os.path.join(base, f"{family}-{model}-{version}")


# ------------------------------------------------------------------------------------------------ verbs
def doctor(resolved, nvml=None) -> dict:
    """-> {"ok": bool, "checks": [{name, ok, detail, required}]}.  `nvml`: a function index -> {"total_mib", "free_mib", "compute_pids"}
    that raises for a GPU that is not there (tests pass a fake; the default reads NVML and changes nothing)."""
    checks = []

    def add(name, ok, detail, required=True):
        checks.append(dict(name=name, ok=bool(ok), detail=detail, required=required))
    add("python", sys.version_info >= (3, 10), sys.version.split()[0])
    try:
        import torch
        add("torch", True, torch.__version__)
    except Exception as e:    # noqa: BLE001
        add("torch", False, f"not importable: {e}")
    from .ops import build as kbuild
    lib = os.path.join(os.path.dirname(kbuild.__file__), "librexl3_kernels.so")
    add("kernel library", os.path.isfile(lib), lib if os.path.isfile(lib) else "not built: run `python -c 'import __graft_entry__ as g; g.build()'`")
    ranks = resolved.ranks if resolved.kind == "tp" else 1
    need_gpu = "--backend" in resolved.argv and resolved.argv[resolved.argv.index("--backend") + 1] == "cuda"
    if need_gpu:
        try:
            if nvml is None:
                from .cluster.ops import nvml_probe as nvml
            seen = 0
            for i in range(ranks):
                try:
                    facts = nvml(i)
                except Exception:    # noqa: BLE001
                    break
                seen += 1
                add(f"gpu{i} memory", facts["free_mib"] >= 0.9 * facts["total_mib"] and not facts.get("compute_pids"),
                    f"{facts['free_mib']} MiB free of {facts['total_mib']}, {len(facts.get('compute_pids') or [])} compute processes", required=False)
            add("gpus", seen >= ranks, f"{seen} answered the probe, the profile needs {ranks}")
        except Exception as e:    # noqa: BLE001
            add("gpus", False, f"NVML probe failed: {e}")
    host, port = resolved.http_host, resolved.http_port
    with socket.socket() as sk:
        sk.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            sk.bind((host, port))
            add("port", True, f"{host}:{port} is free")
        except OSError as e:
            add("port", False, f"{host}:{port}: {e}")
    return dict(ok=all(c["ok"] or not c["required"] for c in checks), checks=checks)


def health(host: str, port: int, path: str = "/health/ready", timeout: float = 2.0):
    try:
        with urllib.request.urlopen(f"http://{host}:{port}{path}", timeout=timeout) as r:
            return r.status, r.read(2048).decode("utf-8", "replace")
    except urllib.error.HTTPError as e:
        return e.code, e.read(2048).decode("utf-8", "replace")
    except Exception as e:    # noqa: BLE001
        return 0, str(e)


def command_of(resolved) -> list:
    if resolved.kind == "tp":
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={resolved.ranks}", "--master-addr", "127.0.0.1",
                "--master-port", str(resolved.rendezvous_port), "-m", "rexl3_b200.server"] + resolved.argv
    return [sys.executable, "-m", "rexl3_b200.server"] + resolved.argv


def setup(vdir: str, resolved, crc: bool = False) -> None:
    problems = recipes.verify_tree(vdir)
    if problems:
        raise LaunchError("TREE_CHANGED", "the sealed recipe does not match its manifest: " + "; ".join(problems))
    lock = read_lock(vdir)
    bad = check_lock(lock, resolved.model_dir, crc=crc)
    if bad:
        raise LaunchError("PACK_MISMATCH", "; ".join(bad))


def start(vdir: str, resolved, state: State, crc: bool = False, wait: bool = True, out=sys.stdout) -> int:
    if state.alive():
        raise LaunchError("ALREADY_RUNNING", f"pid {state.read().get('pid')} recorded in {state.file} is alive; use stop first")
    setup(vdir, resolved, crc)
    os.makedirs(state.dir, exist_ok=True)
    cmd = command_of(resolved)
    log = open(state.log, "ab")
    proc = subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, env={**os.environ, **resolved.env}, start_new_session=True)
    host, port = resolved.http_host, resolved.http_port
    state.write(dict(pid=proc.pid, proc_start=_proc_start(proc.pid), started=time.time(), command=cmd, host=host, port=port, log=state.log,
                     runtime_id=resolved.runtime_id, profile=resolved.profile))
    print(f"started pid {proc.pid}; log {state.log}", file=out)
    if not wait:
        return 0
    deadline = time.time() + float(resolved.readiness_timeout_s)
    try:
        while time.time() < deadline:
            rc = proc.poll()
            if rc is not None:
                raise LaunchError("SERVER_EXITED", f"the server exited with status {rc} before it was ready; see {state.log}", 1)
            code, _ = health(host, port)
            if code == 200:
                print(f"ready on http://{host}:{port}", file=out)
                break
            time.sleep(0.5)
        else:
            raise LaunchError("NOT_READY", f"not ready after {resolved.readiness_timeout_s} s; see {state.log}", 1)
        return proc.wait()
    except KeyboardInterrupt:
        stop(state, out=out)
        return 130
    except LaunchError:
        stop(state, out=out)
        raise


def stop(state: State, grace_s: float = 15.0, out=sys.stdout) -> bool:
    doc = state.read()
    if not state.alive():
        print("not running", file=out)
        return False
    pid = int(doc["pid"])
    try:
        os.killpg(pid, signal.SIGTERM)          # the server was started as the leader of its own process group
    except OSError:
        os.kill(pid, signal.SIGTERM)
    t0 = time.time()
    while time.time() - t0 < grace_s and state.alive():
        try:
            os.waitpid(pid, os.WNOHANG)
        except OSError:
            pass
        time.sleep(0.1)
    if state.alive():
        try:
            os.killpg(pid, signal.SIGKILL)
        except OSError:
            pass
    print(f"stopped pid {pid}", file=out)
    return True


def tail(path: str, lines: int = 80) -> str:
    try:
        with open(path, "rb") as f:
            f.seek(0, os.SEEK_END)
            size = f.tell()
            f.seek(max(0, size - 65536))
            return b"\n".join(f.read().splitlines()[-lines:]).decode("utf-8", "replace")
    except OSError:
        return ""


def main(argv=None, out=sys.stdout, nvml=None) -> int:
    p = argparse.ArgumentParser(prog="rexl3-launch", allow_abbrev=False, description="lifecycle verbs of a runtime recipe")
    p.add_argument("verb", choices=VERBS)
    p.add_argument("--recipe", required=True, help="the recipe's version directory")
    p.add_argument("--site", help="JSON file of site fields (model_dir, http_host, http_port, ...)")
    p.add_argument("--profile")
    p.add_argument("--state-dir")
    p.add_argument("--crc", action="store_true", help="setup / verify also hash every locked file")
    p.add_argument("--no-wait", action="store_true", help="start: do not stay in the foreground")
    p.add_argument("--lines", type=int, default=80)
    a = p.parse_args(argv)
    try:
        root, family, model, version = split_recipe(a.recipe)
        state = State(a.state_dir or default_state_dir(a.recipe))
        if a.verb == "install-deps":
            print("install-deps: refused. This runtime installs nothing (no package index is assumed); `doctor` lists what is missing.", file=out)
            return 2
        if a.verb == "status":
            doc = state.read()
            up = state.alive()
            code, body = health(doc.get("host", "127.0.0.1"), int(doc.get("port", 8000)), "/health") if up else (0, "")
            print(json.dumps(dict(running=up, pid=doc.get("pid") if up else None, health=code, profile=doc.get("profile"), runtime_id=doc.get("runtime_id"))), file=out)
            return 0 if up else 3
        if a.verb == "stop":
            return 0 if stop(state, out=out) else 3
        if a.verb == "logs":
            print(tail(state.log, a.lines), file=out)
            return 0
        if a.verb == "reset-state":
            if state.alive():
                raise LaunchError("STILL_RUNNING", "stop the server before resetting its state")
            for path in (state.file, state.log):
                if os.path.isfile(path):
                    os.remove(path)
            print(f"state of {family}/{model}/{version} removed", file=out)
            return 0
        site = {}
        if a.site:
            with open(a.site, encoding="utf-8") as f:
                site = json.load(f)
        try:
            resolved = recipes.resolve(root, family, model, site, version, a.profile)
        except recipes.RecipeError as e:
            raise LaunchError("RECIPE", str(e))
        if a.verb == "print-command":
            env = " ".join(f"{k}={shlex.quote(v)}" for k, v in sorted(resolved.env.items()))
            print((env + " " if env else "") + " ".join(shlex.quote(c) for c in command_of(resolved)), file=out)
            return 0
        if a.verb == "doctor":
            rep = doctor(resolved, nvml)
            for c in rep["checks"]:
                print(f"{'ok  ' if c['ok'] else ('FAIL' if c['required'] else 'warn')} {c['name']}: {c['detail']}", file=out)
            return 0 if rep["ok"] else 1
        if a.verb == "setup":
            setup(a.recipe, resolved, a.crc)
            print("sealed tree intact; model folder matches the lock", file=out)
            return 0
        if a.verb == "verify":
            setup(a.recipe, resolved, a.crc)
            doc = state.read()
            if state.alive() and resolved.smoke_request:
                req = urllib.request.Request(f"http://{doc['host']}:{doc['port']}/v1/chat/completions", data=json.dumps(resolved.smoke_request).encode(),
                                             headers={"Content-Type": "application/json"})
                with urllib.request.urlopen(req, timeout=120) as r:
                    reply = json.load(r)
                text = reply["choices"][0]["message"].get("content", "")
                print(f"smoke request answered ({reply['usage']['completion_tokens']} tokens): {text[:60]!r}", file=out)
            print("verified", file=out)
            return 0
        if a.verb == "diagnostics":
            bundle = dict(recipe=f"{family}/{model}/{version}", doctor=doctor(resolved, nvml), command=command_of(resolved), env=sorted(resolved.env),
                          state={k: v for k, v in state.read().items() if k != "command"}, running=state.alive(), log_tail=tail(state.log, a.lines),
                          tree_problems=recipes.verify_tree(a.recipe))
            print(json.dumps(bundle, indent=1), file=out)
            return 0
        if a.verb == "start":
            return start(a.recipe, resolved, state, a.crc, wait=not a.no_wait, out=out)
    except LaunchError as e:
        print(f"rexl3-launch: {e}", file=sys.stderr)
        return e.exit_status
    return 2


if __name__ == "__main__":
    sys.exit(main())
