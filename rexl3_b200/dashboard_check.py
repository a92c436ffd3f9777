"""Check the dashboard's panel catalogue against what the binaries really export: every `rexl3_*` series a panel of
`dashboard/panels.json` queries must appear in the `/metrics` text of a live server (mock backend, a few requests run) or of the router.
Role of the reference's `tools/dashboard_check.py`: a renamed or dropped metric breaks this check instead of silently blanking a panel.

    python -m rexl3_b200.dashboard_check [dashboard/panels.json]        # exit status 1 when a panel names a series nobody exports
"""
from __future__ import annotations

import asyncio
import json
import os
import re
import sys

SERIES = re.compile(r"rexl3_[a-z0-9_]+")
SUFFIXES = ("", "_bucket", "_sum", "_count")


def panel_series(path: str) -> dict:
    doc = json.load(open(path))
    out = {}
    for p in doc["panels"]:
        out[p.get("title", p.get("id", "?"))] = set(SERIES.findall(json.dumps(p)))
    return out


def server_series() -> set:
    """Series names in the `/metrics` text of a mock-backend server after two chat requests (the second hits the prefix cache)."""
    from starlette.testclient import TestClient

    from .server import main
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512", "--slots", "4", "--max-model-len", "512", "--queue-depth", "8"])
    app, handle = main.make_app(args)
    try:
        if not handle.wait_ready(20):
            raise RuntimeError("the mock server did not become ready")
        with TestClient(app) as c:
            body = {"messages": [{"role": "user", "content": "the same long question, asked twice, " * 12}], "max_tokens": 8}
            c.post("/v1/chat/completions", json=body)
            c.post("/v1/chat/completions", json=body)
            text = c.get("/metrics").text
    finally:
        handle.stop()
    return {ln.split("{")[0].split(" ")[0] for ln in text.splitlines() if ln.startswith("rexl3_")}


def router_series() -> set:
    from aiohttp.test_utils import TestClient, TestServer

    from .router import Backend, Fleet
    from .router.app import Router, build_apps

    async def run():
        fleet = Fleet([Backend("a", "http://127.0.0.1:9")])
        router = Router(fleet, probe_interval_s=3600)
        app, _admin = build_apps(router)
        async with TestClient(TestServer(app)) as c:
            r = await c.get("/metrics?scope=router")
            return await r.text()
    text = asyncio.run(run())
    return {ln.split("{")[0].split(" ")[0] for ln in text.splitlines() if ln.startswith("rexl3_")}


def check(path: str, exported: set | None = None) -> dict:
    """-> {panel title: sorted series nobody exports}; empty dict = the catalogue is consistent."""
    if exported is None:
        server = server_series()
        # the router re-exports every series of its backends as rexl3_router_<name>{backend=...}
        exported = server | router_series() | {"rexl3_router_" + n[len("rexl3_"):] for n in server}
    bad = {}
    for title, names in panel_series(path).items():
        miss = sorted(n for n in names if not any(n == e or (n + s) == e or n == e + s for e in exported for s in SUFFIXES))
        if miss:
            bad[title] = miss
    return bad


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    path = argv[0] if argv else os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "dashboard", "panels.json")
    bad = check(path)
    for title, miss in bad.items():
        print(f"panel {title!r}: nobody exports {', '.join(miss)}")
    print("ok" if not bad else f"{len(bad)} panels name unexported series")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
