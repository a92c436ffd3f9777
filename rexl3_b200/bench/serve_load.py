"""Continuous-batching load test through the HTTP API: N concurrent streaming `/v1/completions` requests with prompt lengths drawn
log-uniformly from [min, max] tokens, against a server this script starts (random-init model, byte tokenizer: one character is one
token) or one that is already running (`--url`).  Reports p50 / p90 time to first token and aggregate decode tokens/s.

    python -m rexl3_b200.bench.serve_load --streams 32 --min-prompt 1024 --max-prompt 32768 --max-tokens 128 --kv-dtype fp8
    python -m rexl3_b200.bench.serve_load --backend mock --streams 8 --max-prompt 2048        # plumbing check without a GPU
"""
from __future__ import annotations

import argparse
import asyncio
import json
import math
import os
import random
import signal
import statistics
import subprocess
import sys
import time


async def one(session, url, model, prompt, max_tokens, out):
    t0 = time.perf_counter()
    first = None
    n = 0
    body = {"model": model, "prompt": prompt, "max_tokens": max_tokens, "stream": True, "temperature": 0}
    async with session.post(url + "/v1/completions", json=body) as r:
        if r.status != 200:
            out.append(dict(error=r.status, text=(await r.text())[:200]))
            return
        async for raw in r.content:
            line = raw.decode("utf-8", "replace").strip()
            if not line.startswith("data:") or line == "data: [DONE]":
                continue
            try:
                doc = json.loads(line[5:])
            except ValueError:
                continue
            if doc.get("choices") and doc["choices"][0].get("text"):
                if first is None:
                    first = time.perf_counter() - t0
                n += 1
            if doc.get("usage"):
                n = doc["usage"].get("completion_tokens", n)
    out.append(dict(ttft=first, tokens=n, total=time.perf_counter() - t0, prompt=len(prompt)))


async def run(url, model, prompts, max_tokens):
    import aiohttp
    out = []
    t0 = time.perf_counter()
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=3600)) as s:
        await asyncio.gather(*(one(s, url, model, p, max_tokens, out) for p in prompts))
    return out, time.perf_counter() - t0


def wait_ready(url, timeout_s):
    import urllib.request
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        try:
            if urllib.request.urlopen(url + "/health/ready", timeout=2).status == 200:
                return True
        except Exception:
            time.sleep(1.0)
    return False


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="")
    ap.add_argument("--backend", default="cuda", choices=["cuda", "mock"])
    ap.add_argument("--model", default="dense-27b")
    ap.add_argument("--streams", type=int, default=32)
    ap.add_argument("--min-prompt", type=int, default=1024)
    ap.add_argument("--max-prompt", type=int, default=32768)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--kv-dtype", default="fp8")
    ap.add_argument("--port", type=int, default=8437)
    ap.add_argument("--seed", type=int, default=1)
    a = ap.parse_args()
    rng = random.Random(a.seed)
    lens = [int(math.exp(rng.uniform(math.log(a.min_prompt), math.log(a.max_prompt)))) for _ in range(a.streams)]
    letters = "abcdefghijklmnopqrstuvwxyz ,.\n"
    prompts = ["".join(rng.choice(letters) for _ in range(n)) for n in lens]
    proc = None
    url = a.url
    if not url:
        url = f"http://127.0.0.1:{a.port}"
        total = sum(lens) + a.streams * (a.max_tokens + 64)
        cmd = [sys.executable, "-m", "rexl3_b200.server", "--host", "127.0.0.1", "--port", str(a.port), "--slots", str(a.streams), "--max-model-len",
               str(a.max_prompt + a.max_tokens + 64), "--queue-depth", str(a.streams * 2), "--served-model-name", "bench"]
        if a.backend == "mock":
            cmd += ["--backend", "mock", "--mock", "vocab=512"]
        else:
            cmd += ["--backend", "cuda", "--random-init", a.model, "--kv-dtype", a.kv_dtype, "--kv-tokens", str(int(total * 1.1)), "--prefill-chunk", "8192",
                    "--window-rows", str(max(64, a.streams)), "--spec", "none", "--prefix-cache", "off"]
        proc = subprocess.Popen(cmd, start_new_session=True)
        if not wait_ready(url, 600):
            proc.send_signal(signal.SIGTERM)
            print(json.dumps({"bench": "serve_load", "error": "server did not become ready"}))
            return 1
    try:
        asyncio.run(run(url, "bench", [prompts[0][:64]], 4))          # one short request first: graph capture and allocator warm-up are not TTFT
        res, wall = asyncio.run(run(url, "bench", prompts, a.max_tokens))
    finally:
        if proc is not None:
            proc.send_signal(signal.SIGTERM)
            try:
                proc.wait(timeout=30)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)
    ok = [r for r in res if "error" not in r and r["ttft"] is not None]
    ttfts = sorted(r["ttft"] for r in ok)
    toks = sum(r["tokens"] for r in ok)
    pct = lambda q: round(ttfts[min(len(ttfts) - 1, int(q * len(ttfts)))] * 1e3, 1) if ttfts else None  # noqa: E731
    print(json.dumps({"bench": "serve_load", "backend": a.backend, "model": a.model, "streams": a.streams, "ok": len(ok), "errors": [r for r in res if "error" in r][:3],
                      "prompt_tokens_total": sum(lens), "prompt_len_min_max": [min(lens), max(lens)], "ttft_p50_ms": pct(0.5), "ttft_p90_ms": pct(0.9),
                      "ttft_mean_ms": round(statistics.mean(ttfts) * 1e3, 1) if ttfts else None, "completion_tokens": toks, "wall_s": round(wall, 2),
                      "decode_tokens_per_s": round(toks / wall, 1), "kv_dtype": a.kv_dtype if a.backend == "cuda" else None, "data": "synthetic"}))
    return 0 if len(ok) == a.streams else 1


if __name__ == "__main__":
    sys.exit(main())
