"""Hybrid (Mamba2 + attention) family: the fp32 oracle's own invariants on CPU."""
import dataclasses

import numpy as np
import pytest
import torch

from rexl3_b200.models import hybrid

SMALL = dataclasses.replace(hybrid.CONFIGS["test-hybrid"], n_layers=3, pattern="MAM", d_model=256, n_q=2, n_kv=1, ffn=256, vocab=512, ssm_heads=4,
                            ssm_groups=2, name="cpu-hybrid")


GDN = dataclasses.replace(SMALL, pattern="GAG", nope=False, gdn_k_heads=1, gdn_v_heads=2, name="cpu-gdn")
KDA = dataclasses.replace(SMALL, pattern="KAK", gdn_k_heads=2, gdn_v_heads=2, name="cpu-kda")


def test_config_geometry():
    cfg = hybrid.CONFIGS["hybrid-h-56l"]
    cfg.validate()
    assert cfg.d_inner == 8192 and cfg.conv_channels == 10240 and cfg.in_proj_width % 128 == 0
    assert cfg.in_proj_width >= 2 * 8192 + 2048 + 128
    assert len(cfg.mamba_layers()) == 48 and len(cfg.attn_layers()) == 8
    assert cfg.kv_bytes_per_token() == 2 * 2 * 128 * 2 * 8


def test_gdn_config_geometry():
    cfg = hybrid.CONFIGS["gdn-hybrid-27b"]
    cfg.validate()
    assert cfg.gdn_conv_channels == 10240 and cfg.gdn_inner == 6144 and len(cfg.gdn_layers()) == 48 and len(cfg.attn_layers()) == 16
    assert cfg.gdn_proj_width % 128 == 0 and cfg.gdn_proj_width >= 6144 + 10240 + 96


@pytest.mark.parametrize("cfg", [SMALL, GDN, KDA], ids=["mamba2", "gdn", "kda"])
def test_chunked_equals_whole_and_position_zero_restarts(cfg):
    SMALL = cfg  # noqa: N806
    w = hybrid.random_weights(SMALL, seed=2)
    ref = hybrid.ReferenceHybrid(w)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, SMALL.vocab, size=21).tolist()
    whole = ref.forward_seq(0, toks, 0)
    a = ref.forward_seq(1, toks[:2], 0)
    b = ref.forward_seq(1, toks[2:13], 2)
    c = ref.forward_seq(1, toks[13:], 13)
    got = torch.cat([a, b, c])
    assert torch.allclose(got, whole, rtol=1e-4, atol=1e-4 * whole.abs().max().item())
    # feeding position 0 again restarts the recurrent state of that sequence
    ref.kv.pop(1)
    again = ref.forward_seq(1, toks, 0)
    assert torch.allclose(again, whole, rtol=1e-5, atol=1e-5 * whole.abs().max().item())
    # the Mamba2 layers matter: zeroing one layer's state input changes the logits
    other = ref.forward_seq(2, toks[::-1], 0)
    assert not torch.allclose(other[-1], whole[-1])


def test_engine_plans_no_drafts_without_rollback():
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.mock import MockBackend
    from rexl3_b200.sampling import GREEDY

    class NoRollback(MockBackend):
        def supports_rollback(self):
            return False

        def step(self, reqs, candidates):
            assert all(len(r.tokens) == 1 for r in reqs)
            return super().step(reqs, candidates)

    eng = Engine(NoRollback(), None, window_rows=16, spec="copy")
    assert not eng.can_rollback
    eng.submit(Request("a", [1, 2, 3, 1, 2, 3, 1, 2, 3], 12, GREEDY))
    n = 0
    for _ in range(100):
        if not eng.has_work():
            break
        for ev in eng.step():
            assert ev.kind != "error", ev.message
            if ev.kind == "tokens":
                n += len(ev.tokens)
    assert n == 12


@pytest.mark.parametrize("cfg", [SMALL, GDN], ids=["mamba2", "gdn"])
def test_engine_exactness_checks_on_the_cpu_hybrid_backend(cfg):
    """The engine's exactness harness over the fp32 hybrid oracle: a stream's tokens do not depend on its window mates, on batching or on
    how the prompt was chunked; a request with drafts enabled decodes the same tokens (the engine plans none for this backend)."""
    from rexl3_b200.engine import harness
    from rexl3_b200.engine.cpu_backend import CpuHybridBackend
    w = hybrid.random_weights(cfg, seed=5)

    def make():
        return CpuHybridBackend(w, max_slots=4, max_rows=16)
    for check in ("row_invariance", "serial_batched_equals_solo", "chunked_prefill_equals_whole", "drafted_equals_serial", "rollback_equals_replay"):
        assert getattr(harness, check)(make, cfg.vocab, n=6) is None, check


def test_cpu_hybrid_backend_scoring_leaves_the_state_untouched():
    from rexl3_b200.engine.backend import RowRequest
    from rexl3_b200.engine.cpu_backend import CpuHybridBackend
    be = CpuHybridBackend(hybrid.random_weights(SMALL, seed=5), max_slots=2)
    toks = [5, 9, 200, 31, 7, 7, 100]
    be.prefill_slice(0, 0, toks[:4], 8, True)
    a = be.score_rows(0, 4, toks[4:])
    b = be.score_rows(0, 4, toks[4:])                 # scoring twice gives the same rows: the first call did not advance the state
    assert np.array_equal(a, b)
    out = be.step([RowRequest(0, [toks[4]], 4)], 8)
    assert int(out[0][0].ids[0]) == int(np.argmax(a[0]))
    be.commit(0, 1)
    # a window of three rows of which one is kept: the state afterwards is the state of feeding that one row alone
    want = be.score_rows(0, 5, [toks[5], toks[6]])
    be.step([RowRequest(0, [toks[5], 1, 2], 5)], 8)
    be.commit(0, 1)
    got = be.step([RowRequest(0, [toks[6]], 6)], 8)
    assert int(got[0][0].ids[0]) == int(np.argmax(want[1]))


def test_hybrid_pack_roundtrip(tmp_path):
    """A hybrid model written as a pack and loaded back is the same model: config, every tensor, and the oracle's logits."""
    from rexl3_b200.format import verify
    from rexl3_b200.quant import quantize
    cfg = dataclasses.replace(SMALL, pattern="MKG", gdn_k_heads=1, gdn_v_heads=2, n_layers=3, name="cpu-pack")
    w = hybrid.random_weights(cfg, seed=8)
    folder = str(tmp_path / "pack")
    quantize.write_pack(folder, w)
    cfg2 = quantize.config_from_pack(folder)
    assert isinstance(cfg2, hybrid.HybridConfig)
    assert dataclasses.asdict(cfg2) == dataclasses.asdict(dataclasses.replace(cfg, head_bits=cfg.bits))      # the pack records the head width explicitly
    w2 = quantize.load_pack(folder)
    for a, b in zip(w.layers, w2.layers):
        assert type(a) is type(b)
        assert np.array_equal(a.in_proj.trellis, b.in_proj.trellis) and np.array_equal(a.out_proj.svh, b.out_proj.svh)
        assert np.array_equal(a.dt_bias, b.dt_bias) and np.array_equal(a.a_log, b.a_log) and np.array_equal(a.conv_w, b.conv_w)
        assert getattr(a, "kda", None) == getattr(b, "kda", None)
    toks = [3, 99, 250, 17, 400, 8]
    assert torch.equal(hybrid.ReferenceHybrid(w).forward_seq(0, toks, 0), hybrid.ReferenceHybrid(w2).forward_seq(0, toks, 0))
    assert len(verify.fingerprint(folder)) == 64


def test_quantize_hybrid_cli_writes_a_loadable_pack_close_to_the_float_model(tmp_path):
    from rexl3_b200.quant import quantize
    from rexl3_b200.quant.__main__ import main as quant_main
    cfg = dataclasses.replace(hybrid.CONFIGS["tiny-hybrid"], n_layers=2, pattern="MG", bits=6.0, name="cpu-q")
    fp = quantize.random_fp_weights_hybrid(cfg, seed=2)
    w = quantize.quantize_hybrid(cfg, fp, seed=2)
    # each quantized projection reproduces its float matrix (zero-padded to the stored width) to 6-bit accuracy
    for L, F in zip(w.layers, fp["layers"]):
        proj, ref = (L.qkv, np.concatenate([F["q"], F["k"], F["v"]], axis=1)) if hasattr(L, "qkv") else (L.in_proj, F["in_proj"])
        got = proj.dense()[:, :ref.shape[1]]
        assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 0.05
        pad = proj.dense()[:, ref.shape[1]:]             # columns nothing reads: only quantization noise of their shared 128-block
        assert pad.size == 0 or np.abs(pad).max() < 0.1 * np.abs(ref).max()
    folder = str(tmp_path / "q")
    quantize.write_pack(folder, w)
    w2 = quantize.load_pack(folder)
    toks = [3, 99, 250, 17]
    assert torch.equal(hybrid.ReferenceHybrid(w).forward_seq(0, toks, 0), hybrid.ReferenceHybrid(w2).forward_seq(0, toks, 0))
    # the command-line entry point on a built-in hybrid config (two layers of it)
    assert quant_main(["--arch", "tiny-hybrid", "--out", str(tmp_path / "cli"), "--layers", "1"]) == 0
    c2 = quantize.config_from_pack(str(tmp_path / "cli"))
    assert c2.pattern == "M" and c2.n_layers == 1 and len(quantize.load_pack(str(tmp_path / "cli")).layers) == 1


def test_delta_state_pool_order_matches_the_kernel_address_formula():
    """The delta-net state is stored in the order its kernel reads it; the canonical view undoes exactly that permutation.  The address
    below is the kernel's: thread (j, half) of warp j / 16, lane 2 (j % 16) + half, load step s, element e."""
    pool = torch.zeros(1, 1, 128, 128)
    flat = pool.view(-1)
    for j in range(128):
        for half in range(2):
            warp, lane = j // 16, 2 * (j % 16) + half
            for s in range(16):
                for e in range(4):
                    flat[warp * (16 * 128) + s * 128 + lane * 4 + e] = j * 1000 + (64 * half + 4 * s + e)
    want = (torch.arange(128)[:, None] * 1000 + torch.arange(128)[None, :]).float()
    assert torch.equal(hybrid.delta_state_canonical(pool)[0, 0], want)
    # every warp-wide load step covers one contiguous 512-byte run
    for warp in range(8):
        for s in range(16):
            addrs = sorted(warp * 2048 + s * 128 + lane * 4 + e for lane in range(32) for e in range(4))
            assert addrs == list(range(addrs[0], addrs[0] + 128))


def test_server_serves_a_hybrid_model_on_the_cpu_backend():
    from starlette.testclient import TestClient

    from rexl3_b200.server import main
    args = main.parser().parse_args(["--backend", "cpu", "--random-init", "tiny-hybrid", "--slots", "2", "--max-model-len", "256"])
    app, handle = main.make_app(args)
    try:
        assert handle.wait_ready(60)
        with TestClient(app) as c:
            body = {"prompt": "hello hybrid", "max_tokens": 6, "temperature": 0}
            a, b = c.post("/v1/completions", json=body).json(), c.post("/v1/completions", json=body).json()
            assert a["model"] == "tiny-hybrid" and a["usage"]["completion_tokens"] >= 1
            assert a["choices"][0]["text"] == b["choices"][0]["text"]            # a reused slot restarts its recurrent state at position 0
    finally:
        handle.stop()


@pytest.mark.parametrize("cfg", [SMALL, GDN], ids=["mamba2", "gdn"])
def test_prefix_cache_for_recurrent_state_through_slice_cuts(cfg):
    """A backend with recurrent state caches a block only where a prefill slice ended; the engine cuts a slice at the prompt's last
    block boundary, the second prompt restores the snapshot taken there, and decodes what a cold run decodes."""
    from rexl3_b200.engine import harness
    from rexl3_b200.engine.cpu_backend import CpuHybridBackend
    w = hybrid.random_weights(cfg, seed=5)

    def make():
        return CpuHybridBackend(w, max_slots=4, max_rows=16)
    assert make().prefix_needs_cuts()
    assert harness.cached_equals_cold(make, cfg.vocab, n=6) is None


def test_deepest_snapshot_selection():
    from rexl3_b200.engine.gpu_backend import deepest_snapshot
    assert deepest_snapshot([("hpage", 1, None), ("hpage", 2, {0: None}), ("hpage", 3, None)]) == 1
    assert deepest_snapshot([("hpage", 1, None)]) == -1 and deepest_snapshot([]) == -1
