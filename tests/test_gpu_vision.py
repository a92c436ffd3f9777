"""Image prompts on the CUDA backend: the engine's prefill carries the tower's rows and the (T, H, W) positions whatever the slice sizes,
decode rows rotate at position + delta, equal images share prefix-cache blocks, and the HTTP route serves an image part end to end."""
import base64
import dataclasses
import io

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _png(seed, h=224, w=336):
    from PIL import Image
    arr = np.random.default_rng(seed).integers(0, 256, size=(h, w, 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr, "RGB").save(buf, "PNG")
    return base64.b64encode(buf.getvalue()).decode()


def _part(seed):
    return {"type": "image_url", "image_url": {"url": "data:image/png;base64," + _png(seed)}}


@pytest.fixture(scope="module")
def setup():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from rexl3_b200.models import dense
    from rexl3_b200.server.media import VisionIngress
    from rexl3_b200.vision import tower
    cfg = dataclasses.replace(dense.CONFIGS["test-hd128"], mrope_sections=(24, 20, 20))
    model = dense.DenseGPU(dense.random_weights(cfg, seed=3), num_pages=64, max_rows=64, max_seqs=4, max_blocks_per_seq=8, max_prefill_rows=512)
    vcfg = tower.CONFIGS["test-vit"]
    IMG = 7
    ing = VisionIngress(vcfg, lambda: tower.VisionTower(vcfg, seed=2, device="cuda"), IMG, "", mrope=True, min_pixels=28 * 28, max_pixels=28 * 28 * 40)
    return model, ing, IMG


def _prompt(ing, IMG, seed, tail=(8, 9, 10)):
    rng = np.random.default_rng(100)
    head = rng.integers(20, 4000, size=30).tolist()
    return ing.prepare(head + [IMG] + list(tail), [ing.decode(_part(seed))])


def test_engine_image_prompt_slices_delta_and_prefix_cache(setup):
    from rexl3_b200.engine import Engine, Request
    from rexl3_b200.engine.gpu_backend import DenseGpuBackend
    from rexl3_b200.sampling import GREEDY
    from rexl3_b200.sched import CacheBudget, PrefixIndex
    model, ing, IMG = setup
    ids, md = _prompt(ing, IMG, 1)
    ids2, md2 = _prompt(ing, IMG, 2)
    n = len(ids)
    assert len(md.rows) > 16 and md.rope_delta < 0 and n > 64 and ids == ids2          # same tokens, other pixels

    def run(prompt, media, chunk, prefix=None, be=None):
        be = be or DenseGpuBackend(model, max_slots=4)
        eng = Engine(be, spec="none", prefill_chunk=chunk, prefix=prefix)
        eng.submit(Request("r", list(prompt), 10, GREEDY, media=media))
        out = []
        while eng.has_work():
            for ev in eng.step():
                assert ev.kind != "error", ev.message
                out.extend(ev.tokens if ev.kind == "tokens" else [])
        return out, eng, be

    whole, _, be = run(ids, md, 4096)
    assert be.stats()["media_rows"] == len(md.rows)
    for chunk in (16, 40):                                                               # slices that cut the image run
        assert run(ids, md, chunk)[0] == whole
    assert run(ids2, md2, 4096)[0] != whole                                              # the reply follows the pixels
    # the same two steps by hand: prefill logits with the rows and positions, then one decode row at position n + delta
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")  # noqa: E731
    bt = torch.zeros(4, 8, dtype=torch.int32, device="cuda")
    bt[0, :3] = i32([40, 41, 42])
    pos = list(range(n))
    slot = lambda p: int(bt[0, p // 64]) * 64 + p % 64  # noqa: E731
    pf = dict(seq_ids=i32([0]), q_start=i32([0]), q_len=i32([n]), pos0=i32([0]), nseq=1, max_qlen=n)
    er = (torch.as_tensor(md.rows, device="cuda"), md.embeds.to("cuda", torch.bfloat16))
    lg = model.forward_rows(i32(ids), i32(pos), i32([slot(p) for p in pos]), i32([0] * n), i32([p + 1 for p in pos]), bt, prefill=pf,
                            logit_rows=torch.tensor([n - 1], device="cuda"), embed_rows=er, pos3=torch.as_tensor(md.pos3, device="cuda").contiguous())
    t1 = int(lg[0, :model.cfg.vocab].argmax())
    assert t1 == whole[0]
    model.window_seq_rows = 1
    lg = model.forward_rows(i32([t1]), i32([n + md.rope_delta]), i32([slot(n)]), i32([0]), i32([n + 1]), bt)
    assert int(lg[0, :model.cfg.vocab].argmax()) == whole[1]
    # prefix cache: the same image restores blocks, another image with the same tokens does not get them
    be = DenseGpuBackend(model, max_slots=4)
    px = PrefixIndex(CacheBudget(1 << 30), block_tokens=be.prefix_block_tokens())
    a, eng, _ = run(ids, md, 4096, px, be)
    b, eng, _ = run(ids, md, 4096, px, be)
    assert a == b == whole and eng.counters["cached_tokens"] >= 64
    c, eng3, _ = run(ids2, md2, 4096, px, be)
    assert c != whole and eng3.counters["cached_tokens"] == 0                                  # nothing was restored for the other image


def test_chat_route_serves_an_image_on_the_cuda_backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from starlette.testclient import TestClient
    from rexl3_b200.server.main import make_app, parser
    args = parser().parse_args(["--backend", "cuda", "--random-init", "test-hd128", "--slots", "3", "--max-model-len", "1024", "--prefill-chunk", "256",
                                "--kv-tokens", "4096", "--window-rows", "16", "--vision-tower", "test-vit", "--vision-max-pixels", str(28 * 28 * 40)])
    app, handle = make_app(args)
    try:
        assert handle.wait_ready(120), handle.error
        with TestClient(app) as c:
            def ask(seed):
                r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [{"type": "text", "text": "look: "}, _part(seed)]}],
                                                         "max_tokens": 6, "temperature": 0, "return_token_ids": True})
                assert r.status_code == 200, r.text
                return r.json()
            a, a2, b = ask(1), ask(1), ask(2)
            assert a["choices"][0]["token_ids"] == a2["choices"][0]["token_ids"] and a["choices"][0]["token_ids"] != b["choices"][0]["token_ids"]
            assert a["usage"]["prompt_tokens"] > 30
            assert c.get("/v1/models").json()["data"][0]["vision"]["tower"] == "test-vit"
    finally:
        handle.stop()


def test_chat_route_with_the_packs_own_tower(tmp_path):
    """A pack with a tower beside it (vision.safetensors + vision_config): `--vision-tower pack` loads it, the reply follows the pixels, and
    the rows equal what the stored tower gives on the host."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from starlette.testclient import TestClient
    from rexl3_b200.models import dense
    from rexl3_b200.quant import quantize
    from rexl3_b200.server.main import make_app, parser
    from rexl3_b200.vision import tower
    cfg = dense.CONFIGS["test-hd128"]
    folder = str(tmp_path / "pack")
    quantize.write_pack(folder, dense.random_weights(cfg, seed=3))
    tower.save_tower(folder, tower.VisionTower(tower.CONFIGS["test-vit"], seed=9, device="cpu", dtype=torch.bfloat16))
    args = parser().parse_args(["--backend", "cuda", "--model", folder, "--slots", "3", "--max-model-len", "1024", "--prefill-chunk", "256",
                                "--kv-tokens", "4096", "--window-rows", "16", "--vision-tower", "pack", "--vision-max-pixels", str(28 * 28 * 40)])
    app, handle = make_app(args)
    try:
        assert handle.wait_ready(120), handle.error
        with TestClient(app) as c:
            def ask(seed):
                r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [_part(seed), {"type": "text", "text": " what?"}]}],
                                                         "max_tokens": 5, "temperature": 0, "return_token_ids": True})
                assert r.status_code == 200, r.text
                return r.json()["choices"][0]["token_ids"]
            assert ask(1) == ask(1) and ask(1) != ask(2)
            v = c.get("/v1/models").json()["data"][0]["vision"]
            assert v["weights"].startswith("vision.safetensors") and v["out_dim"] == cfg.d_model
    finally:
        handle.stop()
    # a pack without a tower is refused at start-up, by name
    bare = str(tmp_path / "bare")
    quantize.write_pack(bare, dense.random_weights(cfg, seed=3))
    with pytest.raises(SystemExit, match="holds no vision tower"):
        make_app(parser().parse_args(["--backend", "cuda", "--model", bare, "--vision-tower", "pack"]))
