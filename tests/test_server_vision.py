"""Image parts of chat requests through the HTTP path on the mock backend: decode, preprocessing, the (CPU) vision tower, placeholder
expansion, content-addressed prefix hashes, refusals by name."""
import base64
import io

import numpy as np
import pytest
from starlette.testclient import TestClient

from rexl3_b200.server import main, media


def png(seed: int, h: int = 40, w: int = 56, mode: str = "RGB", fmt: str = "PNG") -> str:
    from PIL import Image
    rng = np.random.default_rng(seed)
    arr = rng.integers(0, 256, size=(h, w, 4 if mode == "RGBA" else 3), dtype=np.uint8)
    buf = io.BytesIO()
    Image.fromarray(arr, mode).save(buf, fmt)
    return base64.b64encode(buf.getvalue()).decode()


@pytest.fixture(scope="module")
def client():
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512", "--slots", "4", "--max-model-len", "2048", "--queue-depth", "8",
                                     "--vision-tower", "test-vit", "--vision-max-pixels", str(28 * 28 * 12), "--vision-max-images", "2",
                                     "--prefix-cache", "on"])
    app, handle = main.make_app(args)
    assert handle.wait_ready(10)
    with TestClient(app) as c:
        yield c
    handle.stop()


def ask(c, parts, **kw):
    body = {"messages": [{"role": "user", "content": parts}], "max_tokens": 8, "seed": 1}
    body.update(kw)
    return c.post("/v1/chat/completions", json=body)


def image_part(b64: str, form: str = "url") -> dict:
    if form == "url":
        return {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}}
    if form == "bare":
        return {"type": "image_url", "image_url": "data:image/png;base64," + b64}
    return {"type": "image", "image": b64}


def test_image_parts_become_rows_and_the_reply_follows_the_pixels(client):
    a = png(1)
    text_only = ask(client, [{"type": "text", "text": "what is this? "}]).json()
    r1 = ask(client, [{"type": "text", "text": "what is this? "}, image_part(a)]).json()
    r1b = ask(client, [{"type": "text", "text": "what is this? "}, image_part(a, "bare")]).json()
    r1c = ask(client, [{"type": "text", "text": "what is this? "}, image_part(a, "image")]).json()
    r2 = ask(client, [{"type": "text", "text": "what is this? "}, image_part(png(2))]).json()
    inp = media.VisionIngress(__import__("rexl3_b200.vision.tower", fromlist=["x"]).CONFIGS["test-vit"], None, 0, "", mrope=False,
                              max_pixels=28 * 28 * 12).decode(image_part(a))[0]
    # the prompt grew by the image's merged patches plus the two vision brackets
    assert r1["usage"]["prompt_tokens"] == text_only["usage"]["prompt_tokens"] + inp.image_tokens + 2
    c1, c2 = r1["choices"][0]["message"]["content"], r2["choices"][0]["message"]["content"]
    assert c1 == r1b["choices"][0]["message"]["content"] == r1c["choices"][0]["message"]["content"]          # one image, three spellings
    assert c1 != c2 and c1 != text_only["choices"][0]["message"]["content"]                                  # the reply depends on the pixels
    rendered = client.post("/v1/chat/completions/render", json={"messages": [{"role": "user", "content": [image_part(a)]}]}).json()
    pad = 256 + 8 + 1
    assert rendered["token_ids"].count(pad) == inp.image_tokens and rendered["prompt"].count("<|image_pad|>") == 1


def test_same_image_hits_the_prefix_cache_and_another_image_does_not(client):
    long_text = "describe every detail of the picture, slowly and in order. " * 3
    a, b = png(3, 84, 84), png(4, 84, 84)
    first = ask(client, [image_part(a), {"type": "text", "text": long_text}]).json()
    again = ask(client, [image_part(a), {"type": "text", "text": long_text}]).json()
    other = ask(client, [image_part(b), {"type": "text", "text": long_text}]).json()
    assert first["usage"]["prompt_tokens"] > 128
    assert again["usage"]["prompt_tokens_details"]["cached_tokens"] >= 64
    assert again["choices"][0]["message"]["content"] == first["choices"][0]["message"]["content"]
    # same placeholder tokens, other pixels: only the text before the image (one short block at most) may be shared
    assert other["usage"]["prompt_tokens_details"]["cached_tokens"] < 64
    assert other["choices"][0]["message"]["content"] != first["choices"][0]["message"]["content"]


def test_transparent_and_jpeg_images_and_two_images_in_one_turn(client):
    r = ask(client, [image_part(png(5, mode="RGBA")), {"type": "text", "text": " and "}, image_part(png(6, fmt="JPEG"))])
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 8


def test_refusals_are_named(client):
    def err(parts):
        r = ask(client, parts)
        assert r.status_code == 400, r.text
        return r.json()["error"]
    e = err([{"type": "image_url", "image_url": {"url": "https://example.com/cat.png"}}])
    assert e["code"] == "remote_media_refused" and "not fetched" in e["message"]
    assert err([{"type": "image_url", "image_url": {"url": "data:image/png;base64,@@@"}}])["code"] == "invalid_image"
    assert err([{"type": "image_url", "image_url": {"url": "data:image/png;base64," + base64.b64encode(b"not an image").decode()}}])["code"] == "invalid_image"
    assert err([{"type": "image_url"}])["code"] == "invalid_image"
    assert err([image_part(png(1)), image_part(png(2)), image_part(png(3))])["code"] == "too_many_images"
    # the user's text spells the placeholder itself: the counts no longer match
    assert err([{"type": "text", "text": "<|image_pad|>"}, image_part(png(1))])["code"] == "image_placeholder_mismatch"
    assert err([{"type": "video_url", "video_url": {"url": "data:video/mp4;base64,AAAA"}}])["code"] == "unsupported"


def test_a_server_without_a_tower_refuses_image_parts():
    args = main.parser().parse_args(["--backend", "mock", "--mock", "vocab=512", "--slots", "2", "--max-model-len", "512"])
    app, handle = main.make_app(args)
    assert handle.wait_ready(10)
    with TestClient(app) as c:
        r = ask(c, [image_part(png(1))])
        assert r.status_code == 400 and "image input is not supported" in r.json()["error"]["message"]
    handle.stop()


def test_media_inputs_hash_by_content():
    from rexl3_b200.engine.backend import MediaInputs
    from rexl3_b200.sched import chain_hashes
    prompt = [1, 2] + [9] * 70 + [3]
    rows = np.arange(2, 72)
    ma = MediaInputs(rows, np.zeros((70, 4), np.float32), None, 0, [(0, 70, b"a" * 32)])
    mb = MediaInputs(rows, np.zeros((70, 4), np.float32), None, 0, [(0, 70, b"b" * 32)])
    ha, hb = chain_hashes(ma.hash_tokens(prompt), 64), chain_hashes(mb.hash_tokens(prompt), 64)
    assert ha != hb and ha == chain_hashes(ma.hash_tokens(prompt), 64) and ha != chain_hashes(prompt, 64)
