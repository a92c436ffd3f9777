"""Image parts of chat requests: decode, preprocess, encode with the vision tower, and lay the rows into the prompt.

A chat message's content may be a list of parts; `{"type": "image_url", "image_url": {"url": "data:image/png;base64,..."}}` (or
`{"type": "image", "image": "<base64 or data URI>"}`) carries an image inline.  The chat format writes one placeholder token per image into
the rendered prompt (`<|vision_start|><|image_pad|><|vision_end|>` for the Qwen formats); here every placeholder grows into as many tokens
as the image has merged patches, the tower's rows replace those tokens' embeddings, and the (T, H, W) rotary positions and the content
digests for the prefix cache are made.  Remote URLs are refused by name: the server fetches nothing.

Behaviour parity: reference crates/vision/src/lib.rs (decode, smart resize, patch rows), crates/server/src/http.rs (image parts of chat
messages, refusal of parts a model cannot take), crates/sched/src/lib.rs:300-360 (image pseudo-tokens in prefix hashes).
"""
from __future__ import annotations

import base64
import binascii
import hashlib
import io

import numpy as np

from ..engine.backend import MediaInputs

IMAGE_PART_TYPES = ("image_url", "image")
FORMATS = ("PNG", "JPEG", "WEBP", "BMP", "GIF")


class MediaError(ValueError):
    """A media part that cannot be honoured; `code` goes into the error object."""

    def __init__(self, message: str, code: str = "invalid_image"):
        super().__init__(message)
        self.code = code


def _payload(part: dict) -> str:
    ty = part.get("type")
    v = part.get(ty)
    if isinstance(v, dict):
        v = v.get("url")
    if not isinstance(v, str) or not v:
        raise MediaError(f"a '{ty}' part needs a '{ty}' string (a data: URI or base64) or an object with a 'url'")
    return v


def decode_image(part: dict, max_bytes: int = 16 << 20, max_pixels: int = 64 << 20) -> tuple:
    """-> (HxWx3 or HxWx4 uint8 array, the image file's bytes).  Refuses remote URLs, oversized payloads, unknown containers and images whose
    header announces more than `max_pixels` before any pixel is decoded."""
    v = _payload(part)
    low = v[:16].lower()
    if low.startswith(("http://", "https://", "file:", "ftp:")):
        raise MediaError("remote image URLs are not fetched by this server: send the image inline as a data: URI", "remote_media_refused")
    if low.startswith("data:"):
        head, sep, b64 = v.partition(",")
        if not sep or ";base64" not in head.lower():
            raise MediaError("a data: URI must be base64 encoded (data:image/png;base64,...)")
        v = b64
    if len(v) > max_bytes * 4 // 3 + 4:
        raise MediaError(f"the image is larger than {max_bytes} bytes", "image_too_large")
    try:
        raw = base64.b64decode(v, validate=True)
    except (binascii.Error, ValueError):
        raise MediaError("the image payload is not valid base64")
    if len(raw) > max_bytes:
        raise MediaError(f"the image is larger than {max_bytes} bytes", "image_too_large")
    from PIL import Image
    try:
        im = Image.open(io.BytesIO(raw))
        if im.format not in FORMATS:
            raise MediaError(f"image container '{im.format}' is not accepted (one of {', '.join(FORMATS)})")
        w, h = im.size
        if w < 1 or h < 1 or w * h > max_pixels:
            raise MediaError(f"the image is {w} x {h}: more than {max_pixels} pixels", "image_too_large")
        im.seek(0)
        im = im.convert("RGBA" if (im.mode in ("RGBA", "LA", "PA") or "transparency" in im.info) else "RGB")
        arr = np.asarray(im, dtype=np.uint8)
    except MediaError:
        raise
    except Exception as e:      # PIL raises many types on damaged files
        raise MediaError(f"the image cannot be decoded: {type(e).__name__}: {e}")
    return arr, raw


class VisionIngress:
    """The server's image path: a vision tower, its preprocessing limits and the prompt's placeholder token."""

    def __init__(self, cfg, make_tower, image_token_id: int, placeholder_text: str, *, mrope: bool, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280, max_images: int = 8, max_image_bytes: int = 16 << 20):
        """cfg: vision.tower.VisionConfig; make_tower(): builds the tower on first use (the device runtime is then already up)."""
        import threading
        self.cfg, self._make_tower, self._tower, self._lock = cfg, make_tower, None, threading.Lock()
        self.image_token_id, self.placeholder_text = int(image_token_id), placeholder_text
        self.mrope = mrope
        self.min_pixels, self.max_pixels, self.max_images, self.max_image_bytes = min_pixels, max_pixels, max_images, max_image_bytes
        self.images_seen = 0
        self.rows_encoded = 0

    @property
    def tower(self):
        with self._lock:
            if self._tower is None:
                self._tower = self._make_tower()
            return self._tower

    def decode(self, part: dict):
        from ..vision import preprocess
        arr, raw = decode_image(part, self.max_image_bytes)
        cfg = self.cfg
        inp = preprocess.preprocess_image(arr, cfg.patch, cfg.merge, cfg.temporal, self.min_pixels, self.max_pixels)
        # the digest covers what the tower sees (resized, normalised patch rows) and the grid, so a re-encoded copy of the same pixels shares cache
        dig = hashlib.sha256(np.ascontiguousarray(inp.pixel_values).tobytes() + repr(tuple(int(x) for x in inp.grid_thw)).encode()).digest()
        return inp, dig

    def prepare(self, ids: list, images: list) -> tuple:
        """ids: the rendered prompt's tokens with ONE placeholder token per image, in order; images: [(ImageInputs, digest)].
        -> (the prompt with every placeholder repeated once per merged patch, MediaInputs)."""
        import torch
        from ..vision import tower as vt
        where = [i for i, t in enumerate(ids) if t == self.image_token_id]
        if len(where) != len(images):
            raise MediaError(f"the rendered prompt holds {len(where)} image placeholders for {len(images)} images (does the text contain the "
                             f"placeholder itself?)", "image_placeholder_mismatch")
        out, prev = [], 0
        for i, (inp, _) in zip(where, images):
            out.extend(ids[prev:i])
            out.extend([self.image_token_id] * inp.image_tokens)
            prev = i + 1
        out.extend(ids[prev:])
        rows, pos3 = vt.splice(out, self.image_token_id, [tuple(int(x) for x in inp.grid_thw) for inp, _ in images], self.cfg.merge)
        embeds, keys, first = [], [], 0
        with torch.no_grad():
            for inp, dig in images:
                e = self.tower.encode(inp.pixel_values, inp.grid_thw, inp.position_ids)
                embeds.append(e.float().cpu())
                keys.append((first, int(e.shape[0]), dig))
                first += int(e.shape[0])
        emb = torch.cat(embeds, 0) if embeds else torch.zeros(0, self.cfg.out_dim)
        self.images_seen += len(images)
        self.rows_encoded += int(emb.shape[0])
        delta = int(pos3.max()) + 1 - len(out) if (self.mrope and len(out)) else 0
        return out, MediaInputs(rows, emb, pos3 if self.mrope else None, delta, keys)
