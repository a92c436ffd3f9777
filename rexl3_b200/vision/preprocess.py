"""Image preprocessing on the CPU, byte-exact with PIL for the resize and value-exact with the usual HF processor arithmetic after it.

Role of the reference's `gb-vision` crate (crates/vision/src/lib.rs:1-50, resize.rs, preprocessor.rs) for the Qwen-VL style pipeline:
  1. `smart_resize`: pick (H, W), multiples of patch * merge, keeping the aspect ratio within a pixel budget;
  2. `bicubic_resize_u8`: the two-pass separable bicubic PIL runs on 8-bit images (support 2 scaled by the shrink factor, a = -0.5,
     coefficients normalised in float64 then turned into 22-bit fixed point, horizontal pass first, each pass rounded and clipped to 8 bits);
  3. rescale by 1/255 and normalise per channel in float32;
  4. `patchify`: frames are repeated to the temporal patch, cut into patch x patch tiles and ordered so the `merge x merge` tiles that the
     tower's merger fuses are consecutive; one row per tile, channel-major inside a row;
  5. `patch_position_ids`: the (row, column) index of every tile in that order, for the tower's 2-D rotary embedding.
Decoding of PNG / JPEG / WebP containers is left to PIL where it is installed; everything here takes an HxWx3 uint8 array.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)
PRECISION_BITS = 32 - 8 - 2


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280) -> tuple:
    """(H, W): both multiples of `factor`, area within [min_pixels, max_pixels], aspect ratio kept as closely as rounding allows."""
    if min(height, width) <= 0:
        raise ValueError("empty image")
    if max(height, width) / min(height, width) > 200:
        raise ValueError(f"aspect ratio {max(height, width) / min(height, width):.1f} is above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _bicubic(x: np.ndarray, a: float = -0.5) -> np.ndarray:
    x = np.abs(x)
    return np.where(x < 1.0, ((a + 2.0) * x - (a + 3.0)) * x * x + 1.0, np.where(x < 2.0, (((x - 5.0) * x + 8.0) * x - 4.0) * a, 0.0))


def _coefficients(in_size: int, out_size: int):
    """Per output pixel: first input index, tap count and 22-bit fixed-point weights, as PIL computes them."""
    scale = in_size / out_size
    filterscale = max(scale, 1.0)
    support = 2.0 * filterscale
    ksize = int(math.ceil(support)) * 2 + 1
    bounds = np.zeros((out_size, 2), dtype=np.int64)
    kk = np.zeros((out_size, ksize), dtype=np.float64)
    ss = 1.0 / filterscale
    for xx in range(out_size):
        center = (xx + 0.5) * scale
        xmin = max(int(center - support + 0.5), 0)
        xmax = min(int(center + support + 0.5), in_size) - xmin
        w = _bicubic((np.arange(xmax) + xmin - center + 0.5) * ss)
        tot = w.sum()
        if tot != 0.0:
            w = w / tot
        kk[xx, :xmax] = w
        bounds[xx] = (xmin, xmax)
    fixed = np.where(kk < 0, (kk * (1 << PRECISION_BITS) - 0.5).astype(np.int64), (kk * (1 << PRECISION_BITS) + 0.5).astype(np.int64))
    return bounds, fixed


def _pass(img: np.ndarray, out_size: int) -> np.ndarray:
    """Resample axis 1 of img [rows, in_size, channels] (uint8) to out_size."""
    rows, in_size, ch = img.shape
    bounds, kk = _coefficients(in_size, out_size)
    src = img.astype(np.int64)
    out = np.empty((rows, out_size, ch), dtype=np.uint8)
    half = 1 << (PRECISION_BITS - 1)
    for xx in range(out_size):
        x0, n = bounds[xx]
        acc = half + np.tensordot(src[:, x0:x0 + n, :], kk[xx, :n], axes=([1], [0]))
        out[:, xx, :] = np.clip(acc >> PRECISION_BITS, 0, 255).astype(np.uint8)
    return out


def bicubic_resize_u8(img: np.ndarray, height: int, width: int) -> np.ndarray:
    """HxWxC uint8 -> height x width x C uint8, the bytes `PIL.Image.resize((width, height), BICUBIC)` produces."""
    if img.dtype != np.uint8 or img.ndim != 3:
        raise ValueError("expects an HxWxC uint8 array")
    h, w, _ = img.shape
    out = img
    if w != width:
        out = _pass(out, width)                                               # horizontal first, as PIL does
    if h != height:
        out = _pass(out.transpose(1, 0, 2), height).transpose(1, 0, 2)
    return np.ascontiguousarray(out)


def patchify(frames: np.ndarray, patch: int = 14, merge: int = 2, temporal: int = 2):
    """frames float32 [T, C, H, W] (H, W multiples of patch * merge) -> (rows [grid_t * grid_h * grid_w, C * temporal * patch * patch],
    (grid_t, grid_h, grid_w)).  A single image is one frame; frames are padded to a multiple of `temporal` by repeating the last one."""
    t, c, h, w = frames.shape
    if h % (patch * merge) or w % (patch * merge):
        raise ValueError("image size must be a multiple of patch * merge")
    if t % temporal:
        frames = np.concatenate([frames, np.repeat(frames[-1:], temporal - t % temporal, axis=0)])
        t = frames.shape[0]
    gt, gh, gw = t // temporal, h // patch, w // patch
    x = frames.reshape(gt, temporal, c, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                              # gt, gh/m, gw/m, m, m, c, temporal, p, p
    return np.ascontiguousarray(x).reshape(gt * gh * gw, c * temporal * patch * patch), (gt, gh, gw)


def patch_position_ids(grid: tuple, merge: int = 2) -> np.ndarray:
    """int32 [rows, 2]: (row, column) of every tile in `patchify` order."""
    gt, gh, gw = grid
    hh = np.arange(gh)[:, None].repeat(gw, 1).reshape(gh // merge, merge, gw // merge, merge).transpose(0, 2, 1, 3).reshape(-1)
    ww = np.arange(gw)[None, :].repeat(gh, 0).reshape(gh // merge, merge, gw // merge, merge).transpose(0, 2, 1, 3).reshape(-1)
    ids = np.stack([hh, ww], axis=1).astype(np.int32)
    return np.tile(ids, (gt, 1))


@dataclass
class ImageInputs:
    pixel_values: np.ndarray       # float32 [rows, C * temporal * patch * patch]
    grid_thw: tuple                # (grid_t, grid_h, grid_w)
    position_ids: np.ndarray       # int32 [rows, 2]
    image_tokens: int              # placeholder tokens the prompt gets for this image (rows / merge^2)


def preprocess_image(img: np.ndarray, patch: int = 14, merge: int = 2, temporal: int = 2, min_pixels: int = 56 * 56,
                     max_pixels: int = 14 * 14 * 4 * 1280, mean=CLIP_MEAN, std=CLIP_STD) -> ImageInputs:
    """HxWx3 (or HxWx4: composited over white) uint8 -> what the tower and the prompt need."""
    if img.ndim == 3 and img.shape[2] == 4:
        a = img[:, :, 3:4].astype(np.uint16)
        img = ((img[:, :, :3].astype(np.uint16) * a + 255 * (255 - a) + 127) // 255).astype(np.uint8)
    h, w = smart_resize(img.shape[0], img.shape[1], patch * merge, min_pixels, max_pixels)
    px = bicubic_resize_u8(img, h, w)
    x = px.astype(np.float32) * np.float32(1.0 / 255.0)
    x = (x - np.asarray(mean, dtype=np.float32)) / np.asarray(std, dtype=np.float32)
    rows, grid = patchify(x.transpose(2, 0, 1)[None], patch, merge, temporal)
    return ImageInputs(rows.astype(np.float32), grid, patch_position_ids(grid, merge), rows.shape[0] // (merge * merge))


def preprocess_video(frames, patch: int = 14, merge: int = 2, temporal: int = 2, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 320,
                     mean=CLIP_MEAN, std=CLIP_STD) -> ImageInputs:
    """A clip as a sequence of HxWx3 uint8 frames of one size -> one ImageInputs whose grid_t counts temporal patches (frame pairs).  Every
    frame is resized to the same (H, W) chosen from the first frame; the pixel budget is per frame."""
    frames = list(frames)
    if not frames:
        raise ValueError("empty clip")
    if any(f.shape != frames[0].shape for f in frames):
        raise ValueError("the frames of a clip must share one size")
    h, w = smart_resize(frames[0].shape[0], frames[0].shape[1], patch * merge, min_pixels, max_pixels)
    m, sd = np.asarray(mean, dtype=np.float32), np.asarray(std, dtype=np.float32)
    stack = np.stack([((bicubic_resize_u8(f[:, :, :3], h, w).astype(np.float32) * np.float32(1.0 / 255.0)) - m) / sd for f in frames])
    rows, grid = patchify(np.ascontiguousarray(stack.transpose(0, 3, 1, 2)), patch, merge, temporal)
    return ImageInputs(rows.astype(np.float32), grid, patch_position_ids(grid, merge), rows.shape[0] // (merge * merge))
