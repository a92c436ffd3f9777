"""Vision tower of the image path: patches -> embeddings that replace the prompt's image placeholder rows.

Shape of the reference's Qwen-class tower (crates/cuda/csrc/vision.cu:1-12, crates/vision): a linear patch embedding over
C * temporal * patch * patch values, a learned position table interpolated bilinearly to the image's grid, pre-LayerNorm blocks with
bidirectional attention inside one image (axial 2-D rotary embedding: half of each head's pairs rotate by the patch row, half by its
column), a tanh-GELU MLP, and a merger that folds every merge x merge window (consecutive rows in `preprocess.patchify` order) into one token of
the language model's width.  The encoder runs one image at a time and is not part of the serial == drafted contract; it is deterministic.

Here it is a PyTorch module on the GPU: its GEMMs are plain library GEMMs (linear layers), its attention is PyTorch's fused bidirectional
attention; fp32 residual stream, LayerNorm statistics in fp32, bf16 operands.  `VisionTower.reference()` is the same network in fp32 on any
device (the oracle of the tests).  `splice` puts the encoded rows into a prompt and builds the (T, H, W) positions interleaved M-RoPE wants.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class VisionConfig:
    hidden: int = 1152
    heads: int = 16
    depth: int = 27
    mlp: int = 4304
    patch: int = 14
    temporal: int = 2
    merge: int = 2
    channels: int = 3
    pos_grid: int = 48            # the learned table is pos_grid x pos_grid
    out_dim: int = 5120           # the language model's width
    eps: float = 1e-6
    rope_theta: float = 1e4
    name: str = "vit"

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def patch_values(self) -> int:
        return self.channels * self.temporal * self.patch * self.patch

    def validate(self) -> None:
        if self.hidden % self.heads or self.head_dim % 4:
            raise ValueError("hidden must split into heads whose width is a multiple of 4 (axial rotary pairs)")


CONFIGS = {
    "qwen-vit-27": VisionConfig(),
    "test-vit": VisionConfig(hidden=128, heads=4, depth=2, mlp=256, pos_grid=8, out_dim=512, name="test-vit"),
}


def _weights(cfg: VisionConfig, seed: int, device, dtype):
    g = torch.Generator(device="cpu").manual_seed(seed)
    rn = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(device=device, dtype=dtype)  # noqa: E731
    h, m = cfg.hidden, cfg.mlp
    w = dict(patch_w=rn(h, cfg.patch_values, scale=1 / math.sqrt(cfg.patch_values)), patch_b=rn(h, scale=0.02),
             pos_table=rn(cfg.pos_grid * cfg.pos_grid, h, scale=0.02), blocks=[])
    for _ in range(cfg.depth):
        w["blocks"].append(dict(ln1_w=1 + rn(h, scale=0.05), ln1_b=rn(h, scale=0.02), qkv_w=rn(3 * h, h, scale=1 / math.sqrt(h)), qkv_b=rn(3 * h, scale=0.02),
                                proj_w=rn(h, h, scale=0.5 / math.sqrt(h)), proj_b=rn(h, scale=0.02), ln2_w=1 + rn(h, scale=0.05), ln2_b=rn(h, scale=0.02),
                                fc1_w=rn(m, h, scale=1 / math.sqrt(h)), fc1_b=rn(m, scale=0.02), fc2_w=rn(h, m, scale=0.5 / math.sqrt(m)), fc2_b=rn(h, scale=0.02)))
    mh = h * cfg.merge * cfg.merge
    w.update(ln_w=1 + rn(h, scale=0.05), ln_b=rn(h, scale=0.02), m1_w=rn(mh, mh, scale=1 / math.sqrt(mh)), m1_b=rn(mh, scale=0.02),
             m2_w=rn(cfg.out_dim, mh, scale=1 / math.sqrt(mh)), m2_b=rn(cfg.out_dim, scale=0.02))
    return w


def interpolation_table(grid_h: int, grid_w: int, pos_grid: int):
    """Bilinear sampling of a pos_grid x pos_grid table on a grid_h x grid_w lattice that spans it corner to corner: (indices int64 [rows, 4],
    weights float32 [rows, 4]) in row-major patch order."""
    ys = np.linspace(0, pos_grid - 1, grid_h, dtype=np.float64)
    xs = np.linspace(0, pos_grid - 1, grid_w, dtype=np.float64)
    y0, x0 = np.floor(ys).astype(np.int64), np.floor(xs).astype(np.int64)
    y1, x1 = np.minimum(y0 + 1, pos_grid - 1), np.minimum(x0 + 1, pos_grid - 1)
    fy, fx = (ys - y0)[:, None], (xs - x0)[None, :]
    idx = np.stack([y0[:, None] * pos_grid + x0[None, :], y0[:, None] * pos_grid + x1[None, :], y1[:, None] * pos_grid + x0[None, :],
                    y1[:, None] * pos_grid + x1[None, :]], -1).reshape(-1, 4)
    wgt = np.stack([(1 - fy) * (1 - fx), (1 - fy) * fx, fy * (1 - fx), fy * fx], -1).reshape(-1, 4).astype(np.float32)
    return idx, wgt


VISION_FILE = "vision.safetensors"
_BLOCK_KEYS = ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")
_TOP_KEYS = ("patch_w", "patch_b", "pos_table", "ln_w", "ln_b", "m1_w", "m1_b", "m2_w", "m2_b")


def _flat(w: dict) -> dict:
    out = {f"vision.{k}": w[k] for k in _TOP_KEYS}
    for i, blk in enumerate(w["blocks"]):
        out.update({f"vision.blocks.{i}.{k}": blk[k] for k in _BLOCK_KEYS})
    return out


def save_tower(folder: str, tower: "VisionTower") -> None:
    """Writes the tower beside a pack: `vision.safetensors` (bf16 tensors `vision.*`) and a `vision_config` object in config.json."""
    import dataclasses
    import json
    import os
    from ..format import safetensors_io as sio
    tensors, dtypes = {}, {}
    for name, t in _flat(tower.w).items():
        tensors[name] = t.detach().to("cpu", torch.bfloat16).contiguous().view(torch.int16).numpy().view(np.uint16)
        dtypes[name] = "BF16"
    sio.write_file(os.path.join(folder, VISION_FILE), tensors, {"format": "rexl3-vision-v1"}, dtypes)
    path = os.path.join(folder, "config.json")
    doc = json.load(open(path)) if os.path.exists(path) else {}
    doc["vision_config"] = dataclasses.asdict(tower.cfg)
    with open(path, "w") as f:
        json.dump(doc, f, indent=1)


def config_from_pack(folder: str) -> "VisionConfig | None":
    """The pack's `vision_config`, or None when the pack has no tower.  Unknown keys are refused by name."""
    import json
    import os
    path = os.path.join(folder, "config.json")
    if not os.path.exists(path) or not os.path.exists(os.path.join(folder, VISION_FILE)):
        return None
    vc = json.load(open(path)).get("vision_config")
    if not isinstance(vc, dict):
        raise ValueError(f"{folder}: {VISION_FILE} is there but config.json has no vision_config")
    known = {f.name for f in __import__("dataclasses").fields(VisionConfig)}
    bad = sorted(set(vc) - known)
    if bad:
        raise ValueError(f"{folder}: vision_config has unknown keys {bad}")
    cfg = VisionConfig(**vc)
    cfg.validate()
    return cfg


def load_tower(folder: str, device="cuda", dtype=torch.bfloat16) -> "VisionTower":
    """The tower stored beside a pack.  Every tensor the shape needs must be there with the right shape; surplus tensors are refused."""
    import os
    from ..format import safetensors_io as sio
    cfg = config_from_pack(folder)
    if cfg is None:
        raise ValueError(f"{folder}: the pack holds no vision tower ({VISION_FILE} + vision_config)")
    tower = VisionTower(cfg, seed=0, device="cpu", dtype=torch.float32)          # shapes (and a place to put the tensors)
    want = _flat(tower.w)
    scan = sio.read_header(os.path.join(folder, VISION_FILE))
    if scan.issues:
        raise ValueError(f"{folder}/{VISION_FILE}: {scan.issues[0]}")
    have = dict(scan.entries)
    missing, extra = sorted(set(want) - set(have)), sorted(set(have) - set(want))
    if missing or extra:
        raise ValueError(f"{folder}/{VISION_FILE}: missing {missing[:3]}{'...' if len(missing) > 3 else ''}, unexpected {extra[:3]}{'...' if len(extra) > 3 else ''}")
    def put(dst: dict, key: str, name: str):
        e = have[name]
        if e.dtype != "BF16" or tuple(e.shape) != tuple(dst[key].shape):
            raise ValueError(f"{VISION_FILE}: {name} is {e.dtype} {list(e.shape)}, the shape needs BF16 {list(dst[key].shape)}")
        bits = sio.read_tensor(folder, e)
        dst[key] = torch.from_numpy(np.array(bits, copy=True).view(np.int16)).view(torch.bfloat16).to(device=device, dtype=dtype)
    for k in _TOP_KEYS:
        put(tower.w, k, f"vision.{k}")
    for i, blk in enumerate(tower.w["blocks"]):
        for k in _BLOCK_KEYS:
            put(blk, k, f"vision.blocks.{i}.{k}")
    tower.device, tower.dtype = torch.device(device), dtype
    tower.inv_freq = tower.inv_freq.to(tower.device)
    tower.from_pack = True
    return tower


class VisionTower:
    def __init__(self, cfg: VisionConfig, seed: int = 0, device="cuda", dtype=torch.bfloat16):
        cfg.validate()
        self.cfg, self.device, self.dtype, self.seed = cfg, torch.device(device), dtype, seed
        self.from_pack = False
        self.w = _weights(cfg, seed, self.device, dtype)
        hd = cfg.head_dim
        self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))).to(self.device)   # hd / 4 frequencies per axis

    def reference(self, device="cpu") -> "VisionTower":
        """The same network (same seed, weights rounded as stored) computing in fp32: the oracle."""
        ref = VisionTower(self.cfg, self.seed, device, torch.float32)
        src = _weights(self.cfg, self.seed, device, self.dtype)

        def widen(x):
            return [{k: v.float() for k, v in b.items()} for b in x] if isinstance(x, list) else x.float()
        ref.w = {k: widen(v) for k, v in src.items()}
        return ref

    # ------------------------------------------------------------------ pieces
    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """x [rows, heads, hd] (fp32); pos int [rows, 2] (patch row, patch column).  The first hd / 2 dims rotate by the row, the second by the
        column; inside each half the pairs are (d, d + hd / 4)."""
        hd = x.shape[-1]
        q = hd // 4
        out = []
        for axis in range(2):
            part = x[..., axis * 2 * q:(axis + 1) * 2 * q]
            ang = pos[:, axis].float()[:, None] * self.inv_freq[None]               # [rows, q]
            c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
            a, b = part[..., :q], part[..., q:]
            out.append(torch.cat([a * c - b * s, b * c + a * s], -1))
        return torch.cat(out, -1)

    def _ln(self, x, w, b):
        return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), self.cfg.eps)

    def _lin(self, x, w, b):
        return F.linear(x.to(w.dtype), w, b).float()

    # ------------------------------------------------------------------ forward
    def encode(self, pixel_values, grid_thw, position_ids) -> torch.Tensor:
        """pixel_values float [rows, C * temporal * patch * patch] in merger order, grid_thw (t, h, w), position_ids int [rows, 2]
        -> [rows / merge^2, out_dim] in the tower's dtype."""
        cfg, w = self.cfg, self.w
        gt, gh, gw = (int(v) for v in grid_thw)
        x = torch.as_tensor(pixel_values, device=self.device, dtype=torch.float32)
        pos = torch.as_tensor(position_ids, device=self.device, dtype=torch.int64)
        rows = x.shape[0]
        if rows != gt * gh * gw or x.shape[1] != cfg.patch_values:
            raise ValueError(f"pixel rows {tuple(x.shape)} do not match the grid {grid_thw} and {cfg.patch_values} values per patch")
        h = self._lin(x, w["patch_w"], w["patch_b"])
        idx, wgt = interpolation_table(gh, gw, cfg.pos_grid)
        if int(pos[:, 0].max()) >= gh or int(pos[:, 1].max()) >= gw or int(pos.min()) < 0:
            raise ValueError("position ids outside the grid")
        lattice = pos[:, 0] * gw + pos[:, 1]                                      # row-major index of every row's patch
        idx_t = torch.as_tensor(idx, device=self.device)[lattice]
        wgt_t = torch.as_tensor(wgt, device=self.device)[lattice]
        h = h + (w["pos_table"].float()[idx_t] * wgt_t[..., None]).sum(1)
        per_frame = gh * gw
        for blk in w["blocks"]:
            y = self._ln(h, blk["ln1_w"], blk["ln1_b"])
            qkv = self._lin(y, blk["qkv_w"], blk["qkv_b"]).view(rows, 3, cfg.heads, cfg.head_dim)
            q, k, v = self._rope(qkv[:, 0], pos), self._rope(qkv[:, 1], pos), qkv[:, 2]
            outs = []
            for f in range(gt):                                                   # attention stays inside one temporal patch (one image / frame pair)
                sl = slice(f * per_frame, (f + 1) * per_frame)
                qq, kk, vv = (t[sl].transpose(0, 1).unsqueeze(0).to(self.dtype) for t in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qq, kk, vv).squeeze(0).transpose(0, 1).reshape(per_frame, cfg.hidden))
            h = h + self._lin(torch.cat(outs, 0), blk["proj_w"], blk["proj_b"])
            y = self._ln(h, blk["ln2_w"], blk["ln2_b"])
            h = h + self._lin(F.gelu(self._lin(y, blk["fc1_w"], blk["fc1_b"]), approximate="tanh"), blk["fc2_w"], blk["fc2_b"])
        y = self._ln(h, w["ln_w"], w["ln_b"]).view(rows // (cfg.merge * cfg.merge), -1)    # merge x merge windows are consecutive rows
        y = self._lin(F.gelu(self._lin(y, w["m1_w"], w["m1_b"])), w["m2_w"], w["m2_b"])
        return y.to(self.dtype)


def splice(tokens: list, image_token: int, images: list, merge: int = 2):
    """Where a prompt's image placeholders are and which positions interleaved M-RoPE gives every token.

    tokens: the prompt with one run of `image_token` per image (run length = that image's tokens); images: [(grid_t, grid_h, grid_w)] in order.
    -> (rows int64 [n_image_tokens]: indices of the placeholder rows in prompt order, pos3 int32 [len(tokens), 3]).  Text tokens advance all
    three axes together; an image's tokens share the T position of its first token per temporal patch and spread H / W over its merged grid;
    the text after an image continues at 1 + the largest position the image used (Qwen2-VL's rule)."""
    pos3 = np.zeros((len(tokens), 3), dtype=np.int32)
    rows, nxt, i, img = [], 0, 0, 0
    while i < len(tokens):
        if tokens[i] != image_token:
            pos3[i] = nxt
            nxt += 1
            i += 1
            continue
        if img >= len(images):
            raise ValueError("more image placeholder runs than images")
        gt, gh, gw = images[img]
        mh, mw = gh // merge, gw // merge
        n = gt * mh * mw
        if tokens[i:i + n] != [image_token] * n or (i + n < len(tokens) and tokens[i + n] == image_token and False):
            raise ValueError(f"image {img} needs a run of {n} placeholder tokens at position {i}")
        t = np.repeat(np.arange(gt), mh * mw)
        hh = np.tile(np.repeat(np.arange(mh), mw), gt)
        ww = np.tile(np.arange(mw), gt * mh)
        pos3[i:i + n, 0], pos3[i:i + n, 1], pos3[i:i + n, 2] = nxt + t, nxt + hh, nxt + ww
        rows.extend(range(i, i + n))
        nxt += max(gt, mh, mw)
        i += n
        img += 1
    if img != len(images):
        raise ValueError("fewer image placeholder runs than images")
    return np.asarray(rows, dtype=np.int64), pos3
