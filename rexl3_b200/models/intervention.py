"""Runtime interventions: a manifest plus direction files applied at serving time without touching the weights (family-neutral, fail-closed;
reference crates/model/src/intervention.rs:1-16).

An intervention directory holds `intervention.json` and direction files (`.npy`, or `.pt` holding one tensor): float vectors [d_model] or
[r, d_model].  At load every layer index is checked against the model, every file against its pinned sha256 and the model's width; the
directions of a layer are orthonormalised in manifest order (Gram-Schmidt in float64), and at the application point - the output of the
layer's feed-forward block, before it joins the residual stream - each forward does

    y <- y - alpha * sum_j (y . d_j) d_j

(a rank-r ablation of the block's output).  Any mismatch refuses the boot naming both sides: an overlay made for another model or another
layer numbering never applies silently.

    {"schema": "rexl3.intervention.v1", "model": {"name": "dense-27b", "n_layers": 64, "d_model": 5120}, "application_point": "ffn_output",
     "alpha": 1.0, "directions": [{"file": "refusal.npy", "sha256": "...", "layers": [20, 21, 22]}]}
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass

import numpy as np

SCHEMA = "rexl3.intervention.v1"
POINTS = ("ffn_output",)


class InterventionError(ValueError):
    pass


@dataclass
class LayerOverlay:
    layer: int
    alpha: float
    basis: np.ndarray        # float32 [r, d_model], orthonormal rows


def _load_vectors(path: str) -> np.ndarray:
    if path.endswith(".npy"):
        a = np.load(path, allow_pickle=False)
    elif path.endswith(".pt"):
        import torch
        t = torch.load(path, map_location="cpu", weights_only=True)
        if isinstance(t, dict) and len(t) == 1:
            t = next(iter(t.values()))
        if not hasattr(t, "numpy"):
            raise InterventionError(f"{path}: expected one tensor, found {type(t).__name__}")
        a = t.float().numpy()
    else:
        raise InterventionError(f"{path}: direction files are .npy or .pt")
    a = np.asarray(a, dtype=np.float64)
    if a.ndim == 1:
        a = a[None]
    if a.ndim != 2 or a.shape[0] < 1:
        raise InterventionError(f"{path}: a direction file holds [d_model] or [r, d_model], found shape {list(a.shape)}")
    if not np.isfinite(a).all():
        raise InterventionError(f"{path}: a direction holds a non-finite value")
    return a


def orthonormalise(rows: np.ndarray, what: str = "directions") -> np.ndarray:
    """Gram-Schmidt in the given order (float64); a direction that is (numerically) inside the span of the earlier ones is refused."""
    out = []
    for i, v in enumerate(rows):
        u = v.astype(np.float64).copy()
        n0 = np.linalg.norm(u)
        if n0 == 0.0:
            raise InterventionError(f"{what}: direction {i} is zero")
        for q in out:
            u -= (u @ q) * q
        for q in out:                      # second pass: keeps the basis orthogonal to rounding level
            u -= (u @ q) * q
        n = np.linalg.norm(u)
        if n < 1e-6 * n0:
            raise InterventionError(f"{what}: direction {i} lies in the span of the directions before it")
        out.append(u / n)
    return np.stack(out)


def load(folder: str, *, n_layers: int, d_model: int, model_name: str | None = None) -> dict:
    """-> {layer index: LayerOverlay}.  Raises InterventionError (naming the manifest's side and the model's side) on any mismatch."""
    mpath = os.path.join(folder, "intervention.json")
    try:
        man = json.load(open(mpath))
    except (OSError, json.JSONDecodeError) as e:
        raise InterventionError(f"{mpath}: {e}") from None
    if man.get("schema") != SCHEMA:
        raise InterventionError(f"{mpath}: schema {man.get('schema')!r}, this build reads {SCHEMA!r}")
    point = man.get("application_point")
    if point not in POINTS:
        raise InterventionError(f"{mpath}: application point {point!r}, supported: {', '.join(POINTS)}")
    mm = man.get("model") or {}
    for key, have in (("n_layers", n_layers), ("d_model", d_model)):
        if mm.get(key) != have:
            raise InterventionError(f"{mpath}: made for a model with {key} {mm.get(key)!r}, the loaded model has {key} {have}")
    if model_name is not None and mm.get("name") not in (None, model_name):
        raise InterventionError(f"{mpath}: made for model {mm.get('name')!r}, the loaded model is {model_name!r}")
    alpha = float(man.get("alpha", 1.0))
    if not np.isfinite(alpha):
        raise InterventionError(f"{mpath}: alpha is not finite")
    dirs = man.get("directions")
    if not isinstance(dirs, list) or not dirs:
        raise InterventionError(f"{mpath}: no directions")
    per_layer: dict = {}
    for i, d in enumerate(dirs):
        name = d.get("file")
        if not isinstance(name, str) or os.path.basename(name) != name:
            raise InterventionError(f"{mpath}: directions[{i}].file must be a plain file name inside the directory")
        path = os.path.join(folder, name)
        try:
            blob = open(path, "rb").read()
        except OSError as e:
            raise InterventionError(f"{path}: {e}") from None
        sha = hashlib.sha256(blob).hexdigest()
        if d.get("sha256") != sha:
            raise InterventionError(f"{path}: sha256 {sha} differs from the manifest's pinned {d.get('sha256')!r}")
        vec = _load_vectors(path)
        if vec.shape[1] != d_model:
            raise InterventionError(f"{path}: directions of width {vec.shape[1]}, the loaded model has d_model {d_model}")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers or not all(isinstance(x, int) and not isinstance(x, bool) for x in layers):
            raise InterventionError(f"{mpath}: directions[{i}].layers must be a non-empty list of layer indices")
        for li in layers:
            if not 0 <= li < n_layers:
                raise InterventionError(f"{mpath}: directions[{i}] names layer {li}, the loaded model has layers 0..{n_layers - 1}")
            per_layer.setdefault(li, []).append(vec)
    return {li: LayerOverlay(li, alpha, orthonormalise(np.concatenate(v), f"layer {li}").astype(np.float32)) for li, v in sorted(per_layer.items())}


def write(folder: str, *, n_layers: int, d_model: int, directions: list, alpha: float = 1.0, model_name: str | None = None) -> str:
    """Writes an intervention directory: directions = [(file name, array [d] or [r, d], [layers])].  Returns the manifest path."""
    os.makedirs(folder, exist_ok=True)
    ds = []
    for name, arr, layers in directions:
        path = os.path.join(folder, name)
        np.save(path, np.asarray(arr, dtype=np.float32), allow_pickle=False)
        ds.append(dict(file=name, sha256=hashlib.sha256(open(path, "rb").read()).hexdigest(), layers=[int(x) for x in layers]))
    man = dict(schema=SCHEMA, model=dict(name=model_name, n_layers=n_layers, d_model=d_model), application_point="ffn_output", alpha=alpha, directions=ds)
    mpath = os.path.join(folder, "intervention.json")
    json.dump(man, open(mpath, "w"), indent=1)
    return mpath


def apply_reference(y, overlay: LayerOverlay):
    """y [T, d] (any float tensor) -> y - alpha (y B^T) B, the oracle form."""
    import torch
    B = torch.from_numpy(overlay.basis).to(device=y.device, dtype=y.dtype)
    return y - overlay.alpha * (y @ B.T) @ B
