"""Hessian-aware rounding for the EXL3 quantizer: Hessian finalize / damp, rotation into the coded basis, block-16 LDL
factorisation and the LDLQ error-feedback loop over 16-row tile blocks.

Stages named by the reference's quantizer outline (crates/quant/src/lib.rs:1-30, crates/quant/src/core/mod.rs:1-12:
"Hessian finalize/damp, sign flips + block-128 Hadamard, block-16 LDL, LDLQ rounding, ... scale refit"); the arithmetic
here is the textbook form, in float64 with a fixed order of operations.

For a linear layer y = x @ W (W is [K, N]) with input second moment H = E[x x^T], the output error of a quantized Q is
tr((Q - W)^T H (Q - W)).  With H = L D L^T (L unit block-lower-triangular, blocks of 16 rows = one row of trellis tiles)
that is sum_b || D_b^(1/2) (L^T e)_b ||^2 with e = Q - W, and (L^T e)_b = e_b + sum_{j>b} L[j,b]^T e_j.  Coding the
row blocks from the last to the first and giving block b the target W_b - sum_{j>b} L[j,b]^T e_j leaves in (L^T e)_b
only the rounding error of block b itself: errors already made are compensated by the rows not coded yet.
"""
from __future__ import annotations

import numpy as np

from ..format import exl3

BLOCK = 16


def finalize_hessian(h: np.ndarray, damp: float = 0.01) -> np.ndarray:
    """Symmetrise, give dead inputs (zero diagonal) a unit diagonal, and add damp * mean(diag) to the diagonal."""
    h = np.asarray(h, dtype=np.float64)
    if h.ndim != 2 or h.shape[0] != h.shape[1]:
        raise ValueError("the Hessian is a square matrix over the layer's inputs")
    h = 0.5 * (h + h.T)
    d = np.diag(h).copy()
    dead = d <= 0
    if dead.any():
        h[dead, :] = 0
        h[:, dead] = 0
        h[dead, dead] = 1.0
        d = np.diag(h).copy()
    h = h + np.eye(h.shape[0]) * (damp * float(d.mean()))
    return h


def rotate_hessian(h: np.ndarray, su: np.ndarray) -> np.ndarray:
    """Second moment of the rotated input x' = Had(su * x): Had diag(su) H diag(su) Had (Had symmetric, block-diagonal, 128 wide)."""
    h = np.asarray(h, dtype=np.float64) * su[:, None] * su[None, :]
    h = exl3.rotate(h)                       # columns: h @ Had
    return exl3.rotate(h.T.copy()).T.copy()  # rows:    Had @ h


def block_ldl(h: np.ndarray, block: int = BLOCK):
    """H = L D L^T with L unit block-lower-triangular (identity diagonal blocks) and D block-diagonal.  -> (L, D)."""
    n = h.shape[0]
    if n % block:
        raise ValueError("size must be a multiple of the block")
    c = np.linalg.cholesky(h)
    d = np.zeros_like(h)
    inv = np.zeros_like(h)
    for b in range(0, n, block):
        cb = c[b:b + block, b:b + block]
        d[b:b + block, b:b + block] = cb @ cb.T
        inv[b:b + block, b:b + block] = np.linalg.inv(cb)
    return c @ inv, d


def ldlq(w: np.ndarray, h: np.ndarray, code_block, block: int = BLOCK) -> np.ndarray:
    """Quantize the rows of `w` [K, N] in blocks of `block` rows from the last block to the first with LDL error feedback.

    `code_block(b, target)` codes one [block, N] slab (row block index b) and returns the values it decodes to.  Returns the
    decoded Q [K, N]; the caller keeps whatever `code_block` stored (the packed tiles)."""
    k = w.shape[0]
    L, _ = block_ldl(h, block)
    q = np.zeros_like(w)
    err = np.zeros_like(w)                   # W - Q for the blocks already coded
    for b in range(k // block - 1, -1, -1):
        r0, r1 = b * block, (b + 1) * block
        target = w[r0:r1] + L[r1:, r0:r1].T @ err[r1:]
        q[r0:r1] = code_block(b, target)
        err[r0:r1] = w[r0:r1] - q[r0:r1]     # feedback carries the error against the ORIGINAL weights
    return q


def proxy_error(w: np.ndarray, q: np.ndarray, h: np.ndarray) -> float:
    """tr((Q - W)^T H (Q - W)) / tr(W^T H W): the relative output error the Hessian predicts."""
    e = q - w
    return float(np.einsum("kn,kj,jn->", e, h, e) / max(np.einsum("kn,kj,jn->", w, h, w), 1e-300))


def refit_scale(w: np.ndarray, q: np.ndarray, h: np.ndarray | None = None) -> float:
    """The scalar s minimising the (Hessian-weighted) error of s * Q against W."""
    if h is None:
        num, den = float((w * q).sum()), float((q * q).sum())
    else:
        hq = h @ q
        num, den = float((w * hq).sum()), float((q * hq).sum())
    return num / den if den > 0 else 1.0
