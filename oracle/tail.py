"""The decode tail's fit and its float64 model. Test infrastructure only.

Restates `tail_basis` / `tail_model` of the reference
(src/fold_attention/decode/cache.py:260-337) in numpy float64 by a different
route than the shipped fit, so the two check each other: the ridge regression
is a least-squares problem on the keys stacked over sqrt(ridge) I, and the
rank's directions are the right singular vectors of the fitted values. Pinned
against outputs of the reference's own `tail_model` in
`tests/golden/tail_model.npz` through the quantities the fit defines up to a
sign per rank: the effective K -> V map `vr u` and the block rows.
"""

from __future__ import annotations

import numpy as np

TAIL_BLOCK = 64
KBR = 256.0


def block_mean(x):
    """(S, W) -> means over consecutive 64-row blocks, the last over the rows it has."""
    S = x.shape[0]
    return np.stack([x[i:i + TAIL_BLOCK].mean(0) for i in range(0, S, TAIL_BLOCK)])


def centre(x):
    return x - np.repeat(block_mean(x), TAIL_BLOCK, 0)[: x.shape[0]]


def tail_fit(kint, ek, v, rank, lam=1e-3):
    """One row group: `kint` (S, D) plane A (integers), `ek` (S,) scales, `v`
    (S, D) values. Returns `(u int8 (r, D), vr (D, r), y (S, r), rows (nb, D))`;
    rank 0 gives `(None, None, None, block means)`."""
    kint = np.asarray(kint, np.float64)
    ek = np.asarray(ek, np.float64)
    v = np.asarray(v, np.float64)
    S, D = kint.shape
    rows = block_mean(v)
    if not rank:
        return None, None, None, rows
    kc, vc = centre(kint * ek[:, None]), centre(v)
    ridge = lam * (kc * kc).sum() / D
    stacked = np.concatenate([kc, np.sqrt(ridge) * np.eye(D)])
    target = np.concatenate([vc, np.zeros((D, D))])
    M = np.linalg.lstsq(stacked, target, rcond=None)[0]             # (D, D): v ~ k M
    _, _, vt = np.linalg.svd(kc @ M, full_matrices=False)
    basis = vt[:rank].T                                             # (D, r)
    proj = M @ basis
    step = np.maximum(np.abs(proj).max(0), 1e-30) / 127.0
    u = np.clip(np.rint(proj / step[None, :]), -127, 127)
    # the kernels' projection: the exact integer, times ek / 256 in fp32, rounded once
    y = ((kint @ u).astype(np.float32) * (ek.astype(np.float32) * np.float32(1.0 / KBR))[:, None]).astype(np.float64)
    vr = basis * (step * KBR)[None, :]
    rows = rows - block_mean(y) @ vr.T
    return u.T.astype(np.int8), vr, y, rows


def reentry(kint, ek, u, vr, rows):
    """Where each key's mass re-enters if it is dropped, (S, D): its block's
    row plus its own projection mapped back."""
    S = kint.shape[0]
    out = np.repeat(np.asarray(rows, np.float64), TAIL_BLOCK, 0)[:S]
    if u is not None:
        kint = np.asarray(kint, np.float64)
        y = ((kint @ np.asarray(u, np.float64).T).astype(np.float32)
             * (np.asarray(ek, np.float32) * np.float32(1.0 / KBR))[:, None]).astype(np.float64)
        out = out + y @ np.asarray(vr, np.float64).T
    return out


def append(kint_row, ek_row, v_row, off, u, vr, vsum, ysum):
    """One appended key's update of its block (`off` its slot in the page):
    returns the block's new `(vsum, ysum, row)` in fp32, each operation rounded
    as the step kernel rounds it (src/fold_attention/decode/write.py:193-300)."""
    f = np.float32
    first = off % TAIL_BLOCK == 0
    nk = f(off % TAIL_BLOCK + 1)
    vs = (np.zeros_like(vsum) if first else vsum).astype(f) + np.asarray(v_row, f)
    row = vs / nk
    ys = None
    if u is not None:
        dots = np.asarray(kint_row, np.int64) @ np.asarray(u, np.int64).T
        yj = dots.astype(f) * (f(ek_row) * f(1.0 / KBR))
        ys = (np.zeros_like(ysum) if first else ysum).astype(f) + yj
        yb = ys / nk
        for j in range(u.shape[0]):
            row = row - yb[j] * np.asarray(vr, f)[:, j]
    return vs, ys, row
