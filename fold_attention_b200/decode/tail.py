"""The decode tail: where a truncated step's dropped mass re-enters.

Without a tail, the mass of the keys a finite depth drops re-enters at the
request's mean V. With one, a dropped key re-enters at its own 64-key block's
mean V plus the part of its V that its K predicts: a linear map fitted on the
prompt, `v - vblk ~ (k - kblk) M`, cut to the r directions that carry most of
the fitted values. The decode then needs, per row group, the int8 projection
`u` `(r, D)` (applied to plane A of K by the logit matmul's own instruction),
the map back `vr` `(D, r)`, and per 64-key block of the pool one row
`vblk - yblk vr^T` in V's 16-bit format; the append keeps the block sums and
rows current. bf16 V caches only.

The model is the reference's (`cache.tail_basis` / `cache.tail_model` and
`FoldKVCache._fit_tail`, src/fold_attention/decode/cache.py:270-337,
kv_cache.py:300-417). The fit here works from the D x D moment matrices
(`moments`, fp32 products over a request's own keys; `rank_map`, float64
Cholesky and eigenvectors one matrix at a time): the fitted values' Gram
matrix is `M^T (Kc^T Kc) M`, so no second pass over the keys is needed.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

TAIL_BLOCK = 64     # keys per block row: the warp-level decode kernel's tile
KBR = 256.0         # the kernel multiplies plane-A dot products by ek / 256


@dataclass
class TailState:
    """A serving cache's tail: every 64-key pool block's row (`rows`, V's
    dtype), V sum and projection sum, and each row group's rank map."""

    rows: torch.Tensor            # (pool_rows / 64, D) V's 16-bit dtype
    vsum: torch.Tensor            # (pool_rows / 64, D) f32
    ysum: torch.Tensor | None     # (pool_rows / 64, r) f32
    u: torch.Tensor | None        # (NBH, r, D) int8
    vr: torch.Tensor | None       # (NBH, D, r) f32

    @property
    def rank(self) -> int:
        return 0 if self.u is None else int(self.u.shape[1])


def check_rank(rank, D):
    if rank not in (0, 16) or rank > D:
        raise ValueError(f"tail rank {rank}: 0 (block rows alone) or 16 (two 8-row operands of the logit matmul)")


def plane_rows(plane, prow, off, D):
    """Pool rows `prow` (any shape) of an int8 K plane in channel order, as
    floats: a row's 16-byte units are stored XOR-swizzled by its page slot
    `off` (broadcastable to `prow`)."""
    nu = min(D // 16, 8)
    sh = 3 - (nu.bit_length() - 1)
    x = (off >> sh) & (nu - 1)
    unit = torch.arange(nu, device=plane.device) ^ x.expand(prow.shape)[..., None]       # logical u <- stored u ^ x
    raw = plane[prow].view(*prow.shape, nu, D // nu)
    idx = unit[..., None].expand(*prow.shape, nu, D // nu)
    return torch.gather(raw, -2, idx).view(*prow.shape, D).float()


def block_sums(x):
    """`(N, S, W)` -> sums over consecutive 64-row blocks `(N, nb, W)` and the
    blocks' row counts `(nb,)` (the last block may be short)."""
    N, S, W = x.shape
    nb = -(-S // TAIL_BLOCK)
    full = x.new_zeros((N, nb * TAIL_BLOCK, W))
    full[:, :S] = x
    cnt = (S - TAIL_BLOCK * torch.arange(nb, device=x.device)).clamp(max=TAIL_BLOCK)
    return full.view(N, nb, TAIL_BLOCK, W).sum(2), cnt


def _minus_block_mean(x):
    sums, cnt = block_sums(x)
    mean = sums / cnt[None, :, None].to(x.dtype)
    return x - mean.repeat_interleave(TAIL_BLOCK, 1)[:, : x.shape[1]]


def moments(kint, ek, vs):
    """The block-centred moment matrices of N row groups over S keys:
    `Kc^T Kc` and `Kc^T Vc` `(N, D, D)` float64, K the kernel's own view of it
    (plane A times its scale, exact in fp32). The products run in fp32 over
    the keys and are a request's own whatever its batch."""
    kc = _minus_block_mean(kint * ek.float()[:, :, None])
    vc = _minus_block_mean(vs.float())
    kt = kc.transpose(1, 2)
    return (kt @ kc).double(), (kt @ vc).double()


def rank_map(kk, kv, rank, lam=1e-3):
    """The rank-`rank` K -> V maps from moment matrices `(N, D, D)`: ridge
    regression (the ridge `lam` times the mean diagonal of `kk`), cut to the
    `rank` leading eigenvectors of the fitted values' Gram matrix
    `M^T kk M`. Returns `u` `(N, rank, D)` int8 (one scale per rank, folded
    into `vr`) and `vr` `(N, D, rank)` f32 (with the 256 of the kernels'
    `ek / 256` folded in). The factorisations are batched calls, whose
    per-matrix results do not depend on the other matrices; a batch of one
    is padded to two, because a single matrix takes another routine
    (reference: kv_cache.py:300-312)."""
    N, D, _ = kk.shape
    if N == 1:
        u, vr = rank_map(kk.expand(2, D, D).contiguous(), kv.expand(2, D, D).contiguous(), rank, lam)
        return u[:1].contiguous(), vr[:1].contiguous()
    eye = torch.eye(D, device=kk.device, dtype=kk.dtype)
    ridge = lam * kk.diagonal(dim1=1, dim2=2).mean(-1)
    chol = torch.linalg.cholesky(kk + (ridge[:, None, None] + 1e-30) * eye)     # a one-key prompt has no moments
    M = torch.cholesky_solve(kv, chol)                                         # (N, D, D): v ~ k M
    gram = M.transpose(1, 2) @ kk @ M
    _, vec = torch.linalg.eigh(0.5 * (gram + gram.transpose(1, 2)))
    basis = vec[:, :, -rank:].flip(-1)                                         # leading direction first
    proj = M @ basis                                                           # (N, D, rank): y = k proj
    step = proj.abs().amax(1).clamp_min(1e-30) / 127.0                         # (N, rank)
    u = torch.round(proj / step[:, None, :]).clamp(-127, 127)
    vr = basis * (step * KBR)[:, None, :]
    return u.transpose(1, 2).to(torch.int8).contiguous(), vr.float().contiguous()


def fit_rank_map(kint, ek, vs, rank, lam=1e-3):
    """`rank_map` of `moments`: `kint` `(N, S, D)` plane A of K as floats
    (integers), `ek` `(N, S)` the keys' scales, `vs` `(N, S, D)` the values."""
    return rank_map(*moments(kint, ek, vs), rank, lam)


def project(kint, ek, u):
    """Every key's projection `(N, S, r)` f32 as the kernels compute it: the
    exact integer product of plane A with `u`, times the key's `ek / 256`,
    rounded once."""
    dots = kint.float() @ u.float().transpose(1, 2)      # integers under 2^24: exact in fp32 in any order
    return dots * (ek.float() * (1.0 / KBR))[:, :, None]


def fit_prompt(kint, ek, v, rank, lam=1e-3, fit=None):
    """N row groups' tail over a prompt of S keys: `(u, vr, vsum, ysum, rows)`
    with the block sums `(N, nb, D)`, `(N, nb, r)` and rows `(N, nb, D)` in
    f32; `u`, `vr` and `ysum` are None at rank 0 (block rows alone). `fit`
    fits the map on the first `fit` keys only; the block rows always cover
    every key."""
    check_rank(rank, v.shape[-1])
    vs = v.float()
    vsum, cnt = block_sums(vs)
    cntf = cnt[None, :, None].float()
    rows = vsum / cntf
    if not rank:
        return None, None, vsum, None, rows
    n = kint.shape[1] if fit is None else fit
    u, vr = fit_rank_map(kint[:, :n], ek[:, :n], vs[:, :n], rank, lam)
    ysum, _ = block_sums(project(kint, ek, u))
    rows = rows - (ysum / cntf) @ vr.transpose(1, 2)
    return u, vr, vsum, ysum, rows


def tail_model(ka, ek, v, *, rank=0, lam=1e-3, fit=None):
    """A contiguous cache's tail, as `prepare_fold_decode(tail=)` takes it: `ka`
    `(NBH, S, D)` plane A as the cache stores it (swizzled by position), `ek`
    `(NBH, S)` the keys' scales, `v` `(NBH, S, D)` the bf16 values; S a multiple
    of 64. Same call as the reference's `cache.tail_model`
    (src/fold_attention/decode/cache.py:307-337); `paged` moves the rows to a
    paged pool's blocks."""
    NBH, S, D = v.shape
    pos = torch.arange(S, device=v.device)
    prow = torch.arange(NBH, device=v.device)[:, None] * S + pos[None, :]
    kint = plane_rows(ka.reshape(NBH * S, D), prow, pos, D)
    u, vr, vsum, ysum, rows = fit_prompt(kint, ek.reshape(NBH, S), v, rank, lam, fit)
    return TailState(rows=rows.to(torch.bfloat16).reshape(-1, D).contiguous(), vsum=vsum.reshape(-1, D).contiguous(),
                     ysum=None if ysum is None else ysum.reshape(-1, rank).contiguous(), u=u, vr=vr)


def paged(tail, page_table, page_size, n_kv_heads, blocks_per_group):
    """A contiguous cache's tail (`tail_model`) for the same cache paged through
    `page_table` `(requests, pages)`: block `j` of row group `(b, h)` moves to
    the pool block of its first key (a page holds whole blocks)."""
    if page_size % TAIL_BLOCK:
        raise ValueError(f"page_size={page_size}: the tail keeps one row per {TAIL_BLOCK} keys, so a page must hold whole blocks")
    B = page_table.shape[0]
    pb = page_size // TAIL_BLOCK
    j = torch.arange(blocks_per_group, device=page_table.device)
    pg = page_table[:, (j // pb).clamp(max=page_table.shape[1] - 1)].long()                   # (B, blocks)
    h = torch.arange(n_kv_heads, device=page_table.device)
    dst = ((pg[:, None, :] * n_kv_heads + h[None, :, None]) * pb + (j % pb)[None, None, :]).reshape(-1)
    n_pool = (int(page_table.max()) + 1) * n_kv_heads * pb

    def move(x):
        if x is None:
            return None
        out = x.new_zeros((n_pool, x.shape[-1]))
        out[dst] = x.reshape(B * n_kv_heads * blocks_per_group, -1)
        return out

    return TailState(rows=move(tail.rows), vsum=move(tail.vsum), ysum=move(tail.ysum), u=tail.u, vr=tail.vr)
