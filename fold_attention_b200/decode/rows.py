"""Query-row layouts beyond one token per request: a draft's rows and its tree.

A row group is the query rows that share one KV head of one request. Under a
draft of `q_len` positions it holds `G // q_len` query heads at `q_len`
positions each, row `g * q_len + t`; the draft's own keys are the cache's last
`q_len`, and which of them a row sees is one int32 word per row (bit `j`: node
`j`). Same layouts and names as the reference's `decode/rows.py:19-122`
(`draft_mask`, `pack_tree`, `pack_rows`, `unpack_rows`).
"""

from __future__ import annotations

import torch


def draft_mask(parents) -> torch.Tensor:
    """`(q_len, q_len)` bool: node `i` sees node `j` when `j` is `i` or one of
    its ancestors. `parents[i]` is node `i`'s parent (-1 for a root) and must
    come before it: a parent is in the cache before its child. The chain
    `[-1, 0, 1, ...]` is the causal mask."""
    par = [int(x) for x in parents]
    n = len(par)
    seen = torch.eye(n, dtype=torch.bool)
    for i, up in enumerate(par):
        if up >= i:
            raise ValueError(f"node {i} has parent {up}: a parent is written to the cache before its child, so its index is lower")
        if up >= 0:
            seen[i] |= seen[up]       # the parent's row is complete: parents come first
    return seen


def pack_tree(mask, causal, q_len, G, NBH, device) -> torch.Tensor:
    """`(NBH, G)` int32 visibility words for rows `g * q_len + t`, from
    `causal` (row `t` sees nodes `0..t`) or a `(q_len, q_len)` /
    `(NBH, q_len, q_len)` bool `mask`."""
    if q_len > 32:
        raise ValueError(f"draft_len={q_len}: a row's visibility is one int32, so at most 32 nodes")
    if causal:
        m = torch.tril(torch.ones(q_len, q_len, dtype=torch.bool))[None]
    else:
        m = torch.as_tensor(mask)
        m = (m if m.dtype == torch.bool else m != 0)
        if m.dim() == 2:
            m = m[None]
        if m.dim() != 3 or tuple(m.shape[-2:]) != (q_len, q_len) or m.shape[0] not in (1, NBH):
            raise ValueError(f"mask is ({q_len}, {q_len}) or ({NBH}, {q_len}, {q_len}) bool, got {tuple(m.shape)}")
        if not bool(torch.diagonal(m, dim1=-2, dim2=-1).all()):
            raise ValueError("a draft node sees its own key: the mask's diagonal must be set (a row without it has an empty softmax)")
    weights = torch.ones(q_len, dtype=torch.int64) << torch.arange(q_len)
    words = (m.to(torch.int64).cpu() * weights).sum(-1)                  # (1 or NBH, q_len), values < 2^32
    words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    return words.repeat(1, G // q_len).expand(NBH, G).contiguous().to(device)


def pack_rows(x, n_kv_heads, q_len=1) -> torch.Tensor:
    """`(B, q_len, H_q, ...)` to the kernels' `(B * H_KV, G, ...)` with row
    `g * q_len + t` the `g`-th query head of its KV head at position `t`."""
    B, T, H = x.shape[:3]
    rest = tuple(x.shape[3:])
    if T != q_len:
        raise ValueError(f"axis 1 is the draft length: expected {q_len}, got {T}")
    if H % n_kv_heads:
        raise ValueError(f"H_q={H} is not a multiple of n_kv_heads={n_kv_heads}")
    g0 = H // n_kv_heads
    y = x.reshape(B, T, n_kv_heads, g0, *rest).transpose(1, 2).transpose(2, 3)      # (B, H_KV, g0, T, ...)
    return y.reshape(B * n_kv_heads, g0 * T, *rest).contiguous()


def unpack_rows(x, n_kv_heads, q_len=1) -> torch.Tensor:
    """The inverse of `pack_rows`: `(NBH, G, ...)` to `(B, q_len, H_q, ...)`."""
    NBH, G = x.shape[:2]
    rest = tuple(x.shape[2:])
    if G % q_len or NBH % n_kv_heads:
        raise ValueError(f"G={G} is {G // max(q_len, 1)} heads x q_len={q_len} and NBH={NBH} requests x n_kv_heads={n_kv_heads}")
    B, g0 = NBH // n_kv_heads, G // q_len
    y = x.reshape(B, n_kv_heads, g0, q_len, *rest).transpose(2, 3).transpose(1, 2)   # (B, T, H_KV, g0, ...)
    return y.reshape(B, q_len, n_kv_heads * g0, *rest).contiguous()
