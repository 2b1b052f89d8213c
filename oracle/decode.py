"""Float64 models of the decode. Test infrastructure only.

`coarse_logits`, `mass_model` and `truncated_softmax` restate the models the
reference's tests hold (tests/test_decode.py:902-928, :983-1011, :151-153);
`decode_model` is the kernel's documented function on the cache's own planes
(src/fold_attention/decode/kernel.py:774-870, 1032-1201, 1400-1476): verdicts
from the coarse logit under a given reference Z, plane-B refinement inside the
gates, exact weights, dropped mass re-entering at V's mean.
Works on torch tensors of any device (the GPU tests run it on the GPU to keep
float64 einsums quick); nothing in the shipped package imports it.
"""

from __future__ import annotations

import math

import torch

KBR = 256.0


def unswizzle(plane, slots, head_dim):
    """Undo the cache's XOR swizzle: `plane` (..., S, D) int8 rows stored at
    page slots `slots` (S,)."""
    D = head_dim
    nu = min(D // 16, 8)
    sh = 3 - (nu.bit_length() - 1)
    x = ((slots >> sh) & (nu - 1)).to(plane.device)
    idx = torch.arange(nu, device=plane.device)[None, :] ^ x[:, None]
    v = plane.reshape(*plane.shape[:-1], nu, 16)
    idx = idx.view(*([1] * (v.dim() - 3)), *idx.shape, 1).expand_as(v)
    return torch.gather(v, -2, idx).reshape(plane.shape)


def _fma(a, b, c):
    """a*b + c with one rounding (exact in float64 at these magnitudes)."""
    return (a.double() * b.double() + c.double()).float()


def coarse_logits(qa, qb, eq, ka, ek, z=None):
    """(256 c1 + c2) * eq * (ek/256) for unswizzled plane A `ka` (N, S, D),
    exactly; relative to `z` (N, G) as one fused multiply-add when given."""
    c1 = torch.einsum("ngd,nsd->ngs", qa.double(), ka.double())
    c2 = torch.einsum("ngd,nsd->ngs", qb.double(), ka.double())
    e = eq.float()[..., None] * (ek.float()[:, None, :] * (1.0 / KBR))
    cc = (c1 * 256 + c2).float()
    if z is None:
        return cc * e
    return _fma(cc, e, -z[..., None].expand_as(cc))


def mass_model(s, n, NS=128, TRIM=4):
    """The mass reference for one row group on coarse logits `s` (G, >= n):
    sink and the newest 63 keys exact, stratum centres as samples, the TRIM
    largest samples counted once and the rest extrapolated."""
    npr = -(-(1 + NS + 31) // 64) * 64
    W = npr - 1 - NS
    lo = n - W
    s = s[:, :n].double()
    exact = [0] + [n - r for r in range(1, W + 1) if n - r >= 1]
    strat, prev = [], None
    for j in range(NS):
        k = ((2 * j + 1) * n) // (2 * NS)
        if 1 <= k < lo and k != prev:
            strat.append(k)
        prev = k
    se = s[:, exact]
    ss = s[:, strat]
    M = torch.maximum(se.amax(-1), ss.amax(-1)) if strat else se.amax(-1)
    d = torch.exp2(ss - M[:, None])
    mass = torch.exp2(se - M[:, None]).sum(-1) + d.sum(-1)
    uns = n - len(exact) - len(strat)
    if len(strat) > TRIM and uns > 0:
        rest = d.sum(-1) - d.sort(-1, descending=True).values[:, :TRIM].sum(-1)
        mass = mass + rest * uns / (len(strat) - TRIM)
    return M + torch.log2(mass)


def truncated_softmax(s, z, v, cut):
    p = torch.where(s < cut[..., None], torch.zeros_like(s), torch.exp2(s - z[..., None]))
    return (p @ v) / p.sum(-1, keepdim=True), p


def decode_model(qa, qb, eq, ka, kb, ek, va, vb, v_scale, z, depth, rk, rv, n, vmean=None, reentry=None,
                 visible=None, row_cut=False, sound=False):
    """One row group's decode in float64 on the cache's own (unswizzled)
    planes: `ka`, `kb` (S, D) int8, `ek` (S,), `va` (S, D) float (bf16 values
    or plane A in scale units), `vb` plane B or None. `depth` None keeps every
    key. `reentry` (S, D), instead of `vmean`: where each key's mass re-enters if it is
    dropped (the tail: its block's row plus its projection mapped back, `oracle.tail.reentry`).
    `visible` (G, >= n) bool hides keys from rows (a draft's tree: a hidden key weighs nothing
    in that row and takes no part in its verdicts); `row_cut` lets a gathered key enter only
    the rows that keep it themselves (src/fold_attention/decode/launch.py:602-627, `group_cut`
    off), the others count it as dropped. `sound` tests the coarse logit plus the bound on what
    plane B of K could add, `eq sum_d (128 |qa_d| + |qb_d| / 2) ek / 256` (decode/kernel.py:573-612).
    Returns (out (G, D), den (G,), live count, refined count)."""
    ka, kb, va = ka[:n], kb[:n], va[:n].double()
    ek = ek[:n]
    G = qa.shape[0]
    s1 = coarse_logits(qa[None], qb[None], eq[None], ka[None], ek[None], z[None])[0]  # (G, n) float32
    if visible is not None:
        s1 = torch.where(visible[:, :n].to(s1.device), s1, torch.full_like(s1, float("-inf")))
    s1c = s1
    if sound:
        bound = eq.float() * (qa.float().abs().sum(-1) * 128.0 + qb.float().abs().sum(-1) * 0.5)
        s1c = _fma(bound[:, None].expand_as(s1), (ek.float() * (1.0 / KBR))[None, :].expand_as(s1), s1)
    if depth is None:
        live = torch.ones(n, dtype=torch.bool, device=s1.device)
    else:
        live = (s1c >= -depth).any(0)
    top = s1.amax(0)
    refk = live & (top >= -rk)
    refv = live & (top >= -rv) if vb is not None else torch.zeros_like(live)
    tk = (eq.float()[:, None] * (ek.float()[None, :] * (1.0 / KBR))).double()
    c3a = torch.einsum("gd,sd->gs", qa.double(), kb.double())
    c3b = torch.einsum("gd,sd->gs", qb.double(), kb.double())
    s = s1.double() + torch.where(refk[None], (c3a + c3b / KBR) * tk, torch.zeros_like(tk))
    e = torch.exp2(s)
    keeps = live[None].expand_as(e)
    if row_cut and depth is not None:
        keeps = keeps & (s1c >= -depth)
    w = torch.where(keeps, e, torch.zeros_like(e))
    m = torch.where(keeps, torch.zeros_like(e), e).sum(-1)
    vt = va
    if vb is not None:
        vt = va + torch.where(refv[:, None], vb[:n].double() / 8.0, torch.zeros_like(va))
    num = w @ vt
    if vmean is not None and depth is not None:
        num = num + m[:, None] * vmean.double()[None, :]
    if reentry is not None and depth is not None:
        num = num + torch.where(keeps, torch.zeros_like(e), e) @ reentry[:n].double().to(e.device)
    den = w.sum(-1) + m
    return num * v_scale / den[:, None], den, int(live.sum()), int(refk.sum())


def attend_fp32(q, k, v):
    """Dense softmax attention of one query token per row: q (G, D), k, v
    (S, D); FP32 inputs, float64 accumulation (the end-to-end error reference:
    tests/test_kv_cache.py:87-102, benchmarks/harness/baselines.py:68-86)."""
    s = (q.double() @ k.double().T) / math.sqrt(q.shape[-1])
    return torch.softmax(s, -1) @ v.double()
