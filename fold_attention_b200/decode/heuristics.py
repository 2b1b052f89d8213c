"""The rules that choose a decode build for a batch.

Two kinds of rule live here. The accuracy-affecting defaults (`refine_for`,
`refine_bands_for`, `weight_terms_for`) are the reference's published gates
(src/fold_attention/decode/heuristics.py:70-190), kept so a cache built with
default arguments computes the same function. The scheduling rule
(`pick_split`) is B200's own: the reference's is a fit to H100 measurements.
"""

from __future__ import annotations

# (refine_k by context band) for a dense bf16 V, keyed by (head-dim class, group class)
_DENSE_K = {
    (128, 1): (12, 12, 12), (128, 4): (10, 10, 12), (128, 8): (10, 10, 12), (128, 16): (10, 12, 12),
    (64, 1): (12, 12, 12), (64, 4): (10, 10, 10), (64, 8): (12, 12, 10),
}
# ((refine_k, refine_v) by context band) for a dense 8-bit V
_DENSE_V8 = {
    (128, 1): ((10, 12),) * 3, (128, 4): ((10, 10),) * 3,
    (128, 8): ((10, 10), (10, 10), (10, 12)), (128, 16): ((10, 10), (10, 12), (10, 12)),
    (64, 1): ((10, 10), (10, 10), (12, 8)), (64, 4): ((10, 8), (10, 10), (10, 8)),
    (64, 8): ((10, 10),) * 3,
}
# lower edges of the depth steps the truncated gates were measured at
_DEPTH_STEPS = (11.0, 12.5, 13.5, 15.0, 17.0, 19.0)
_TRUNC_K = {
    (128, 1): (10, 8, 8, 8, 10, 12, 12), (128, 4): (10, 10, 10, 8, 10, 12, 12),
    (128, 8): (10, 8, 8, 8, 10, 12, 12), (128, 16): (6, 10, 10, 10, 10, 12, 12),
    (64, 1): (8, 10, 10, 10, 10, 12, 12), (64, 4): (6, 8, 8, 8, 10, 10, 10),
    (64, 8): (10, 10, 10, 10, 10, 12, 12),
}
_TRUNC_V8 = {
    (128, 1): ((8, 10), (8, 10), (6, 8), (6, 8), (10, 10), (12, 10), (12, 10)),
    (128, 4): ((8, 10), (6, 8), (6, 8), (6, 8), (10, 10), (10, 10), (10, 10)),
    (128, 8): ((8, 10), (8, 12), (8, 10), (6, 8), (10, 12), (10, 10), (12, 10)),
    (128, 16): ((8, 10), (6, 12), (8, 6), (8, 6), (8, 8), (10, 12), (10, 12)),
    (64, 1): ((6, 6), (6, 6), (6, 6), (10, 10), (10, 10), (10, 10), (12, 10)),
    (64, 4): ((8, 6), (8, 6), (8, 6), (8, 6), (10, 10), (8, 8), (10, 10)),
    (64, 8): ((8, 6), (8, 6), (8, 6), (8, 6), (10, 10), (10, 10), (10, 10)),
}
# the dense bands' edges: halfway in log2 between 4K and 8K, and 16K and 32K
_BAND_EDGES = (5793, 23170)


def _classes(head_dim, group):
    dk = 64 if head_dim <= 64 else 128
    gc = 1 if group <= 2 else 4 if group <= 4 else 8 if group <= 8 or dk == 64 else 16
    return dk, gc


def refine_for(depth, v8=False, *, seq_len, head_dim=128, group=8, tail=True):
    """`(refine_k, refine_v)`: the depths below a row's log-sum-exp inside
    which K's and V's second planes are read (reference heuristics.py:125-157).
    `refine_v` is unused on a bf16 V."""
    key = _classes(head_dim, group)
    if depth is None:
        band = sum(seq_len > e for e in _BAND_EDGES)
        if v8:
            rk, rv = _DENSE_V8[key][band]
            return float(rk), float(rv)
        return float(_DENSE_K[key][band]), 8.0
    step = sum(depth >= e for e in _DEPTH_STEPS)
    if v8:
        rk, rv = _TRUNC_V8[key][step]
        return float(rk), float(rv)
    if depth < 15.0 and not tail:
        return 10.0, 8.0
    return float(_TRUNC_K[key][step]), 8.0


def refine_bands_for(v8=False, *, head_dim=128, group=8):
    """The dense gates' length bands `(edge0, edge1, rk1, rk2, rv1, rv2)`; the
    kernel picks a row group's band from that request's own length, so its
    bits do not depend on its batch (reference heuristics.py:160-175)."""
    (rk1, rv1), (rk2, rv2) = (
        refine_for(None, v8, seq_len=e + 1, head_dim=head_dim, group=group) for e in _BAND_EDGES
    )
    return (float(_BAND_EDGES[0]), float(_BAND_EDGES[1]), rk1, rk2, rv1, rv2)


def weight_terms_for(depth):
    """bf16 terms a weight is carried in: two (value and rounding error)
    dense and from depth 15 up, one below (reference heuristics.py:178-190)."""
    if depth is None:
        return 2
    return 2 if depth >= 15.0 else 1


def tail_rank_for(D, G, v8):
    """The reference's default decode-tail rank (heuristics.py:193-208); only
    -1 (no tail) is built here."""
    if v8:
        return -1
    if G <= 16:
        return 16
    return 0 if D < 128 else -1


def pick_split(n_groups, seq_len, *, max_len=None, sms=148, resident=3):
    """CTAs per row group on B200: enough CTAs for two waves of `resident`
    per SM, but at least eight 64-key tiles each so the pipeline fills.
    `resident` is 3 for the warp-level kernel; the tcgen05 kernel holds one
    CTA an SM and pays a fixed cost per CTA, and measured best at about three
    waves in all (`resident=1.5`: config 5's shape at 32 / 64 / 128 requests
    takes 550 / 1031 / 1892 us a step with 2 / 1 / 1 CTAs a row group, against
    705 with 1 at 32 requests and 1058 with 2 at 64)."""
    want = -int(-2 * sms * resident // max(1, n_groups))
    cap = max(1, seq_len // 512)
    return int(max(1, min(want, cap, 64)))
