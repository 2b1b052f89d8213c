"""How one backward call's work is cut up on B200.

A work item is one key block of one (request, KV head), `subgroup` of the
group's query heads walked in turn, and a run of `record` query blocks (or
every block that can see the key block). The tcgen05 main loop runs one
persistent CTA per SM; the CTAs claim items from a device-built list, longest
first inside L2-sized sections (csrc/bwd_sm100.cu: `bwd_work_list_kernel`,
the claim loop of the producer warp).

With the whole group and the whole range (`Plan(G, 0)`) a key block's dK and
dV never leave one CTA. That is the fastest exit, and both headline shapes
take it. It stops paying when the items are too few or too long for 148 SMs:
one item then outlasts an SM's fair share of the work and the launch ends on
it. Such calls cut the group (`subgroup < G`) or the query range (`record`),
and a key block's items meet on integer grids: each rounds its dK / dV sums
onto the (request, KV head)'s grid and adds them to an int64 (dV: int32 for
short groups) accumulator that the postprocess converts. The reference
chooses between three exits from H100 measurements
(src/fold_attention/backward/plan.py:58-118: private, fp32 combine, integer
fold); here every plan that crosses CTAs folds.

What a plan may depend on: a dense call's plan reads its whole shape, batch
included (as the reference's does, plan.py:74-90), so dK / dV bits may differ
between batch sizes that plan differently, while dQ's never do; a packed
call's plan reads head counts only, so a sequence's gradients are the same
bits whatever it is packed with.
"""

from __future__ import annotations

from dataclasses import dataclass

SMS = 148           # B200
TILE = 128          # query and key block of the tcgen05 main loop
MIN_ITEM = 8        # tiles: below this an item's fixed costs (K, V loads, the dK / dV exit) dominate
PRIVATE_SHARE = 0.6 # a whole-group item may be this much of one SM's share of the tiles (B1 H32/8 S8192: 0.57,
                    # where Plan(4, 0) measured 1005 TFLOP/s against 900 for Plan(2, 0))


@dataclass(frozen=True)
class TileConfig:
    tile_m: int
    tile_n: int


def tile_config(head_dim: int, kernel: str = "auto") -> TileConfig:
    """Query x key block of the kernel that serves `head_dim`."""
    if head_dim not in (64, 96, 128):
        raise NotImplementedError(f"head_dim {head_dim}: 64, 96 and 128 are supported")
    if kernel == "sm100" or (kernel == "auto" and head_dim == 128):
        return TileConfig(TILE, TILE)
    return TileConfig(64, 64)


@dataclass(frozen=True)
class Plan:
    """`subgroup` query heads per work item (a divisor of the group; the whole
    group keeps dK / dV private to a CTA) and `record`, the query blocks per
    item (0: the whole range)."""

    subgroup: int
    record: int = 0

    def folds(self, G: int) -> bool:
        """Whether a key block's dK / dV are summed across work items."""
        return self.subgroup < G or self.record > 0


def _divisors_desc(G):
    return [g for g in range(G, 0, -1) if G % g == 0]


def plan_dense(B, H, H_KV, S, D, causal, cfg: TileConfig | None = None, sms: int = SMS) -> Plan:
    """The largest work items that still balance over `sms` SMs.

    The longest item (key block 0 under a causal mask: it sees every query
    block) should be at most half of one SM's fair share of the tiles, or the
    launch ends waiting for it; a whole group may take `PRIVATE_SHARE` of it,
    because its dK / dV never leave the CTA. Whole groups first; then smaller subgroups;
    then, for a single head still too long (few heads, long sequences),
    records of the query range.
    """
    G = H // H_KV
    if cfg is not None and cfg.tile_n != TILE:
        return Plan(G, 0)        # the mma.sync main loop: whole groups, whole ranges
    nb = -(-S // TILE)
    tiles = B * H * (nb * (nb + 1) // 2 if causal else nb * nb)
    cap = tiles / sms / 2
    if cap < MIN_ITEM:
        return Plan(G, 0)        # a small call: nothing to balance, and folding has fixed costs of its own
    if nb * G <= PRIVATE_SHARE * tiles / sms:
        # whole groups still fit: the private exit (no integer fold, no dK / dV postprocess) is worth
        # more than finer items as long as the longest-first list can hide the longest one
        return Plan(G, 0)
    for sub in _divisors_desc(G):
        if nb * sub <= cap:
            return Plan(sub, 0)
    record = max(MIN_ITEM // 2, int(cap))
    return Plan(1, record if record < nb else 0)


def plan_varlen(H, H_KV, cfg: TileConfig | None = None) -> Plan:
    """A packed call's plan, from head counts alone: a sequence's bits must
    not depend on its neighbours. Groups of more than four heads are walked
    four heads at a time (a long sequence's whole-group items would be the
    launch's tail); smaller groups stay whole."""
    G = H // H_KV
    if cfg is not None and cfg.tile_n != TILE:
        return Plan(G, 0)
    sub = G
    while sub > 4 and sub % 2 == 0:
        sub //= 2
    return Plan(sub, 0)


def work_items(B, H, H_KV, S, plan: Plan) -> int:
    """Entries of the device work list (empty ones included: one per key block
    up to the longest sequence, per record)."""
    G = H // H_KV
    nb = -(-S // TILE)
    nrec = -(-nb // plan.record) if plan.record else 1
    return B * H_KV * (G // plan.subgroup) * nb * nrec
