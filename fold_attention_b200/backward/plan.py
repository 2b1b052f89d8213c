"""How one backward call's work is cut up on B200.

The reference's planner (src/fold_attention/backward/plan.py) chooses between
private, combined and folded dK/dV per shape from H100 measurements. Here the
decomposition is fixed: a work tile is one key block of one (request, KV
head) and walks the whole GQA group and every query block that can see it,
so dK/dV stay private to a CTA and their bits follow from the request alone;
dQ is an integer-grid reduction. Nothing in a plan depends on the batch, so a
request's gradients are the same bits alone and packed with others, dense or
varlen.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class TileConfig:
    tile_m: int
    tile_n: int


def tile_config(head_dim: int, kernel: str = "auto") -> TileConfig:
    """Query x key block of the kernel that serves `head_dim`."""
    if head_dim not in (64, 96, 128):
        raise NotImplementedError(f"head_dim {head_dim}: 64, 96 and 128 are supported")
    if kernel == "sm100":
        return TileConfig(128, 128)
    return TileConfig(64, 64)


@dataclass(frozen=True)
class Plan:
    """`subgroup` query heads per work tile (always the whole group here) and
    the canonical record width (always 0: the whole query range)."""

    subgroup: int
    record: int = 0


def plan_dense(B, H, H_KV, S, D, causal, cfg: TileConfig | None = None) -> Plan:
    return Plan(subgroup=H // H_KV, record=0)


def plan_varlen(H, H_KV, cfg: TileConfig | None = None) -> Plan:
    return Plan(subgroup=H // H_KV, record=0)
