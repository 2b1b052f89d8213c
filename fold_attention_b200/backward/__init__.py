"""The deterministic attention backward (host side)."""

from .launch import BackwardLaunch, attention_forward, prepare_backward
from .plan import Plan, TileConfig, plan_dense, plan_varlen, tile_config

__all__ = [
    "BackwardLaunch",
    "Plan",
    "TileConfig",
    "attention_forward",
    "plan_dense",
    "plan_varlen",
    "prepare_backward",
    "tile_config",
]
