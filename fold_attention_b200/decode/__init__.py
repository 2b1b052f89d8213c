"""Quantised paged-KV decode (host side): the kernel-level entry and the row
layouts, under the reference's names where it has them
(src/fold_attention/decode/__init__.py)."""

from .heuristics import pick_split
from .launch import SharedPrefix, capture_decode, fold_decode, mass_z, prepare_fold_decode
from .rows import draft_mask, pack_rows, pack_tree, unpack_rows
from .tail import TailState, tail_model

__all__ = [
    "SharedPrefix",
    "TailState",
    "capture_decode",
    "draft_mask",
    "fold_decode",
    "mass_z",
    "pack_rows",
    "pack_tree",
    "pick_split",
    "prepare_fold_decode",
    "tail_model",
    "unpack_rows",
]
