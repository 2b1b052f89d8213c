"""Generate tests/golden/rows_layouts.npz from the reference's own `decode/rows.py`.

    python tests/golden/make_rows_golden.py /path/to/reference

The file is pure torch and is imported by path. Stored: `draft_mask` of a few trees,
`pack_tree` words for chains and trees, and `pack_rows` of a seeded tensor.
"""

from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch


def main(root):
    spec = importlib.util.spec_from_file_location("ref_rows", os.path.join(root, "src", "fold_attention", "decode", "rows.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    trees = dict(chain4=[-1, 0, 1, 2], fork6=[-1, 0, 0, 1, 1, 2], two_roots=[-1, -1, 0, 1], wide8=[-1, 0, 1, 1, 0, 4, 4, 2])
    for name, par in trees.items():
        m = ref.draft_mask(par)
        out[f"mask_{name}"] = m.numpy()
        out[f"parents_{name}"] = np.array(par)
        q_len = len(par)
        G = q_len * (8 // q_len if q_len <= 8 else 1)
        out[f"words_{name}"] = ref.pack_tree(m, False, q_len, G, 3, "cpu").numpy()
    for q_len, G in ((2, 8), (4, 8), (8, 8), (32, 32)):
        out[f"causal_{q_len}_{G}"] = ref.pack_tree(None, True, q_len, G, 2, "cpu").numpy()
    g = torch.Generator().manual_seed(9)
    x = torch.randn(3, 2, 8, 5, generator=g)
    out["rows_in"] = x.numpy()
    out["rows_packed_hkv2"] = ref.pack_rows(x, 2, 2).numpy()
    out["rows_packed_hkv4"] = ref.pack_rows(x, 4, 2).numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "rows_layouts.npz")
    np.savez_compressed(path, **out)
    print(path, sorted(out))


if __name__ == "__main__":
    main(sys.argv[1])
