"""Draft row layouts (host logic, no GPU) against the reference's own `decode/rows.py` outputs
(tests/golden/rows_layouts.npz, made by make_rows_golden.py)."""

import os

import numpy as np
import pytest
import torch

from fold_attention_b200.decode.rows import draft_mask, pack_rows, pack_tree, unpack_rows

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "rows_layouts.npz"))


@pytest.mark.parametrize("name", ["chain4", "fork6", "two_roots", "wide8"])
def test_trees(name):
    par = G[f"parents_{name}"].tolist()
    m = draft_mask(par)
    assert np.array_equal(m.numpy(), G[f"mask_{name}"])
    q_len = len(par)
    Gr = q_len * (8 // q_len if q_len <= 8 else 1)
    assert np.array_equal(pack_tree(m, False, q_len, Gr, 3, "cpu").numpy(), G[f"words_{name}"])
    assert np.array_equal(pack_tree(m[None].expand(3, -1, -1), False, q_len, Gr, 3, "cpu").numpy(), G[f"words_{name}"])


@pytest.mark.parametrize("q_len,Gr", [(2, 8), (4, 8), (8, 8), (32, 32)])
def test_chains(q_len, Gr):
    w = pack_tree(None, True, q_len, Gr, 2, "cpu")
    assert w.dtype == torch.int32 and np.array_equal(w.numpy(), G[f"causal_{q_len}_{Gr}"])
    assert np.array_equal(w.numpy(), pack_tree(draft_mask([-1] + list(range(q_len - 1))), False, q_len, Gr, 2, "cpu").numpy())


def test_rows_round_trip():
    x = torch.from_numpy(G["rows_in"])
    assert np.array_equal(pack_rows(x, 2, 2).numpy(), G["rows_packed_hkv2"])
    assert np.array_equal(pack_rows(x, 4, 2).numpy(), G["rows_packed_hkv4"])
    assert torch.equal(unpack_rows(pack_rows(x, 2, 2), 2, 2), x)
    assert torch.equal(unpack_rows(pack_rows(x, 4, 2), 4, 2), x)


def test_refusals():
    with pytest.raises(ValueError, match="parent"):
        draft_mask([-1, 2, 0])
    with pytest.raises(ValueError, match="diagonal"):
        pack_tree(torch.tensor([[True, False], [True, False]]), False, 2, 8, 1, "cpu")
    with pytest.raises(ValueError, match="at most 32"):
        pack_tree(None, True, 33, 33, 1, "cpu")
    with pytest.raises(ValueError, match="draft length"):
        pack_rows(torch.zeros(2, 3, 8, 4), 2, 2)
    with pytest.raises(ValueError, match="multiple of n_kv_heads"):
        pack_rows(torch.zeros(2, 2, 7, 4), 2, 2)
