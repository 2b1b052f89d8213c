"""The backward oracle's own known answers (CPU)."""

import numpy as np
import torch

from oracle import backward as ob


def test_grid_exponent_known_answers():
    # bound 1.0 -> widened to 1.015625 -> ceil(log2) = 1 -> 30 - 1
    assert ob.pow2_scale_exp(1.0, 30) == 29
    # a bound just under a power of two after widening stays in the binade
    assert ob.pow2_scale_exp(0.98, 30) == 30
    assert ob.pow2_scale_exp(0.0, 30) == 100
    assert ob.pow2_scale_exp(1e-38, 30) == 100
    assert ob.pow2_scale_exp(3e38, 30) == -98
    assert ob.pow2_scale_exp(2.0**40, 30) == 30 - 41
    assert ob.root_d(64) == 8.0 and ob.root_d(96) == 16.0 and ob.root_d(128) == 16.0


def test_grid_bound_holds_on_random_inputs():
    """|dQ / scale| * 2^s stays under 2^30 with the documented bound."""
    torch.manual_seed(0)
    S, H, D = 96, 2, 64
    q, k, v, do = (torch.randn(S, H, D).bfloat16() for _ in range(4))
    o, _ = ob.reference_forward(q, k, v)
    dq, _, _ = ob.reference_grads(q, k, v, do)
    st = ob.stats(q, k, v, o.bfloat16(), do, 1)
    for h in range(H):
        s = ob.dq_scale_exp(*st[h], D)
        assert float(dq[:, h].abs().max()) * D**0.5 * 2.0**s < 2.0**30
        assert float(dq[:, h].abs().max()) * D**0.5 * 2.0**s > 2.0**12  # not wastefully coarse


def test_reference_grads_match_fp32_twin():
    torch.manual_seed(1)
    S, H, HKV, D = 64, 4, 2, 32
    q = torch.randn(S, H, D)
    k, v = torch.randn(S, HKV, D), torch.randn(S, HKV, D)
    do = torch.randn(S, H, D)
    a = ob.reference_grads(q, k, v, do)
    b = ob.reference_grads(q, k, v, do, dtype=torch.float32)
    for x, y in zip(a, b):
        assert ob.rel_l2(y, x) < 1e-5
