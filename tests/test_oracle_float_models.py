"""The oracle's float models against outputs of the reference's own functions.

`tests/golden/float_models.npz` was written by `tests/golden/make_float_golden.py`, which ran the
reference's text of `reference_grads` (benchmarks/harness/training.py:124-164) and of the decode
test models `_coarse`, `_mass_model`, `_ref`, `_s16` (tests/test_decode.py:133-153, 902-928,
983-1011) on seeded CPU inputs. The oracle restates them; here it must reproduce them: bit for
bit where the arithmetic is exact or a single rounding (coarse logits), to fp32/fp64 rounding of
a different summation order elsewhere (tolerances written at each check)."""

import math
import os

import numpy as np
import pytest
import torch

from oracle import backward as ob
from oracle import decode as od

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "float_models.npz"))


def t(name):
    return torch.from_numpy(G[name])


@pytest.mark.parametrize("tag", ["mha", "gqa", "full"])
def test_reference_grads_are_the_harness_fp32_gradients(tag):
    q, k, v, do = (t(f"train_{tag}_{n}").bfloat16() for n in ("q", "k", "v", "do"))
    causal = bool(G[f"train_{tag}_causal"])
    for b in range(q.shape[0]):
        got64 = ob.reference_grads(q[b], k[b], v[b], do[b], causal=causal)
        got32 = ob.reference_grads(q[b], k[b], v[b], do[b], causal=causal, dtype=torch.float32)
        for name, a64, a32 in zip(("dq", "dk", "dv"), got64, got32):
            want = t(f"train_{tag}_{name}")[b]
            # the harness sums in fp32 head by head; fp64 autograd is the tighter statement of the same function
            assert ob.rel_l2(want, a64) < 2e-6, (tag, name)
            assert ob.rel_l2(a32, want) < 2e-6, (tag, name)


def test_reference_grads_packed_sequences():
    q, k, v, do = (t(f"train_packed_{n}").bfloat16() for n in ("q", "k", "v", "do"))
    at = 0
    for n in G["train_packed_lens"].tolist():
        sl = slice(at, at + n)
        got = ob.reference_grads(q[sl], k[sl], v[sl], do[sl])
        for name, a in zip(("dq", "dk", "dv"), got):
            assert ob.rel_l2(t(f"train_packed_{name}")[sl], a) < 2e-6, name
        at += n


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_decode_models_are_the_reference_tests_models(tag):
    qa, qb, eq = t(f"dec_{tag}_qa"), t(f"dec_{tag}_qb"), t(f"dec_{tag}_eq")
    ka, kb = t(f"dec_{tag}_ka_unswizzled"), t(f"dec_{tag}_kb_unswizzled")
    ek, z, v = t(f"dec_{tag}_ek"), t(f"dec_{tag}_z"), t(f"dec_{tag}_v")
    S = ka.shape[1]
    # coarse logits: exact integer sums, one rounding (and one fused multiply-add under Z): the same bits
    sc = od.coarse_logits(qa, qb, eq, ka, ek)
    assert torch.equal(sc, t(f"dec_{tag}_coarse"))
    assert torch.equal(od.coarse_logits(qa, qb, eq, ka, ek, z), t(f"dec_{tag}_coarse_z"))
    # the mass estimate: the same float64 expression
    for n, key in ((S, "mass"), (min(S, 50), "mass50")):
        got = torch.stack([od.mass_model(sc[b], n) for b in range(sc.shape[0])])
        assert torch.equal(got, t(f"dec_{tag}_{key}"))
    # the four-term logit from the planes the oracle's decode model uses, against `_s16` (fp32 einsums
    # there, float64 here: fp32 rounding of sums of ~D products)
    tk = eq.double()[..., None] * (ek.double()[:, None, :] / 256.0)
    four = (256.0 * torch.einsum("ngd,nsd->ngs", qa.double(), ka.double()) + torch.einsum("ngd,nsd->ngs", qb.double(), ka.double())
            + torch.einsum("ngd,nsd->ngs", qa.double(), kb.double()) + torch.einsum("ngd,nsd->ngs", qb.double(), kb.double()) / 256.0) * tk
    s16 = t(f"dec_{tag}_s16")
    assert float((four - s16.double()).abs().max()) < 1e-3 * max(1.0, float(s16.abs().max())) * 2.0**-10
    # truncated softmax on the reference's own logits
    cut = t(f"dec_{tag}_cut")
    out, p = od.truncated_softmax(s16.double(), z.double(), v.double(), cut.double())
    assert torch.equal(out, t(f"dec_{tag}_ref_out"))
    assert torch.equal(p.sum(-1), t(f"dec_{tag}_ref_psum"))


def test_the_decode_model_agrees_with_the_truncated_softmax_when_every_key_is_refined():
    """`decode_model` with wide-open refine gates and no dropped-mass re-entry is `_ref` on the
    four-term logit: keys under the cut carry zero weight in the numerator and only their mass
    in the denominator."""
    tag = "a"
    qa, qb, eq = t(f"dec_{tag}_qa"), t(f"dec_{tag}_qb"), t(f"dec_{tag}_eq")
    ka, kb = t(f"dec_{tag}_ka_unswizzled"), t(f"dec_{tag}_kb_unswizzled")
    ek, z, v = t(f"dec_{tag}_ek"), t(f"dec_{tag}_z"), t(f"dec_{tag}_v")
    b, S = 0, ka.shape[1]
    out, den, live, refined = od.decode_model(qa[b], qb[b], eq[b], ka[b], kb[b], ek[b], v[b], None, 1.0, z[b],
                                              None, 1e9, 1e9, S)
    assert live == S and refined == S
    s16 = t(f"dec_{tag}_s16")[b].double()
    w = torch.exp2(s16 - z[b].double()[:, None])
    want = (w @ v[b].double()) / w.sum(-1, keepdim=True)
    assert float((out - want).abs().max()) < 1e-4 * float(want.abs().max())
    assert math.isfinite(float(den.sum()))
