"""The decode tail's fit: the oracle's restatement and the package's own fit against the
reference's `tail_model` outputs (tests/golden/tail_model.npz, made by make_tail_golden.py).

The fit defines `u` and `vr` up to a sign per rank (and, where two directions carry nearly the
same energy, a rotation between them), so the comparison is on what the decode uses: the
effective K -> V map `vr u`, each key's re-entry point, and the block rows.
"""

import os

import numpy as np
import pytest
import torch

from oracle import tail as otail
from oracle.decode import unswizzle

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "tail_model.npz"))
CASES = [("d64", 64), ("d128", 128)]


def _inputs(tag, D):
    ka = torch.from_numpy(G[f"{tag}_ka"])
    S = ka.shape[1]
    kint = unswizzle(ka, torch.arange(S), D).numpy().astype(np.float64)
    return kint, G[f"{tag}_ek"], G[f"{tag}_v"]


def _rel(a, b):
    return np.linalg.norm(a - b) / np.linalg.norm(b)


@pytest.mark.parametrize("tag,D", CASES)
def test_oracle_rank0_rows_are_the_block_means(tag, D):
    kint, ek, v = _inputs(tag, D)
    for n in range(kint.shape[0]):
        rows = otail.tail_fit(kint[n], ek[n], v[n], 0)[3]
        ref = G[f"{tag}_r0_vblk"][n]
        assert np.abs(rows - ref).max() <= 2.0 ** -8 * np.abs(ref).max()      # the reference stores bf16


@pytest.mark.parametrize("tag,D", CASES)
def test_oracle_rank16_matches_the_reference_model(tag, D):
    kint, ek, v = _inputs(tag, D)
    for n in range(kint.shape[0]):
        u, vr, y, rows = otail.tail_fit(kint[n], ek[n], v[n], 16)
        ur, vrr = G[f"{tag}_r16_u"][n].astype(np.float64), G[f"{tag}_r16_vr"][n].astype(np.float64)
        assert u.dtype == np.int8 and np.abs(u).max() == 127
        assert _rel(vr @ u, vrr @ ur) < 2e-2
        mine = otail.reentry(kint[n], ek[n], u, vr, rows)
        ref = otail.reentry(kint[n], ek[n], ur, vrr, G[f"{tag}_r16_vblk"][n])
        assert _rel(mine, ref) < 1e-2
        # and the model explains V: the rank's re-entry points are far closer to V than the block means
        blk = otail.reentry(kint[n], ek[n], None, None, otail.block_mean(v[n].astype(np.float64)))
        assert np.linalg.norm(mine - v[n]) < 0.5 * np.linalg.norm(blk - v[n])


@pytest.mark.parametrize("tag,D", CASES)
def test_package_fit_matches_the_reference_model(tag, D):
    from fold_attention_b200.decode import tail as ptail

    kint, ek, v = _inputs(tag, D)
    kt, et, vt = torch.from_numpy(kint).float(), torch.from_numpy(ek).bfloat16(), torch.from_numpy(v).bfloat16()
    u, vr, vsum, ysum, rows = ptail.fit_prompt(kt, et, vt, 16)
    y = ptail.project(kt, et, u)
    for n in range(kint.shape[0]):
        ur, vrr = G[f"{tag}_r16_u"][n].astype(np.float64), G[f"{tag}_r16_vr"][n].astype(np.float64)
        assert _rel(vr[n].double().numpy() @ u[n].double().numpy(), vrr @ ur) < 2e-2
        mine = otail.reentry(kint[n], ek[n], u[n].numpy(), vr[n].numpy(), rows[n].numpy())
        ref = otail.reentry(kint[n], ek[n], ur, vrr, G[f"{tag}_r16_vblk"][n])
        assert _rel(mine, ref) < 1e-2
        # the package's projection is an exact integer rounded once by the key's scale: the bits the oracle states
        yo = (kint[n] @ u[n].double().numpy().T).astype(np.float32) * (ek[n].astype(np.float32) * np.float32(1 / 256))[:, None]
        assert np.array_equal(y[n].numpy(), yo)
        fit = otail.tail_fit(kint[n], ek[n], v[n], 16)
        assert _rel(mine, otail.reentry(kint[n], ek[n], fit[0], fit[1], fit[3])) < 1e-2
    r0 = ptail.fit_prompt(kt, et, vt, 0)
    assert r0[0] is None and r0[3] is None
    assert np.abs(r0[4].numpy() - G[f"{tag}_r0_vblk"]).max() <= 2.0 ** -8 * np.abs(G[f"{tag}_r0_vblk"]).max()


def test_block_sums_and_a_short_last_block():
    from fold_attention_b200.decode import tail as ptail

    x = torch.arange(130 * 3, dtype=torch.float32).view(1, 130, 3)
    sums, cnt = ptail.block_sums(x)
    assert cnt.tolist() == [64, 64, 2]
    assert torch.equal(sums[0, 2], x[0, 128:].sum(0))
    assert np.allclose(otail.block_mean(x[0].numpy())[2], x[0, 128:].mean(0).numpy())


def test_a_one_key_prompt_fits_nothing():
    from fold_attention_b200.decode import tail as ptail

    k = torch.randint(-127, 128, (2, 1, 64)).float()
    u, vr, vsum, ysum, rows = ptail.fit_prompt(k, torch.full((2, 1), 0.01).bfloat16(), torch.randn(2, 1, 64).bfloat16(), 16)
    assert torch.isfinite(vr).all() and torch.isfinite(rows).all()
    # whatever the map, the block's only key re-enters at its own V
    y = ptail.project(k, torch.full((2, 1), 0.01).bfloat16(), u)
    assert torch.allclose(rows + (y @ vr.transpose(1, 2)), vsum, atol=1e-5)


def test_rank_checks():
    from fold_attention_b200.decode import tail as ptail

    for bad in (8, 12, 32, -1):
        with pytest.raises(ValueError, match="tail rank"):
            ptail.check_rank(bad, 128)
    ptail.check_rank(0, 64)
    ptail.check_rank(16, 64)


def test_append_keeps_the_block_sums_of_a_refit():
    """Appending keys one at a time (the oracle's statement of the step's arithmetic) ends at the
    block sums and row a fit over the same keys gives, to fp32 rounding."""
    rng = np.random.default_rng(3)
    D, n = 64, 70
    kint = rng.integers(-127, 128, (n, D)).astype(np.float64)
    ek = np.full(n, 0.0078125)
    v = rng.standard_normal((n, D)).astype(np.float32)
    u, vr, y, rows = otail.tail_fit(kint, ek, v, 16)
    vsum = np.zeros(D, np.float32)
    ysum = np.zeros(16, np.float32)
    for i in range(n):
        vsum, ysum, row = otail.append(kint[i], ek[i], v[i], i, u, vr, vsum, ysum)
        if i == 63:
            assert np.allclose(row, rows[0], atol=1e-4)
    assert np.allclose(vsum, v[64:].sum(0), atol=1e-5)      # block 1 restarted at key 64
    assert np.allclose(row, rows[1], atol=1e-4)
