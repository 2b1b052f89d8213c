"""The CPU oracle of the cache format against vectors produced by the
reference's own torch quantisers (tests/golden/make_cache_golden.py)."""

import numpy as np
import pytest

from oracle import cache_format as cf


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("tag", ["bf16", "f16"])
def test_key_planes_and_rotation(golden_cache, D, tag):
    g = golden_cache
    k = g[f"key_{D}_{tag}_in"]
    assert np.array_equal(cf.hadamard(k).view(np.int32), g[f"had_{D}_{tag}"].view(np.int32))
    pa, pb, e = cf.key_planes(k)
    assert np.array_equal(pa, g[f"key_{D}_{tag}_pa"])
    assert np.array_equal(pb, g[f"key_{D}_{tag}_pb"])
    assert np.array_equal(e.view(np.int32), g[f"key_{D}_{tag}_e"].view(np.int32))
    assert not (e.view(np.int32) & 0xFFFF).any()  # exact in bf16


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("tag", ["bf16", "f16"])
def test_query_planes(golden_cache, D, tag):
    g = golden_cache
    pa, pb, e = cf.quantize_q(g[f"q_{D}_{tag}_in"])
    assert np.array_equal(pa, g[f"q_{D}_{tag}_pa"])
    assert np.array_equal(pb, g[f"q_{D}_{tag}_pb"])
    assert np.array_equal(e.view(np.int32), g[f"q_{D}_{tag}_e"].view(np.int32))


def test_every_e4m3_value_and_tie(golden_cache):
    g = golden_cache
    pa, pb = cf.e4m3_planes(g["e4m3_in"], 0.5)
    assert np.array_equal(pa, g["e4m3_pa"])
    assert np.array_equal(pb, g["e4m3_pb"])
    pa, pb = cf.e4m3_planes(g["e4m3r_in"], 0.25)
    assert np.array_equal(pa, g["e4m3r_pa"])
    assert np.array_equal(pb, g["e4m3r_pb"])
    # quantize_v's scale (cache.py:148-158) is the writer's rule at headroom 1
    assert cf.v_scale_rule(float(np.abs(g["e4m3r_in"]).max()), 1.0) == g["e4m3r_ev"]


def test_e4m3_decode_table_roundtrip():
    b = np.arange(256, dtype=np.uint8)
    v = cf.e4m3_decode(b)
    ok = np.isfinite(v)
    assert ok.sum() == 254
    assert np.array_equal(cf.e4m3_encode(v[ok]), b[ok])


@pytest.mark.parametrize("t", ["bf", "v8"])
def test_paged_append(golden_cache, t):
    g = golden_cache
    B, HKV, D, PS, ppr = 6, 4, 128, 64, 8
    rows = B * ppr * HKV * PS
    v8 = t == "v8"
    pool = dict(
        ka=np.zeros((rows, D), np.int8),
        kb=np.zeros((rows, D), np.int8),
        ek=np.zeros(rows, np.float32),
        va=np.zeros((rows, D), np.uint8 if v8 else np.float32),
        vb=np.zeros((rows, D), np.uint8) if v8 else None,
    )
    lens, pt = g[f"app_{t}_lens"].astype(np.int64), g[f"app_{t}_pt"]
    row, off = cf.page_row(pt, np.arange(B)[:, None], np.arange(HKV)[None, :], lens[:, None], PS, HKV)
    cf.write_rows(pool, g[f"app_{t}_k"], g[f"app_{t}_v"], 0.25 if v8 else 1.0, row, lens % PS)
    nz = g[f"app_{t}_rows"]
    assert np.array_equal(np.sort(row.reshape(-1)), nz)
    for n in ("ka", "kb", "ek", "va", "vb"):
        if pool[n] is not None:
            assert np.array_equal(pool[n][nz], g[f"app_{t}_{n}"]), n
    mask = np.ones(rows, bool)
    mask[nz] = False
    assert not pool["ka"][mask].any()


def test_prompt_rows(golden_cache):
    g = golden_cache
    lens, pt = g["pr_lens"].tolist(), g["pr_pt"]
    H, PS, D, ppr = 2, 64, 64, 8
    rows = len(lens) * ppr * H * PS
    pool = dict(
        ka=np.zeros((rows, D), np.int8),
        kb=np.zeros((rows, D), np.int8),
        ek=np.zeros(rows, np.float32),
        va=np.zeros((rows, D), np.uint8),
        vb=np.zeros((rows, D), np.uint8),
        vsum=np.zeros((len(lens) * H, D), np.float32),
        vmean=np.zeros((len(lens) * H, D), np.float32),
    )
    ev = cf.write_prompt(pool, g["pr_k"], g["pr_v"], lens, pt, PS, True)
    assert ev == float(g["pr_evs"])
    for n in ("ka", "kb", "ek", "va", "vb"):
        assert np.array_equal(pool[n], g[f"pr_{n}"]), n
    cu = np.concatenate([[0], np.cumsum(lens)])
    ref = np.stack([g["pr_v"][cu[b]:cu[b + 1]].astype(np.float64).sum(0) for b in range(len(lens))])
    assert np.abs(pool["vsum"].astype(np.float64) - ref.reshape(-1, D)).max() < 1e-3
    n = np.repeat(np.array(lens, np.float32), H)[:, None]
    assert np.array_equal(pool["vmean"], pool["vsum"] / (n * np.float32(ev)))


def test_swizzle(golden_cache):
    g = golden_cache
    for n in ("swz", "swz64"):
        x = g[f"{n}_in"]
        b, S, D = x.shape
        got = np.stack([cf.swizzle_units(x[i].view(np.uint8), np.arange(S)).view(np.int8) for i in range(b)])
        assert np.array_equal(got, g[f"{n}_out"])
