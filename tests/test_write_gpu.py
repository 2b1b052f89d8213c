"""Every cache write is the oracle's quantiser to the bit: the step's Q and
appended token, and the prompt's. Mirrors the reference's tests/test_write.py,
with the CPU oracle (pinned on the reference's own torch code) as checker."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import cache_format as cf  # noqa: E402


def _mods():
    from fold_attention_b200.decode.write import step, write_prompt

    return step, write_prompt


def _state(B, H, HKV, D, PS, ppr, v8):
    def z8(n):
        return torch.zeros(n, D, device="cuda", dtype=torch.int8)

    rows = B * ppr * HKV * PS
    vdt = torch.float8_e4m3fn if v8 else torch.bfloat16
    return dict(
        qa=z8(B * H), qb=z8(B * H), eq=torch.zeros(B * H, device="cuda"),
        ka=z8(rows), kb=z8(rows), ek=torch.zeros(rows, device="cuda", dtype=torch.bfloat16),
        va=torch.zeros(rows, D, device="cuda", dtype=vdt),
        vb=torch.zeros(rows, D, device="cuda", dtype=vdt) if v8 else None,
        vsum=torch.zeros(B * HKV, D, device="cuda"), vmean=torch.zeros(B * HKV, D, device="cuda"),
    )


def _np_pool(B, HKV, D, PS, ppr, v8):
    rows = B * ppr * HKV * PS
    return dict(
        ka=np.zeros((rows, D), np.int8), kb=np.zeros((rows, D), np.int8),
        ek=np.zeros(rows, np.float32),
        va=np.zeros((rows, D), np.uint8 if v8 else np.float32),
        vb=np.zeros((rows, D), np.uint8) if v8 else None,
        vsum=np.zeros((B * HKV, D), np.float32), vmean=np.zeros((B * HKV, D), np.float32),
    )


def _run(st, q, k, v, pt, PS, lens, evs, lens_out):
    step, _ = _mods()
    step(q, k, v, st["qa"], st["qb"], st["eq"], st["ek"], pt, PS, lens, st["ka"], st["kb"],
         st["va"], st["vb"], evs, st["vsum"], st["vmean"], lens_out)


def _case(B=6, H=32, HKV=4, D=128, PS=64, ppr=8, seed=3, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(B * H, D, device="cuda", generator=g) * 3).to(dtype)
    k = (torch.randn(B, HKV, D, device="cuda", generator=g) * 2).to(dtype)
    v = (torch.randn(B, HKV, D, device="cuda", generator=g) + 1).to(dtype)
    lens = torch.randint(1, ppr * PS - 1, (B,), device="cuda", generator=g).int()
    pt = torch.randperm(B * ppr, device="cuda", generator=g).int().view(B, ppr)
    return q, k, v, lens, pt


def _f(t):
    return t.float().cpu().numpy()


def _bits(t):
    return t.view(torch.uint8).cpu().numpy() if t.dtype == torch.float8_e4m3fn else t.cpu().numpy()


def _check_pool(got, want, v8):
    assert np.array_equal(got["ka"].cpu().numpy(), want["ka"])
    assert np.array_equal(got["kb"].cpu().numpy(), want["kb"])
    assert np.array_equal(_f(got["ek"]).view(np.int32), want["ek"].view(np.int32))
    if v8:
        assert np.array_equal(_bits(got["va"]), want["va"])
        assert np.array_equal(_bits(got["vb"]), want["vb"])
    else:
        assert np.array_equal(_f(got["va"]), want["va"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("G", [1, 8, 16])
def test_q_planes_are_the_oracles(D, G, dtype):
    B, HKV = 5, 2
    q, _, _, lens, pt = _case(B=B, H=G * HKV, HKV=HKV, D=D, dtype=dtype)
    q[3] = 0
    st = _state(B, G * HKV, HKV, D, 64, 8, True)
    _run(st, q, None, None, pt, 64, lens, 1.0, lens)
    qa, qb, eq = cf.quantize_q(_f(q))
    assert np.array_equal(st["qa"].cpu().numpy(), qa)
    assert np.array_equal(st["qb"].cpu().numpy(), qb)
    assert np.array_equal(st["eq"].cpu().numpy().view(np.int32), eq.view(np.int32))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("v8", [False, True])
@pytest.mark.parametrize("HKV", [1, 4, 8, 20])
def test_the_append_is_the_oracles(D, v8, HKV):
    """K's planes and scale, V's planes, the V sum and mean, the length advanced."""
    B, PS = 6, 64
    _, k, v, lens, pt = _case(B=B, HKV=HKV, D=D, PS=PS)
    got = _state(B, 8, HKV, D, PS, 8, v8)
    want = _np_pool(B, HKV, D, PS, 8, v8)
    sums = torch.randn(B * HKV, D, device="cuda")
    got["vsum"].copy_(sums)
    evs = 0.25 if v8 else 1.0
    out = torch.empty_like(lens)
    _run(got, None, k, v, pt, PS, lens, evs, out)
    assert torch.equal(out, lens + 1)
    pos = lens.cpu().numpy().astype(np.int64)
    row, off = cf.page_row(pt.cpu().numpy(), np.arange(B)[:, None], np.arange(HKV)[None, :],
                           pos[:, None], PS, HKV)
    cf.write_rows(want, _f(k), _f(v), evs, row, pos % PS)
    _check_pool(got, want, v8)
    ws, wm = cf.append_vsum(sums.cpu().numpy(), _f(v).reshape(B * HKV, D),
                            np.repeat(pos, HKV)[:, None], evs)
    assert np.array_equal(got["vsum"].cpu().numpy(), ws)
    assert np.array_equal(got["vmean"].cpu().numpy(), wm)


def test_the_lengths_advance_in_place():
    B, HKV, D, PS = 9, 8, 128, 64
    _, k, v, lens, pt = _case(B=B, HKV=HKV, D=D, PS=PS)
    st = _state(B, 8, HKV, D, PS, 8, True)
    want = _np_pool(B, HKV, D, PS, 8, True)
    pos = lens.cpu().numpy().astype(np.int64)
    row, _ = cf.page_row(pt.cpu().numpy(), np.arange(B)[:, None], np.arange(HKV)[None, :],
                         pos[:, None], PS, HKV)
    cf.write_rows(want, _f(k), _f(v), 0.25, row, pos % PS)
    start = lens.clone()
    _run(st, None, k, v, pt, PS, lens, 0.25, lens)
    assert torch.equal(lens, start + 1)
    assert np.array_equal(st["ka"].cpu().numpy(), want["ka"])


def test_the_step_is_its_two_halves():
    B, H, HKV, D, PS = 6, 32, 4, 128, 64
    q, k, v, lens, pt = _case(B=B, H=H, HKV=HKV, D=D, PS=PS)
    a, b = _state(B, H, HKV, D, PS, 8, True), _state(B, H, HKV, D, PS, 8, True)
    oa, ob = torch.empty_like(lens), torch.empty_like(lens)
    _run(a, q, None, None, pt, PS, lens, 0.5, oa)
    _run(a, None, k, v, pt, PS, lens, 0.5, oa)
    _run(b, q, k, v, pt, PS, lens, 0.5, ob)
    for n in a:
        if a[n] is not None:
            assert torch.equal(a[n].view(torch.int8), b[n].view(torch.int8)), n
    assert torch.equal(oa, ob)


def test_a_rows_bits_are_its_own():
    """A request stepped alone and inside a batch writes the same bits."""
    B, H, HKV, D, PS = 7, 32, 4, 128, 64
    q, k, v, lens, pt = _case(B=B, H=H, HKV=HKV, D=D, PS=PS)
    full = _state(B, H, HKV, D, PS, 8, True)
    _run(full, q, k, v, pt, PS, lens, 0.5, torch.empty_like(lens))
    for b in (0, 4, 6):
        one = _state(B, H, HKV, D, PS, 8, True)
        _run(one, q[b * H:(b + 1) * H], k[b:b + 1], v[b:b + 1], pt[b:b + 1].contiguous(), PS,
             lens[b:b + 1], 0.5, torch.empty_like(lens[:1]))
        assert torch.equal(one["qa"][:H], full["qa"][b * H:(b + 1) * H])
        assert torch.equal(one["qb"][:H], full["qb"][b * H:(b + 1) * H])
        rows = one["ka"].abs().sum(-1).nonzero().flatten()
        assert rows.numel() > 0
        assert torch.equal(one["ka"][rows], full["ka"][rows])
        assert torch.equal(one["kb"][rows], full["kb"][rows])
        assert torch.equal(one["ek"][rows], full["ek"][rows])


def test_every_e4m3_value_and_tie(golden_cache):
    """V's planes over every e4m3 value, every midpoint between neighbours and
    both zeros, against the planes the reference's torch code produced."""
    g = golden_cache
    D, HKV, PS, evs = 128, 1, 64, 0.5
    vals = torch.from_numpy(g["e4m3_in"]).cuda()
    n = -(-vals.numel() // D) * D
    v = torch.cat([vals, torch.zeros(n - vals.numel(), device="cuda")]).bfloat16().view(-1, HKV, D)
    B = v.shape[0]
    k = torch.randn(B, HKV, D, device="cuda").bfloat16()
    lens = torch.arange(B, device="cuda", dtype=torch.int32)
    pt = torch.arange(B, device="cuda", dtype=torch.int32).view(B, 1)
    got = _state(B, 8, HKV, D, PS, 1, True)
    _run(got, None, k, v, pt, PS, lens, evs, torch.empty_like(lens))
    rows = (torch.arange(B, device="cuda") * PS + lens).long()
    va = got["va"].view(torch.uint8)[rows].reshape(-1)[: vals.numel()].cpu().numpy()
    vb = got["vb"].view(torch.uint8)[rows].reshape(-1)[: vals.numel()].cpu().numpy()
    assert np.array_equal(va, g["e4m3_pa"])
    assert np.array_equal(vb, g["e4m3_pb"])


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("v8", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_the_prompt_writer_is_the_oracles(D, v8, dtype):
    _, write_prompt = _mods()
    g = torch.Generator(device="cuda").manual_seed(4)
    lens, H, PS = [700, 1, 256, 513], 4, 64
    N, B, ppr = sum(lens), len(lens), 16
    k = (torch.randn(N, H, D, device="cuda", generator=g) * 3).to(dtype)
    v = (torch.randn(N, H, D, device="cuda", generator=g) + 1).to(dtype)
    pt = torch.randperm(B * ppr, device="cuda", generator=g).int().view(B, ppr)
    got = _state(B, H, H, D, PS, ppr, v8)
    evs = float(write_prompt(k, v, lens, pt, PS, got["ka"], got["kb"], got["va"], got["vb"],
                             got["ek"], got["vsum"], got["vmean"], v_headroom=2.0, v_scale=None))
    if v8:
        assert evs == 2.0 ** math.ceil(math.log2(float(v.abs().amax()) * 2.0 / 448.0))
    else:
        assert evs == 1.0
    want = _np_pool(B, H, D, PS, ppr, v8)
    vf = _f(v)
    if not v8:  # the pool is bf16
        vf = v.bfloat16().float().cpu().numpy()
    wev = cf.write_prompt(want, _f(k), vf if not v8 else _f(v), lens, pt.cpu().numpy(), PS, v8)
    assert wev == evs
    _check_pool(got, want, v8)
    if not v8:
        want["vsum"], want["vmean"] = cf.prompt_vsum(_f(v), lens, 1.0)
    assert np.array_equal(got["vsum"].cpu().numpy(), want["vsum"])
    assert np.array_equal(got["vmean"].cpu().numpy(), want["vmean"])


def test_a_prompts_scales_and_sums_are_its_own():
    _, write_prompt = _mods()
    g = torch.Generator(device="cuda").manual_seed(6)
    lens, H, D, PS = [300, 1100, 57], 2, 128, 64
    N, B, ppr = sum(lens), len(lens), 32
    k = (torch.randn(N, H, D, device="cuda", generator=g) * 3).bfloat16()
    v = (torch.randn(N, H, D, device="cuda", generator=g) + 1).bfloat16()
    pt = torch.arange(B * ppr, device="cuda", dtype=torch.int32).view(B, ppr)
    full = _state(B, H, H, D, PS, ppr, False)
    write_prompt(k, v, lens, pt, PS, full["ka"], full["kb"], full["va"], None, full["ek"],
                 full["vsum"], full["vmean"], v_headroom=2.0, v_scale=None)
    cu = [0] + list(torch.tensor(lens).cumsum(0).tolist())
    for b in range(B):
        one = _state(B, H, H, D, PS, ppr, False)
        write_prompt(k[cu[b]:cu[b + 1]], v[cu[b]:cu[b + 1]], [lens[b]], pt[b:b + 1].contiguous(), PS,
                     one["ka"], one["kb"], one["va"], None, one["ek"], one["vsum"], one["vmean"],
                     v_headroom=2.0, v_scale=None)
        assert torch.equal(one["vsum"][:H], full["vsum"][b * H:(b + 1) * H])
        rows = slice(int(pt[b, 0]) * H * PS, (int(pt[b, -1]) + 1) * H * PS)
        assert torch.equal(one["ka"][rows], full["ka"][rows])
        assert torch.equal(one["ek"][rows], full["ek"][rows])
