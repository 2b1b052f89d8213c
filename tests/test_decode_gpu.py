"""The paged decode: the cache it reads is the oracle's, its reference is the
mass estimate it documents, its verdict counts are the exact coarse-logit
model's, and its output is softmax attention within the stated tolerances
(dense rel-L2 < 4e-3 against FP32 attention, truncated < 2^(-depth/3); both
from the reference's tests/test_kv_cache.py:167-251)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import decode as od  # noqa: E402

LOG2E = 1.4426950408889634


def _fa():
    import fold_attention_b200 as fa

    return fa


def _layer(B, H, HKV, D, lens, seed=0, peaked=True, dtype=torch.bfloat16, vmu=0.0):
    """Packed prompts with the benchmark configs' distributions: K, V, q ~ N(0,1), 1% of
    key positions x8, 0.1% of V entries x20."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=g)
    v = torch.randn(T, HKV, D, device="cuda", generator=g) + vmu
    if peaked:
        hot = torch.rand(T, 1, 1, device="cuda", generator=g) < 0.01
        k = torch.where(hot, k * 8, k)
        out = torch.rand(T, HKV, D, device="cuda", generator=g) < 0.001
        v = torch.where(out, v * 20, v)
    q = torch.randn(B, H, D, device="cuda", generator=g)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    return q.to(dtype), k.to(dtype), v.to(dtype), cu


def _cache(B, H, HKV, D, lens, ps=64, shuffle=True, seed=0, **kw):
    fa = _fa()
    c = fa.FoldKVCache(B, H, HKV, D, max(lens) + 8, page_size=ps, **kw)
    if shuffle:
        g = torch.Generator(device="cuda").manual_seed(seed + 99)
        c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=g).int().view_as(c.page_table))
    return c


def _rows(c, b, h, n):
    pos = torch.arange(n, device="cuda")
    pg = c.page_table[b, pos // c.page_size].long()
    return (pg * c.n_kv_heads + h) * c.page_size + pos % c.page_size, pos % c.page_size


def _planes(c, b, h, n):
    """Row group (b, h)'s unswizzled planes, scales and V in float."""
    rows, slots = _rows(c, b, h, n)
    ka = od.unswizzle(c.ka[rows], slots, c.head_dim)
    kb = od.unswizzle(c.kb[rows], slots, c.head_dim)
    ek = c.ek[rows].float()
    va = c.va[rows].float()
    vb = c.vb[rows].float() if c.vb is not None else None
    return ka, kb, ek, va, vb


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def _attend_ref(q, k, v, cu, b, HKV, G, extra_k=None, extra_v=None):
    """FP32 attention of request b's query rows over its (16-bit) keys."""
    a, e = int(cu[b]), int(cu[b + 1])
    outs = []
    for h in range(HKV):
        kk, vv = k[a:e, h].float(), v[a:e, h].float()
        if extra_k is not None:
            kk = torch.cat([kk, extra_k[b, h].float()[None]])
            vv = torch.cat([vv, extra_v[b, h].float()[None]])
        outs.append(od.attend_fp32(q[b, h * G:(h + 1) * G].float(), kk, vv))
    return torch.cat(outs)


@pytest.mark.parametrize("D,G", [(128, 8), (64, 4), (128, 1)])
def test_the_mass_reference_is_the_estimate_it_documents(D, G):
    HKV = 2
    lens = [8192, 97, 300, 8192 - 777, 64, 1]
    B = len(lens)
    q, k, v, cu = _layer(B, HKV * G, HKV, D, lens, seed=1)
    c = _cache(B, HKV * G, HKV, D, lens, ps=64)
    c.write_prompt(k, v, cu, lens)
    c.attend(q)
    for b in range(B):
        for h in range(HKV):
            bh = b * HKV + h
            ka, _, ek, _, _ = _planes(c, b, h, lens[b])
            s = od.coarse_logits(c.qa[bh][None], c.qb[bh][None], c.eq[bh][None], ka[None], ek[None])[0]
            want = od.mass_model(s, lens[b])
            assert float((c.z[bh].double() - want).abs().max()) < 1e-4, (b, h)


@pytest.mark.parametrize("v8,depth,D,G,ps", [
    (False, None, 128, 8, 64), (True, None, 128, 8, 256), (True, 16.0, 128, 8, 64),
    (False, 12.0, 128, 4, 16), (True, 10.0, 64, 8, 32), (False, None, 64, 2, 64),
])
def test_given_a_reference_the_kernel_is_its_model(v8, depth, D, G, ps):
    """With Z given, the live and refined counts are the exact coarse-logit
    model's (data, not schedule), and the output is the model's function."""
    from fold_attention_b200.decode.launch import prepare_fold_decode

    HKV = 2
    lens = [1500, 700, 64, 2049]
    B = len(lens)
    q, k, v, cu = _layer(B, HKV * G, HKV, D, lens, seed=2, vmu=0.5)
    c = _cache(B, HKV * G, HKV, D, lens, ps=ps, v8=v8, depth=depth)
    c.write_prompt(k, v, cu, lens)
    c.attend(q)  # writes Q planes and the mass reference
    z = (torch.ceil(c.z * 16) / 16).contiguous()  # any reference near the mass will do
    rk, rv = 10.0, 10.0
    for split, chunk in ((1, 0), (3, 0), (0, 512)):
        sp = split if not chunk else -(-max(lens) // chunk)
        run = prepare_fold_decode(
            c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, split=sp,
            truncate=depth is not None, refine_k=rk, refine_v=rv, v8=v8, v2=c.vb, v_scale=c.v_scale,
            vmean=c.vmean, page_table=c.page_table, page_size=ps, seq_lens=c.seq_lens,
            n_kv_heads=HKV, weight_terms=2, chunk_keys=chunk,
        )
        out, den, counts = run()
        torch.cuda.synchronize()
        assert int(run.status) == 0
        for b in range(B):
            for h in range(HKV):
                bh = b * HKV + h
                ka, kb, ek, va, vb = _planes(c, b, h, lens[b])
                want, wden, nlive, nref = od.decode_model(
                    c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, va, vb, c.v_scale, z[bh], depth,
                    rk, rv, lens[b], vmean=c.vmean[bh] if depth is not None else None)
                assert counts[bh].tolist() == [nlive, nref], (split, chunk, b, h)
                assert _rel(out[bh], want) < 2e-3, (split, chunk, b, h, _rel(out[bh], want))
                assert ((den[bh].double() - wden).abs() / wden).max().item() < 2e-3


@pytest.mark.parametrize("v8", [False, True])
@pytest.mark.parametrize("D,H,HKV", [(128, 32, 4), (64, 8, 2), (128, 8, 8)])
def test_decode_after_prefill_is_the_softmax_over_everything_written(v8, D, H, HKV):
    fa = _fa()
    lens = [1024, 333, 4096, 65]
    B, G = len(lens), H // HKV
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=3)
    c = _cache(B, H, HKV, D, lens, ps=64, v8=v8)
    qp = torch.randn(sum(lens), H, D, device="cuda").to(q.dtype)
    out = c.prefill(qp, k, v, cu)
    assert out.shape == qp.shape
    g = torch.Generator(device="cuda").manual_seed(5)
    kn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
    vn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
    got = fa.fold_attn_with_kvcache(q, c, kn, vn)
    assert got.dtype == q.dtype and got.shape == q.shape
    assert c.lens == [n + 1 for n in lens]
    assert c.seq_lens.tolist() == c.lens
    want = torch.stack([_attend_ref(q, k, v, cu, b, HKV, G, kn, vn) for b in range(B)])
    assert _rel(got, want) < 4e-3, _rel(got, want)
    # attend again without appending: the same cache, the same answer
    again = fa.fold_attn_with_kvcache(q[:, None], c)[:, 0]
    assert torch.equal(again, got)


@pytest.mark.parametrize("v8", [False, True])
@pytest.mark.parametrize("depth", [8.0, 12.0, 16.0])
def test_a_truncated_depth_costs_what_it_says(v8, depth):
    lens = [4096, 2000, 8192]
    B, H, HKV, D = len(lens), 16, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=4, vmu=0.3)
    c = _cache(B, H, HKV, D, lens, ps=256, v8=v8, depth=depth)
    c.write_prompt(k, v, cu, lens)
    got = c.attend(q)
    want = torch.stack([_attend_ref(q, k, v, cu, b, HKV, H // HKV) for b in range(B)])
    err = _rel(got, want)
    assert err < 2.0 ** (-depth / 3), err
    live = c.counts[:, 0].sum().item() / (sum(lens) * HKV)
    assert live <= 1.0
    if depth <= 8.0:
        assert live < 0.9, live  # the cut really drops keys


def test_splits_regroup_sums_and_a_fixed_chunk_pins_them():
    """The split only regroups fp32 sums; under a fixed chunk a request's
    output is the same bits alone and inside a batch."""
    lens = [3000, 1000, 5000]
    B, H, HKV, D = len(lens), 16, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=6)
    outs = []
    for split in (1, 2, 7):
        c = _cache(B, H, HKV, D, lens, ps=64, v8=True, depth=16.0, split=split, seed=split)
        c.write_prompt(k, v, cu, lens)
        outs.append(c.attend(q).float())
        assert c.counts.tolist() == c.counts.tolist()
    assert (outs[0] - outs[1]).abs().max().item() < 2e-3 * outs[0].abs().max().item()
    assert (outs[0] - outs[2]).abs().max().item() < 2e-3 * outs[0].abs().max().item()
    full = _cache(B, H, HKV, D, lens, ps=64, v8=True, depth=16.0, chunk=1024, v_scale=0.03125)
    full.write_prompt(k, v, cu, lens)
    o_full = full.attend(q)
    cnt_full = full.counts.clone()
    for b in range(B):
        one = _cache(1, H, HKV, D, [lens[b]], ps=64, v8=True, depth=16.0, chunk=1024, v_scale=0.03125, seed=b)
        a, e = int(cu[b]), int(cu[b + 1])
        one.write_prompt(k[a:e], v[a:e], torch.tensor([0, lens[b]], device="cuda", dtype=torch.int32), [lens[b]])
        o_one = one.attend(q[b:b + 1])
        assert torch.equal(o_one[0], o_full[b])
        assert torch.equal(one.counts, cnt_full[b * HKV:(b + 1) * HKV])


def test_sixty_four_steps_track_the_softmax():
    """Config-4-like serving at a small scale: append + attend for many steps
    with a shuffled page table."""
    fa = _fa()
    lens = [700, 130, 1999]
    B, H, HKV, D = len(lens), 8, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=8)
    c = _cache(B, H, HKV, D, [n + 70 for n in lens], ps=64)
    c.write_prompt(k, v, cu, lens)
    ks = [k[int(cu[b]):int(cu[b + 1])].float() for b in range(B)]
    vs = [v[int(cu[b]):int(cu[b + 1])].float() for b in range(B)]
    g = torch.Generator(device="cuda").manual_seed(9)
    worst = 0.0
    for step in range(64):
        qn = torch.randn(B, H, D, device="cuda", generator=g).bfloat16()
        kn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
        vn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
        got = fa.fold_attn_with_kvcache(qn, c, kn, vn)
        for b in range(B):
            ks[b] = torch.cat([ks[b], kn[b].float()[None]])
            vs[b] = torch.cat([vs[b], vn[b].float()[None]])
        if step % 21 == 0 or step == 63:
            want = torch.stack([
                torch.cat([od.attend_fp32(qn[b, h * 4:(h + 1) * 4].float(), ks[b][:, h], vs[b][:, h]) for h in range(HKV)])
                for b in range(B)])
            worst = max(worst, _rel(got, want))
    assert c.lens == [n + 64 for n in lens]
    assert worst < 4e-3, worst


def test_error_messages():
    fa = _fa()
    with pytest.raises(ValueError, match="do not group"):
        fa.FoldKVCache(2, 7, 2, 128, 256)
    with pytest.raises(ValueError, match="not a power of two"):
        fa.FoldKVCache(2, 8, 2, 128, 256, v8=True, v_scale=0.3)
    with pytest.raises(ValueError, match="truncates nothing"):
        fa.FoldKVCache(2, 8, 2, 128, 256, tail=16)
    with pytest.raises(ValueError, match="bf16 V cache"):
        fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, v8=True, tail=16)
    with pytest.raises(ValueError, match="replaces split"):
        fa.FoldKVCache(2, 8, 2, 128, 256, chunk=100)
    c = fa.FoldKVCache(2, 8, 2, 128, 256)
    k = torch.randn(10, 2, 128, device="cuda").bfloat16()
    with pytest.raises(ValueError, match="batch of 2"):
        c.prefill(k.repeat(1, 4, 1), k, k, torch.tensor([0, 10], device="cuda", dtype=torch.int32))
    with pytest.raises(ValueError, match="not in 1..256"):
        c.prefill(k.repeat(1, 4, 1), k, k, torch.tensor([0, 10, 10], device="cuda", dtype=torch.int32))
    c.write_prompt(k.repeat(52, 1, 1)[:512], k.repeat(52, 1, 1)[:512],
                   torch.tensor([0, 256, 512], device="cuda", dtype=torch.int32))
    with pytest.raises(ValueError, match="max_len=256"):
        c.append(k[:2], k[:2])
    q = torch.randn(2, 8, 128, device="cuda").bfloat16()
    with pytest.raises(ValueError, match="both given or both left out"):
        fa.fold_attn_with_kvcache(q, c, k[:2])


@pytest.mark.parametrize("v8,depth,kernel", [(False, None, "mma"), (True, 16.0, "mma"), (True, 16.0, "sm100")])
def test_check_range_reruns_the_rows_whose_reference_was_off(v8, depth, kernel):
    """A reference moved off a row's mass leaves the window [0.5, 2^60 or 2^100] of the
    denominator; with check_range the step is run again from Z + log2(den) and lands where
    the undisturbed step does (reference kv_cache.py:704-744)."""
    lens = [2000, 700]
    B, H, HKV, D = len(lens), 8, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=12)
    c = _cache(B, H, HKV, D, lens, ps=128, v8=v8, depth=depth, check_range=True, kernel=kernel)
    c.write_prompt(k, v, cu, lens)
    want = torch.stack([_attend_ref(q, k, v, cu, b, HKV, H // HKV) for b in range(B)])
    plain = c.attend(q)
    tol = 4e-3 if depth is None else 2.0 ** (-depth / 3)
    assert _rel(plain, want) < tol
    lo, hi = c._range_window()
    assert hi == (2.0 ** 60 if v8 else 2.0 ** 100)
    for move in (6.0, -70.0 if v8 else -110.0):
        c._step(q, None, None)        # Q's planes and the mass reference, as attend does
        z_mass = c.z.clone()
        c.z[1::2] += move             # every other row group's reference off its mass
        got = c._run(q, None)
        assert bool(((c.den >= lo) & (c.den <= hi)).all())
        assert _rel(got, want) < tol, (move, _rel(got, want))
        # the rows that were not flagged kept their reference: the same bits as the plain step
        assert torch.equal(got.view(B * HKV, -1)[0::2], plain.view(B * HKV, -1)[0::2])
        assert torch.equal(c.z[0::2], z_mass[0::2])
    off = _cache(B, H, HKV, D, lens, ps=128, v8=v8, depth=depth, kernel=kernel)   # without the check
    off.write_prompt(k, v, cu, lens)
    off._step(q, None, None)
    off.z[1::2] += 6.0
    off._run(q, None)
    assert bool((off.den[1::2] < lo).any())   # without the check such rows stay as they came out


@pytest.mark.parametrize("kernel,v8,depth", [("mma", False, None), ("mma", True, 12.0), ("sm100", True, 16.0), ("sm100", False, None)])
def test_where_the_pages_lie_changes_no_bit(kernel, v8, depth):
    """A shuffled page table, the identity one and another page size give the same bits and the
    same counts (the reference's paged-equals-contiguous check, tests/test_decode.py:555-597), and
    a key under the cut weighs exactly nothing: moving V of the dropped keys moves no bit either
    once their mass re-enters nowhere (a zero direction)."""
    lens = [1500, 260, 3000]
    B, H, HKV, D = len(lens), 16, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=12)
    outs = []
    for shuffle, ps, seed in ((False, 128, 0), (True, 128, 1), (True, 256, 2), (True, 128, 3)):
        c = _cache(B, H, HKV, D, lens, ps=ps, shuffle=shuffle, seed=seed, v8=v8, depth=depth, kernel=kernel, chunk=1024,
                   tail=None, v_scale=2.0 ** -3 if v8 else None)
        c.write_prompt(k, v, cu, lens)
        outs.append((c.attend(q).clone(), c.counts.clone(), c.den.clone()))
    for o, cnt, den in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(cnt, outs[0][1]) and torch.equal(den, outs[0][2])
    if depth is not None:
        from fold_attention_b200.decode.launch import prepare_fold_decode

        c = _cache(B, H, HKV, D, lens, ps=128, v8=v8, depth=depth, kernel=kernel, tail=None, v_scale=2.0 ** -3)
        c.write_prompt(k, v, cu, lens)
        c._step(q, None, None)
        cut = torch.full_like(c.z, 4.0)
        kw = dict(split=2, truncate=True, refine_k=2.0, refine_v=2.0, v8=True, v2=c.vb, v_scale=c.v_scale, vmean=torch.zeros_like(c.vmean),
                  page_table=c.page_table, page_size=128, seq_lens=c.seq_lens, n_kv_heads=HKV, weight_terms=2, kernel=kernel)
        z = (torch.ceil(c.z * 16) / 16).contiguous()
        base, _, counts = (t.clone() for t in prepare_fold_decode(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, cut, **kw)())
        assert int(counts[:, 0].sum()) < 0.5 * sum(lens) * HKV
        # scramble V of every key no row keeps: the model's live set, from the coarse logits
        for b, n in enumerate(lens):
            for h in range(HKV):
                bh = b * HKV + h
                ka, _, ek, _, _ = _planes(c, b, h, n)
                s1 = od.coarse_logits(c.qa[bh][None], c.qb[bh][None], c.eq[bh][None], ka[None], ek[None], z[bh][None])[0]
                dead = ~(s1 >= -4.0).any(0)
                rows, _ = _rows(c, b, h, n)
                c.va.view(torch.uint8)[rows[dead]] = 0x38      # e4m3 1.0 everywhere
                c.vb.view(torch.uint8)[rows[dead]] = 0x38
        again = prepare_fold_decode(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, cut, **kw)()[0]
        assert torch.equal(again, base)
