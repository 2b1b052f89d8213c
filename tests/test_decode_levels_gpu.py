"""The decode's layouts beyond the single-level step: a draft's rows and tree, a cascade's shared
prefix, row groups wider than 8 rows, and a row's own cut. Each against the float64 model on the
cache's own planes (counts to the unit) and against FP32 attention over the keys the rows see.
After the reference's tests/test_decode.py:1572-2600 (draft, tree, cascade suites)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import decode as od  # noqa: E402


def _fa():
    import fold_attention_b200 as fa

    return fa


def _kv(lens, HKV, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=g)
    hot = torch.rand(T, 1, 1, device="cuda", generator=g) < 0.02
    k = torch.where(hot, k * 5, k).bfloat16()
    v = (torch.randn(T, HKV, D, device="cuda", generator=g) + 0.5).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    return k, v, cu


def _cache(lens, H, HKV, D, seed, shuffle=True, **kw):
    fa = _fa()
    c = fa.FoldKVCache(len(lens), H, HKV, D, max(lens) + 64, page_size=kw.pop("page_size", 64), **kw)
    if shuffle:
        g = torch.Generator(device="cuda").manual_seed(seed + 7)
        c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=g).int().view_as(c.page_table))
    return c


def _rows(c, b, h, n):
    pos = torch.arange(n, device="cuda")
    pg = c.page_table[b, pos // c.page_size].long()
    return (pg * c.n_kv_heads + h) * c.page_size + pos % c.page_size, pos % c.page_size


def _planes(c, b, h, n):
    rows, slots = _rows(c, b, h, n)
    ka = od.unswizzle(c.ka[rows], slots, c.head_dim)
    kb = od.unswizzle(c.kb[rows], slots, c.head_dim)
    return ka, kb, c.ek[rows].float(), c.va[rows].float(), (c.vb[rows].float() if c.vb is not None else None)


def _l2(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def _quantise_rows(c, qrows):
    """Q's planes and scales for `(NBH, G, D)` rows through the library's own step kernel."""
    from fold_attention_b200.decode import write

    NBH, G, D = qrows.shape
    qa = torch.zeros((NBH, G, D), device="cuda", dtype=torch.int8)
    qb = torch.zeros_like(qa)
    eq = torch.ones((NBH, G), device="cuda", dtype=torch.float32)
    write.step(qrows.reshape(-1, D).contiguous(), None, None, qa.view(-1, D), qb.view(-1, D), eq.view(-1), c.ek, c.page_table,
               c.page_size, c.seq_lens, c.ka, c.kb, c.va, c.vb, c.v_scale, c.vsum, c.vmean, c.seq_lens)
    return qa, qb, eq


# ---------------------------------------------------------------- drafts ----

@pytest.mark.parametrize("v8,depth,q_len,tree", [
    (False, None, 2, "causal"), (True, 10.0, 4, "causal"), (False, 8.0, 4, [-1, 0, 0, 1]), (True, None, 8, [-1, 0, 1, 1, 0, 4, 4, 2]),
])
def test_a_draft_s_rows_see_their_own_nodes(v8, depth, q_len, tree):
    from fold_attention_b200.decode.launch import prepare_fold_decode
    from fold_attention_b200.decode.rows import draft_mask, pack_rows, unpack_rows

    D, HKV = 128, 2
    g0 = 8 // q_len
    H = HKV * g0
    lens = [300, 64 + q_len, 1000]
    B = len(lens)
    k, v, cu = _kv(lens, HKV, D, 21)
    c = _cache(lens, H, HKV, D, 21, v8=v8, depth=depth, tail=None, v_scale=2.0 ** -3 if v8 else None)
    c.write_prompt(k, v, cu, lens)       # the draft's own keys are each request's last q_len
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(B, q_len, H, D, device="cuda", generator=g).bfloat16()
    qa, qb, eq = _quantise_rows(c, pack_rows(q, HKV, q_len))
    NBH, G = B * HKV, 8
    causal = tree == "causal"
    m = torch.tril(torch.ones(q_len, q_len, dtype=torch.bool)) if causal else draft_mask(tree)
    z = torch.empty((NBH, G), device="cuda")
    cut = torch.full_like(z, 1e4 if depth is None else depth)
    for reference, split in (("mass", 1), ("given", 3)):
        run = prepare_fold_decode(
            qa, qb, eq, c.ka, c.kb, c.ek, c.va, z, cut, split=split, truncate=depth is not None, refine_k=10.0, refine_v=10.0,
            v8=v8, v2=c.vb, v_scale=c.v_scale, vmean=c.vmean if depth is not None else None, page_table=c.page_table,
            page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV, reference=reference, weight_terms=2,
            draft_len=q_len, causal=causal, mask=None if causal else m)
        out, den, counts = run()
        torch.cuda.synchronize()
        assert int(run.status) == 0 and run.kernel == "mma"
        worst = 0.0
        for b, n in enumerate(lens):
            for h in range(HKV):
                bh = b * HKV + h
                ka, kb, ek, va, vb = _planes(c, b, h, n)
                vis = torch.ones(G, n, dtype=torch.bool)
                for gi in range(g0):
                    for t in range(q_len):
                        vis[gi * q_len + t, n - q_len:] = m[t]
                want, wden, nlive, nref = od.decode_model(
                    qa[bh], qb[bh], eq[bh], ka, kb, ek, va, vb, c.v_scale, z[bh], depth, 10.0, 10.0, n,
                    vmean=c.vmean[bh] if depth is not None else None, visible=vis, row_cut=True)
                assert counts[bh].tolist() == [nlive, nref], (reference, b, h)
                assert _l2(out[bh], want) < 2e-3, (reference, b, h, _l2(out[bh], want))
                assert ((den[bh].double() - wden).abs() / wden).max().item() < 2e-3
                # and FP32 attention of each row over the keys it sees
                a = int(cu[b])
                for gi in range(g0):
                    for t in range(q_len):
                        see = vis[gi * q_len + t].cuda()
                        ref = od.attend_fp32(q[b, t, h * g0 + gi].float()[None], k[a:a + n, h].float()[see], v[a:a + n, h].float()[see])[0]
                        worst = max(worst, _l2(out[bh, gi * q_len + t], ref))
        assert worst < (6e-3 if depth is None else 2.0 ** (-depth / 3)), worst
    # the rows come back in the caller's layout
    assert unpack_rows(out, HKV, q_len).shape == (B, q_len, H, D)


def test_the_mass_reference_of_a_draft_row_leaves_out_what_it_does_not_see():
    """Row t's reference is the single-token estimate on the cache cut after its own node."""
    from fold_attention_b200.decode.launch import mass_z
    from fold_attention_b200.decode.rows import pack_rows, pack_tree

    D, HKV, q_len, g0 = 128, 2, 4, 2
    lens = [777, 200]
    k, v, cu = _kv(lens, HKV, D, 3)
    c = _cache(lens, HKV * g0, HKV, D, 3)
    c.write_prompt(k, v, cu, lens)
    q = torch.randn(2, q_len, HKV * g0, D, device="cuda").bfloat16()
    qa, qb, eq = _quantise_rows(c, pack_rows(q, HKV, q_len))
    tree = pack_tree(None, True, q_len, 8, 4, "cuda")
    z = torch.empty((4, 8), device="cuda")
    mass_z(qa, qb, eq, c.ka, c.ek, c.page_table, c.page_size, c.seq_lens, HKV, z, tree=tree, draft_len=q_len)
    for b, n in enumerate(lens):
        for h in range(HKV):
            bh = b * HKV + h
            ka, _, ek, _, _ = _planes(c, b, h, n)
            s = od.coarse_logits(qa[bh][None], qb[bh][None], eq[bh][None], ka[None], ek[None])[0]
            for r in range(8):
                t = r % q_len
                hidden = s[r:r + 1].clone()
                hidden[:, n - q_len + t + 1:] = float("-inf")     # the nodes after its own weigh nothing
                want = od.mass_model(hidden, n)
                assert abs(float(z[bh, r]) - float(want)) < 1e-4, (b, h, r)


# --------------------------------------------------------------- cascades ----

@pytest.mark.parametrize("v8,depth", [(False, None), (True, 12.0), (False, 8.0)])
def test_a_cascade_adds_its_levels_under_one_reference(v8, depth):
    from fold_attention_b200.decode.launch import SharedPrefix, prepare_fold_decode

    D, H, HKV = 128, 8, 2
    G = H // HKV
    plens, ulens = [700, 320], [200, 64, 500, 33]
    req_map = torch.tensor([0, 0, 1, -1], device="cuda", dtype=torch.int32)
    kw = dict(v8=v8, depth=depth, tail=None, v_scale=2.0 ** -3 if v8 else None)
    kp, vp, cup = _kv(plens, HKV, D, 31)
    ku, vu, cuu = _kv(ulens, HKV, D, 32)
    P = _cache(plens, H, HKV, D, 31, page_size=128, **kw)
    U = _cache(ulens, H, HKV, D, 32, **kw)
    P.write_prompt(kp, vp, cup, plens)
    U.write_prompt(ku, vu, cuu, ulens)
    B = len(ulens)
    q = torch.randn(B, H, D, device="cuda").bfloat16()
    U._step(q, None, None)
    NBH = B * HKV
    z = torch.empty((NBH, G), device="cuda")
    cut = torch.full_like(z, 1e4 if depth is None else depth)
    trunc = depth is not None
    level = SharedPrefix(P.ka, P.kb, P.ek, P.va, P.page_table, P.seq_lens, P.page_size, req_map=req_map, v2=P.vb,
                         vmean=P.vmean if trunc else None, split=3)
    run = prepare_fold_decode(
        U.qa, U.qb, U.eq, U.ka, U.kb, U.ek, U.va, z, cut, split=2, truncate=trunc, refine_k=10.0, refine_v=10.0, v8=v8, v2=U.vb,
        v_scale=U.v_scale, vmean=U.vmean if trunc else None, page_table=U.page_table, page_size=U.page_size, seq_lens=U.seq_lens,
        n_kv_heads=HKV, reference="mass", weight_terms=2, shared=level)
    out, den, counts = run()
    torch.cuda.synchronize()
    assert int(run.status) == 0
    worst = 0.0
    for b, n in enumerate(ulens):
        pre = int(req_map[b])
        for h in range(HKV):
            bh = b * HKV + h
            parts = [(U, b, n, U.vmean[bh])]
            if pre >= 0:
                parts.append((P, pre, plens[pre], P.vmean[pre * HKV + h]))
            num, dsum, live, ref = 0.0, 0.0, [], []
            zs = []
            for cch, rb, rn, vm in parts:
                ka, kb, ek, va, vb = _planes(cch, rb, h, rn)
                zs.append(od.mass_model(od.coarse_logits(U.qa[bh][None], U.qb[bh][None], U.eq[bh][None], ka[None], ek[None])[0], rn))
            zz = zs[0] if len(zs) == 1 else torch.logaddexp2(zs[0], zs[1])
            assert float((z[bh].double() - zz).abs().max()) < 1e-4          # the rows' mass over both levels
            for cch, rb, rn, vm in parts:
                ka, kb, ek, va, vb = _planes(cch, rb, h, rn)
                o, d, nl, nr = od.decode_model(U.qa[bh], U.qb[bh], U.eq[bh], ka, kb, ek, va, vb, U.v_scale, z[bh], depth, 10.0, 10.0, rn,
                                               vmean=vm if trunc else None, row_cut=True)
                num, dsum = num + o * d[:, None], dsum + d
                live.append(nl)
                ref.append(nr)
            want = num / dsum[:, None]
            assert counts[bh].tolist() == [live[0], ref[0]], (b, h)
            assert run.counts_shared[bh].tolist() == ([live[1], ref[1]] if pre >= 0 else [0, 0]), (b, h)
            assert _l2(out[bh], want) < 2e-3, (b, h, _l2(out[bh], want))
            assert ((den[bh].double() - dsum).abs() / dsum).max().item() < 2e-3
            # FP32 attention over the prefix and the request's own keys together
            a = int(cuu[b])
            kk, vv = ku[a:a + n, h].float(), vu[a:a + n, h].float()
            if pre >= 0:
                pa = int(cup[pre])
                kk = torch.cat([kp[pa:pa + plens[pre], h].float(), kk])
                vv = torch.cat([vp[pa:pa + plens[pre], h].float(), vv])
            ref32 = od.attend_fp32(q[b, h * G:(h + 1) * G].float(), kk, vv)
            worst = max(worst, _l2(out[bh], ref32))
    assert worst < (6e-3 if depth is None else 2.0 ** (-depth / 3)), worst


def test_a_request_in_a_cascade_does_not_see_who_shares_its_prefix():
    from fold_attention_b200.decode.launch import SharedPrefix, prepare_fold_decode

    D, H, HKV = 128, 8, 2
    G = H // HKV
    plens, ulens = [900], [150, 400, 64]
    kp, vp, cup = _kv(plens, HKV, D, 41)
    ku, vu, cuu = _kv(ulens, HKV, D, 42)
    P = _cache(plens, H, HKV, D, 41, depth=10.0, tail=None)
    P.write_prompt(kp, vp, cup, plens)
    q = torch.randn(3, H, D, device="cuda").bfloat16()

    def run_batch(ids):
        lens = [ulens[i] for i in ids]
        rows = torch.cat([torch.arange(int(cuu[i]), int(cuu[i + 1]), device="cuda") for i in ids])
        U = _cache(lens, H, HKV, D, 42 + len(ids), depth=10.0, tail=None)
        U.write_prompt(ku[rows], vu[rows], torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32), lens)
        U._step(q[ids], None, None)
        z = torch.empty((len(ids) * HKV, G), device="cuda")
        level = SharedPrefix(P.ka, P.kb, P.ek, P.va, P.page_table, P.seq_lens, P.page_size, vmean=P.vmean, split=2)
        run = prepare_fold_decode(
            U.qa, U.qb, U.eq, U.ka, U.kb, U.ek, U.va, z, U.cut, split=2, truncate=True, refine_k=10.0, refine_v=10.0,
            v_scale=1.0, vmean=U.vmean, page_table=U.page_table, page_size=U.page_size, seq_lens=U.seq_lens, n_kv_heads=HKV,
            reference="mass", weight_terms=2, shared=level)
        return run()[0].clone()

    together = run_batch([0, 1, 2])
    for i in range(3):
        alone = run_batch([i])
        assert torch.equal(alone[0:HKV], together[i * HKV:(i + 1) * HKV])


# ----------------------------------------------------- wide groups, cuts ----

@pytest.mark.parametrize("H,HKV,v8,depth", [(32, 2, False, None), (32, 1, True, 12.0), (48, 2, False, 10.0)])
def test_row_groups_wider_than_eight_run_as_groups_of_eight(H, HKV, v8, depth):
    fa = _fa()
    D = 128
    G = H // HKV
    lens = [600, 70, 1500]
    B = len(lens)
    k, v, cu = _kv(lens, HKV, D, 51)
    c = _cache(lens, H, HKV, D, 51, v8=v8, depth=depth)
    assert c.kernel == "mma" and c.tail_rank == -1
    c.write_prompt(k, v, cu, lens)
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B, H, D, device="cuda", generator=g).bfloat16()
    kn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
    vn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
    out = fa.fold_attn_with_kvcache(q, c, kn, vn)
    assert out.shape == q.shape and c.counts.shape == (B * HKV * (G // 8), 2)
    worst = 0.0
    for b, n in enumerate(lens):
        a = int(cu[b])
        for h in range(HKV):
            kk = torch.cat([k[a:a + n, h], kn[b, h][None]]).float()
            vv = torch.cat([v[a:a + n, h], vn[b, h][None]]).float()
            ref = od.attend_fp32(q[b, h * G:(h + 1) * G].float(), kk, vv)
            worst = max(worst, _l2(out[b, h * G:(h + 1) * G], ref))
            # each group of eight is the model of its own eight rows: its verdicts are its own
            ka, kb, ek, va, vb = _planes(c, b, h, n + 1)
            for s_ in range(G // 8):
                bh = (b * HKV + h) * (G // 8) + s_
                rows = slice(8 * s_, 8 * s_ + 8)
                rk, rv = c._refine()
                if c._banded():
                    rk_t, rv_t = c.refine_gates()
                    rk, rv = float(rk_t[b]), float(rv_t[b])
                _, _, nlive, nref = od.decode_model(
                    c.qa[b * HKV + h][rows], c.qb[b * HKV + h][rows], c.eq[b * HKV + h][rows], ka, kb, ek, va, vb, c.v_scale,
                    c.z[b * HKV + h][rows], depth, rk, rv, n + 1, vmean=c.vmean[b * HKV + h] if depth is not None else None)
                assert c.counts[bh].tolist() == [nlive, nref], (b, h, s_)
    assert worst < (6e-3 if depth is None else 2.0 ** (-depth / 3)), worst


def test_a_row_s_own_cut_and_the_group_s_differ_as_the_model_says():
    from fold_attention_b200.decode.launch import prepare_fold_decode

    D, H, HKV = 64, 16, 2
    G = H // HKV
    lens = [900, 300]
    k, v, cu = _kv(lens, HKV, D, 61)
    c = _cache(lens, H, HKV, D, 61, depth=6.0, tail=None)
    c.write_prompt(k, v, cu, lens)
    q = torch.randn(2, H, D, device="cuda").bfloat16()
    c._step(q, None, None)
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    outs = {}
    for cutmode in (True, False):
        run = prepare_fold_decode(
            c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, split=2, truncate=True, refine_k=8.0, refine_v=8.0, v_scale=1.0,
            vmean=c.vmean, page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV, weight_terms=2,
            group_cut=cutmode)
        out, den, counts = run()
        torch.cuda.synchronize()
        outs[cutmode] = out.clone()
        for b, n in enumerate(lens):
            for h in range(HKV):
                bh = b * HKV + h
                ka, kb, ek, va, vb = _planes(c, b, h, n)
                want, wden, nlive, nref = od.decode_model(c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, va, vb, 1.0, z[bh], 6.0, 8.0, 8.0, n,
                                                          vmean=c.vmean[bh], row_cut=not cutmode)
                assert counts[bh].tolist() == [nlive, nref]
                assert _l2(out[bh], want) < 2e-3, (cutmode, b, h)
                assert ((den[bh].double() - wden).abs() / wden).max().item() < 2e-3
    assert not torch.equal(outs[True], outs[False])       # the control: the two cuts are different functions


def test_the_levels_are_refused_where_they_cannot_run():
    fa = _fa()
    from fold_attention_b200.decode.launch import SharedPrefix, prepare_fold_decode

    c = fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, page_size=128)
    kw = dict(page_table=c.page_table, page_size=128, seq_lens=c.seq_lens, n_kv_heads=2, truncate=True)
    args = (c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut)
    with pytest.raises(ValueError, match="not a multiple of draft_len"):
        prepare_fold_decode(*args, draft_len=3, causal=True, **kw)
    with pytest.raises(ValueError, match="two answers"):
        prepare_fold_decode(*args, draft_len=2, causal=True, mask=torch.eye(2, dtype=torch.bool), **kw)
    with pytest.raises(ValueError, match="diagonal"):
        prepare_fold_decode(*args, draft_len=2, mask=torch.tensor([[True, False], [True, False]]), **kw)
    with pytest.raises(NotImplementedError, match="warp-level"):
        prepare_fold_decode(*args, draft_len=2, causal=True, kernel="sm100", **kw)
    with pytest.raises(NotImplementedError, match="without a tail"):
        prepare_fold_decode(*args, draft_len=2, causal=True, tail=c.tail, **kw)
    with pytest.raises(TypeError, match="SharedPrefix"):
        prepare_fold_decode(*args, shared=dict(ka=c.ka), vmean=c.vmean, **kw)
    level = SharedPrefix(c.ka, c.kb, c.ek, c.va, c.page_table, c.seq_lens, 128)
    with pytest.raises(ValueError, match="both levels or neither"):
        prepare_fold_decode(*args, shared=level, vmean=c.vmean, **kw)
    with pytest.raises(ValueError, match="no fixed chunk"):
        prepare_fold_decode(*args, shared=level, chunk_keys=128, **kw)
    with pytest.raises(NotImplementedError, match="16, 24 or 32"):
        fa.FoldKVCache(2, 40, 2, 128, 256)
    with pytest.raises(NotImplementedError, match="warp-level"):
        fa.FoldKVCache(2, 32, 2, 128, 256, kernel="sm100", page_size=128)


@pytest.mark.parametrize("D,G,v8", [(128, 8, False), (64, 4, True)])
def test_a_sound_cut_drops_only_what_the_full_logit_drops(D, G, v8):
    from fold_attention_b200.decode.launch import prepare_fold_decode

    HKV = 2
    lens = [1200, 400]
    k, v, cu = _kv(lens, HKV, D, 71)
    c = _cache(lens, HKV * G, HKV, D, 71, depth=6.0, v8=v8, tail=None, v_scale=2.0 ** -3 if v8 else None)
    c.write_prompt(k, v, cu, lens)
    q = torch.randn(2, HKV * G, D, device="cuda").bfloat16()
    c._step(q, None, None)
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    live = {}
    for snd in (False, True):
        run = prepare_fold_decode(
            c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, split=2, truncate=True, refine_k=8.0, refine_v=8.0, v8=v8, v2=c.vb,
            v_scale=c.v_scale, vmean=c.vmean, page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV,
            weight_terms=2, sound=snd)
        out, den, counts = run()
        torch.cuda.synchronize()
        assert int(run.status) == 0
        live[snd] = counts[:, 0].clone()
        for b, n in enumerate(lens):
            for h in range(HKV):
                bh = b * HKV + h
                ka, kb, ek, va, vb = _planes(c, b, h, n)
                want, wden, nlive, nref = od.decode_model(c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, va, vb, c.v_scale, z[bh], 6.0, 8.0, 8.0, n,
                                                          vmean=c.vmean[bh], sound=snd)
                assert counts[bh].tolist() == [nlive, nref], (snd, b, h)
                assert _l2(out[bh], want) < 2e-3
                if snd:
                    # soundness: a key whose full two-plane logit clears some row's cut is live
                    s1 = od.coarse_logits(c.qa[bh][None], c.qb[bh][None], c.eq[bh][None], ka[None], ek[None], z[bh][None])[0]
                    tk = (c.eq[bh].float()[:, None] * (ek.float()[None, :] / 256.0)).double()
                    full = s1.double() + (torch.einsum("gd,sd->gs", c.qa[bh].double(), kb.double())
                                          + torch.einsum("gd,sd->gs", c.qb[bh].double(), kb.double()) / 256.0) * tk
                    bound = (c.eq[bh].float() * (c.qa[bh].float().abs().sum(-1) * 128.0 + c.qb[bh].float().abs().sum(-1) * 0.5)).double()
                    kept = (s1.double() + bound[:, None] * (ek.double()[None, :] / 256.0) >= -6.0).any(0)
                    assert bool(kept[(full >= -6.0).any(0)].all())
    assert bool((live[True] >= live[False]).all()) and int(live[True].sum()) > int(live[False].sum())


def test_a_direction_per_query_row():
    from fold_attention_b200.decode.launch import prepare_fold_decode

    D, G, HKV = 128, 4, 2
    lens = [900, 250]
    k, v, cu = _kv(lens, HKV, D, 81)
    c = _cache(lens, HKV * G, HKV, D, 81, depth=6.0, tail=None)
    c.write_prompt(k, v, cu, lens)
    q = torch.randn(2, HKV * G, D, device="cuda").bfloat16()
    c._step(q, None, None)
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    vm = torch.randn(2 * HKV, G, D, device="cuda")
    run = prepare_fold_decode(
        c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, split=3, truncate=True, refine_k=8.0, refine_v=8.0, v_scale=1.0, vmean=vm,
        page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV, weight_terms=2)
    out, den, counts = run()
    torch.cuda.synchronize()
    for b, n in enumerate(lens):
        for h in range(HKV):
            bh = b * HKV + h
            ka, kb, ek, va, vb = _planes(c, b, h, n)
            for g in range(G):   # the model takes one direction: a row at a time, with the group's verdicts
                want, _, nlive, nref = od.decode_model(c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, va, vb, 1.0, z[bh], 6.0, 8.0, 8.0, n, vmean=vm[bh, g])
                assert _l2(out[bh, g], want[g]) < 2e-3
            assert counts[bh].tolist() == [nlive, nref]
    with pytest.raises(ValueError, match="one per query row"):
        prepare_fold_decode(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, truncate=True, vmean=vm[:, :2], page_table=c.page_table,
                            page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV)


def test_a_captured_decode_replays_the_launch_it_was_made_from():
    from fold_attention_b200.decode import capture_decode, fold_decode, prepare_fold_decode

    D, H, HKV = 128, 8, 2
    lens = [500, 130]
    k, v, cu = _kv(lens, HKV, D, 91)
    c = _cache(lens, H, HKV, D, 91, depth=8.0, tail=None)
    c.write_prompt(k, v, cu, lens)
    q = torch.randn(2, H, D, device="cuda").bfloat16()
    c._step(q, None, None)
    args = (c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut)
    kw = dict(split=2, truncate=True, v_scale=1.0, vmean=c.vmean, page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens,
              n_kv_heads=HKV, reference="mass", weight_terms=2, sound=True, group_cut=False)
    want = tuple(t.clone() for t in fold_decode(*args, **kw))
    launch = prepare_fold_decode(*args, **kw)
    cap = capture_decode(launch)
    for _ in range(2):
        got = cap()
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    assert int(cap.status) == 0 and cap.kernel == "mma"
    # the bound tensors' contents may change between replays
    q2 = torch.randn(2, H, D, device="cuda").bfloat16()
    c._step(q2, None, None)
    want2 = tuple(t.clone() for t in launch())
    got2 = cap()
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(got2, want2)) and not torch.equal(want2[0], want[0])


def test_a_contiguous_cache_is_its_paged_self():
    """Without a page table the planes are `(NBH, S, D)`; the same keys paged give the same bits,
    with a tail too (`tail_model`, then `paged`)."""
    from fold_attention_b200.decode import prepare_fold_decode, tail_model
    from fold_attention_b200.decode.tail import paged

    D, H, HKV, S = 128, 8, 2, 1024
    B = 3
    k, v, cu = _kv([S] * B, HKV, D, 101)
    c = _cache([S] * B, H, HKV, D, 101, shuffle=True, page_size=128, depth=8.0, tail=None)
    c.write_prompt(k, v, cu, [S] * B)
    q = torch.randn(B, H, D, device="cuda").bfloat16()
    c._step(q, None, None)
    NBH, G = B * HKV, H // HKV
    # the same cache, contiguous: gather every row group's pool rows (a row's swizzle depends on its slot
    # in the page, and page slots repeat every 128: position s sits at slot s % 128, the same 8-period)
    rows = torch.stack([_rows(c, b, h, S)[0] for b in range(B) for h in range(HKV)])          # (NBH, S)
    ka, kb, ek, va = c.ka[rows], c.kb[rows], c.ek[rows], c.va[rows]
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    kw = dict(split=2, truncate=True, refine_k=8.0, refine_v=8.0, v_scale=1.0, weight_terms=2)
    paged_run = prepare_fold_decode(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, vmean=c.vmean, page_table=c.page_table,
                                    page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV, kernel="mma", **kw)
    flat_run = prepare_fold_decode(c.qa, c.qb, c.eq, ka, kb, ek, va, z, c.cut, vmean=c.vmean, kernel="mma", **kw)
    a, b_ = paged_run(), flat_run()
    torch.cuda.synchronize()
    assert all(torch.equal(x, y) for x, y in zip(a, b_))
    # a shorter length per row group, and the tail
    lens = torch.tensor([S, 700, 64, S, 900, 130], device="cuda", dtype=torch.int32)
    t = tail_model(ka, ek, va, rank=16)
    flat_t = prepare_fold_decode(c.qa, c.qb, c.eq, ka, kb, ek, va, z, c.cut, tail=t, seq_lens=lens, **kw)()
    tp = paged(t, c.page_table, c.page_size, HKV, S // 64)
    assert tp.rows.shape[0] == c.ka.shape[0] // 64
    seq = lens.view(B, HKV)
    # paged lengths are per request: compare the row groups whose length is their request's
    c.seq_lens.copy_(seq[:, 0])
    paged_t = prepare_fold_decode(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, tail=tp, page_table=c.page_table,
                                  page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=HKV, **kw)()
    torch.cuda.synchronize()
    for bh in range(0, NBH, HKV):
        assert torch.equal(flat_t[0][bh], paged_t[0][bh])
    with pytest.raises(NotImplementedError, match="multiple of 64"):
        prepare_fold_decode(c.qa, c.qb, c.eq, ka[:, :1000], kb[:, :1000], ek[:, :1000], va[:, :1000], z, c.cut, **kw)
