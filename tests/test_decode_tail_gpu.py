"""The decode tail on the GPU: where it is exact, what it preserves, and that the kernel is the
float64 model of it. The cases follow the reference's own (tests/test_decode.py:2603-2870,
tests/test_kv_cache.py:312-330): V constant inside each 64-key block (the block rows are exact),
V linear in the kernel's own view of K (the rank is exact), the denominator, the split, the page
table, the order mean > block rows > rank, the refusals, and a request's tail not seeing its batch.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import decode as od  # noqa: E402
from oracle import tail as otail  # noqa: E402


def _fa():
    import fold_attention_b200 as fa

    return fa


def _keys(lens, HKV, D, seed):
    """Keys with a real cache's logit spread: N(0,1), 2 % of positions x6."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=g)
    hot = torch.rand(T, 1, 1, device="cuda", generator=g) < 0.02
    return torch.where(hot, k * 6, k).bfloat16(), g


def _cu(lens):
    return torch.tensor([0] + list(np.cumsum(lens)), device="cuda", dtype=torch.int32)


def _rows(c, b, h, n):
    pos = torch.arange(n, device="cuda")
    pg = c.page_table[b, pos // c.page_size].long()
    return (pg * c.n_kv_heads + h) * c.page_size + pos % c.page_size, pos % c.page_size


def _kernel_k(c, b, h, n):
    """Row group (b, h)'s keys as the kernel sees them: plane A times the key's scale."""
    rows, slots = _rows(c, b, h, n)
    return od.unswizzle(c.ka[rows], slots, c.head_dim).float() * c.ek[rows].float()[:, None]


def _case(mode, lens=(2048, 1500), H=16, HKV=2, D=128, rank=16, seed=5, shuffle=True, **kw):
    """A cache whose V is `blocks` (constant inside every 64-key block), `linear` (its block's
    mean plus a rank-`rank` image of K's deviation from its own block mean, K as the kernel sees
    it) or `mixed` (blocks + a rank-6 image + noise). Returns (cache factory, q, k, v, cu)."""
    fa = _fa()
    lens = list(lens)
    B = len(lens)
    k, g = _keys(lens, HKV, D, seed)
    cu = _cu(lens)
    q = torch.randn(B, H, D, device="cuda", generator=g).bfloat16()

    def make(**over):
        c = fa.FoldKVCache(B, H, HKV, D, max(lens) + 200, page_size=over.pop("page_size", 128), **{**kw, **over})
        if shuffle:
            gg = torch.Generator(device="cuda").manual_seed(seed + 99)
            c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=gg).int().view_as(c.page_table))
        return c

    probe = make(depth=8.0, tail=None)
    probe.write_prompt(k, torch.zeros_like(k), cu, lens)
    v = torch.empty(sum(lens), HKV, D, device="cuda")
    for b, n in enumerate(lens):
        nb = -(-n // 64)
        for h in range(HKV):
            blk = (torch.randn(nb, D, device="cuda", generator=g) + 1.5).repeat_interleave(64, 0)[:n]
            x = blk
            if mode != "blocks":
                r = rank if mode == "linear" else 6
                kq = _kernel_k(probe, b, h, n)
                km = torch.from_numpy(np.repeat(otail.block_mean(kq.double().cpu().numpy()), 64, 0)[:n]).to(kq)
                a = torch.randn(D, r, device="cuda", generator=g) / D ** 0.5
                bm = torch.randn(r, D, device="cuda", generator=g)
                x = x + (kq - km) @ a @ bm * (4.0 if mode == "linear" else 2.0)
            if mode == "mixed":
                x = x + 0.5 * torch.randn(n, D, device="cuda", generator=g)
            v[int(cu[b]):int(cu[b + 1]), h] = x
    return make, q, k, v.bfloat16(), cu, lens


def _reference_z(c):
    """Each row's exact log-sum-exp (base 2) on the cache's coarse logits."""
    z = torch.empty_like(c.z)
    for b, n in enumerate(c.lens):
        for h in range(c.n_kv_heads):
            bh = b * c.n_kv_heads + h
            rows, slots = _rows(c, b, h, n)
            ka = od.unswizzle(c.ka[rows], slots, c.head_dim)
            s = od.coarse_logits(c.qa[bh][None], c.qb[bh][None], c.eq[bh][None], ka[None], c.ek[rows].float()[None])[0]
            z[bh] = torch.logsumexp(s.double() * np.log(2.0), -1).float() / np.log(2.0)
    return z


def _run(c, z, T, *, tail="own", vmean=False, split=2, chunk=0, weight_terms=2, rk=10.0):
    from fold_attention_b200.decode.launch import prepare_fold_decode

    cut = torch.full_like(c.z, float(T))
    run = prepare_fold_decode(
        c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, cut, split=split, truncate=True, refine_k=rk, refine_v=rk,
        v_scale=1.0, vmean=c.vmean if vmean else None, tail=c.tail if tail == "own" else tail,
        page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=c.n_kv_heads,
        weight_terms=weight_terms, chunk_keys=chunk)
    out, den, counts = run()
    torch.cuda.synchronize()
    assert int(run.status) == 0
    return out.clone(), den.clone(), counts.clone()


def _full(c, z):
    """The full softmax over the cache's own planes, float64 (depth None keeps every key)."""
    outs = []
    for b, n in enumerate(c.lens):
        for h in range(c.n_kv_heads):
            bh = b * c.n_kv_heads + h
            rows, slots = _rows(c, b, h, n)
            ka, kb = od.unswizzle(c.ka[rows], slots, c.head_dim), od.unswizzle(c.kb[rows], slots, c.head_dim)
            outs.append(od.decode_model(c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, c.ek[rows].float(), c.va[rows].float(),
                                        None, 1.0, z[bh], None, 1e4, 1e4, n)[0])
    return torch.stack(outs)


def _full_kept(c, z, T):
    """The live keys' mass alone at depth T (the model without any re-entry), per row."""
    outs = []
    for b, n in enumerate(c.lens):
        for h in range(c.n_kv_heads):
            bh = b * c.n_kv_heads + h
            rows, slots = _rows(c, b, h, n)
            ka = od.unswizzle(c.ka[rows], slots, c.head_dim)
            s = od.coarse_logits(c.qa[bh][None], c.qb[bh][None], c.eq[bh][None], ka[None], c.ek[rows].float()[None], z[bh][None])[0]
            live = (s >= -T).any(0)
            outs.append(torch.where(live[None], torch.exp2(s.double()), torch.zeros_like(s, dtype=torch.float64)).sum(-1).float())
    return torch.stack(outs)


def _l2(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def _filled(make, q, k, v, cu, lens, **over):
    c = make(**over)
    c.write_prompt(k, v, cu, lens)
    c._step(q, None, None)      # Q's planes and the mass reference
    return c


@pytest.mark.parametrize("D,G,rank,terms", [(128, 8, 16, 2), (128, 4, 0, 1), (64, 8, 16, 1), (64, 2, 0, 2), (128, 1, 16, 1)])
def test_the_kernel_is_the_tail_s_model(D, G, rank, terms):
    """Against the float64 model with every dropped key re-entering at its block's row plus its
    projection mapped back, on the cache's own planes and the tail the cache holds."""
    HKV = 2
    make, q, k, v, cu, lens = _case("mixed", lens=(1500, 700, 64, 2049), H=HKV * G, HKV=HKV, D=D, depth=8.0, tail=rank)
    c = _filled(make, q, k, v, cu, lens)
    assert c.tail.rank == rank
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    for split, chunk in ((1, 0), (3, 0), (0, 512)):
        sp = split if not chunk else -(-max(lens) // chunk)
        out, den, counts = _run(c, z, 8.0, split=sp, chunk=chunk, weight_terms=terms)
        for b, n in enumerate(lens):
            for h in range(HKV):
                bh = b * HKV + h
                rows, slots = _rows(c, b, h, n)
                ka, kb = od.unswizzle(c.ka[rows], slots, D), od.unswizzle(c.kb[rows], slots, D)
                ek = c.ek[rows].float()
                blk_rows = c.tail.rows[rows[::64] // 64].float().cpu().numpy()
                re = otail.reentry(ka.cpu().numpy(), ek.cpu().numpy(),
                                   c.tail.u[bh].cpu().numpy() if rank else None,
                                   c.tail.vr[bh].cpu().numpy() if rank else None, blk_rows)
                want, wden, nlive, nref = od.decode_model(
                    c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, c.va[rows].float(), None, 1.0, z[bh], 8.0, 10.0, 10.0, n,
                    reentry=torch.from_numpy(re))
                assert counts[bh].tolist() == [nlive, nref], (split, chunk, b, h)
                assert nlive < n or n <= 64
                assert _l2(out[bh], want) < 3e-3, (split, chunk, b, h, _l2(out[bh], want))
                # one bf16 weight term rounds each live key's weight in the denominator too
                assert ((den[bh].double() - wden).abs() / wden).max().item() < (2e-3 if terms == 2 else 6e-3)


def test_the_tail_is_exact_where_v_is_its_block_mean():
    make, q, k, v, cu, lens = _case("blocks", depth=8.0, tail=0)
    c = _filled(make, q, k, v, cu, lens)
    z = _reference_z(c)
    full = _full(c, z)
    dense = _l2(_run(c, z, 1e4)[0], full)
    for T in (4.0, 6.0):
        tail = _l2(_run(c, z, T)[0], full)
        mean = _l2(_run(c, z, T, tail=None, vmean=True)[0], full)
        assert tail < 1.1 * dense + 1e-3, (T, tail, dense)
        assert mean > 3 * tail, (T, mean, tail)       # the control: one mean per head is far off on the same cache
        assert _run(c, z, T)[2][:, 0].sum().item() < 0.5 * sum(lens) * c.n_kv_heads      # the cut really drops keys


def test_the_rank_is_exact_where_v_is_linear_in_k():
    make, q, k, v, cu, lens = _case("linear", depth=8.0, tail=16)
    c = _filled(make, q, k, v, cu, lens)
    c0 = _filled(make, q, k, v, cu, lens, tail=0)
    z = _reference_z(c)
    full = _full(c, z)
    dense = _l2(_run(c, z, 1e4)[0], full)
    for T in (6.0, 8.0):
        got = _l2(_run(c, z, T)[0], full)
        blk = _l2(_run(c0, z, T)[0], full)
        assert got < 1.15 * dense + 2e-3, (T, got, dense)
        assert blk > 3 * got, (T, blk, got)


@pytest.mark.parametrize("rank", [0, 16])
def test_the_tail_denominator_is_the_total_mass(rank):
    make, q, k, v, cu, lens = _case("mixed", depth=8.0, tail=rank)
    c = _filled(make, q, k, v, cu, lens)
    z = _reference_z(c)           # the coarse logits' log-sum-exp: the total mass is near 1
    total = _run(c, z, 1e4)[1]    # every key kept: the whole softmax's mass on the refined logits
    den = _run(c, z, 8.0)[1]
    assert ((den - total).abs() / total).max().item() < 1e-2
    assert (total - 1.0).abs().max().item() < 0.15
    # the control: at depth 4 the kept mass alone is visibly short of it
    make0 = _run(c, z, 4.0)
    kept = _full_kept(c, z, 4.0)
    assert ((kept - total).abs() / total).max().item() > 2e-3
    assert ((make0[1] - total).abs() / total).max().item() < 2e-2


@pytest.mark.parametrize("split", [1, 3, 4])
def test_the_tail_survives_the_split(split):
    make, q, k, v, cu, lens = _case("mixed", depth=8.0, tail=16)
    c = _filled(make, q, k, v, cu, lens)
    z = _reference_z(c)
    base = _run(c, z, 8.0, split=2)[0]
    got = _run(c, z, 8.0, split=split)[0]
    assert (got - base).abs().max().item() / base.abs().max().item() < 1e-5


def test_the_tail_is_ordered_by_what_it_knows():
    make, q, k, v, cu, lens = _case("mixed", depth=8.0, tail=16)
    c = _filled(make, q, k, v, cu, lens)
    c0 = _filled(make, q, k, v, cu, lens, tail=0)
    z = _reference_z(c)
    full = _full(c, z)
    mean = _l2(_run(c, z, 8.0, tail=None, vmean=True)[0], full)
    blk = _l2(_run(c0, z, 8.0)[0], full)
    rk = _l2(_run(c, z, 8.0)[0], full)
    assert blk < mean, (blk, mean)
    assert rk < blk, (rk, blk)


@pytest.mark.parametrize("n", [1024, 5000])
def test_the_tail_pages_like_the_contiguous_call(n):
    """A shuffled page table and pages of another size change no bit: a block row lives at its
    first key's pool row over 64."""
    outs = []
    for shuffle, ps in ((False, 128), (True, 128), (True, 256), (True, 64)):
        make, q, k, v, cu, lens = _case("mixed", lens=(n, 700), depth=8.0, tail=16, shuffle=shuffle)
        c = _filled(make, q, k, v, cu, lens, page_size=ps)
        z = (torch.ceil(c.z * 16) / 16).contiguous()
        outs.append(_run(c, z, 8.0, split=0 + 3)[0])
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


def test_a_request_s_tail_does_not_see_its_batch():
    make, q, k, v, cu, lens = _case("mixed", lens=(900, 333, 1200), depth=8.0, tail=16)
    together = _filled(make, q, k, v, cu, lens)
    assert together.tail_rank == 16
    fa = _fa()
    HKV = together.n_kv_heads
    for b, n in enumerate(lens):
        one = fa.FoldKVCache(1, together.n_heads, HKV, together.head_dim, n + 200, page_size=128, depth=8.0, tail=16)
        a = int(cu[b])
        one.write_prompt(k[a:a + n], v[a:a + n], _cu([n]), [n])
        assert torch.equal(one.tail.u, together.tail.u[b * HKV:(b + 1) * HKV])
        assert torch.equal(one.tail.vr, together.tail.vr[b * HKV:(b + 1) * HKV])
        for h in range(HKV):
            r1, _ = _rows(one, 0, h, n)
            r2, _ = _rows(together, b, h, n)
            assert torch.equal(one.tail.rows[r1[::64] // 64], together.tail.rows[r2[::64] // 64])


@pytest.mark.parametrize("rank,dtype", [(16, torch.bfloat16), (0, torch.bfloat16), (16, torch.float16)])
def test_the_append_keeps_the_blocks_current(rank, dtype):
    """After 150 appended tokens (new blocks, a new page) every block's sums and row are what the
    step's arithmetic gives from the cache's own planes and the prompt's map."""
    fa = _fa()
    make, q, k, v, cu, lens = _case("mixed", lens=(300, 1000), H=8, HKV=2, D=128, depth=8.0, tail=rank)
    c = make()
    c.write_prompt(k, v, cu, lens)
    u0 = c.tail.u.clone() if rank else None
    g = torch.Generator(device="cuda").manual_seed(11)
    vs = [v[int(cu[b]):int(cu[b + 1])].float() for b in range(2)]
    for step in range(150):
        kn = torch.randn(2, 2, 128, device="cuda", generator=g).to(dtype)
        vn = (torch.randn(2, 2, 128, device="cuda", generator=g) + 1.0).to(dtype)
        qn = torch.randn(2, 8, 128, device="cuda", generator=g).to(dtype)
        out = c.decode(qn, kn, vn)
        assert torch.isfinite(out).all()
        for b in range(2):
            vs[b] = torch.cat([vs[b], vn[b].float()[None]])
    if rank:
        assert torch.equal(c.tail.u, u0)       # the map is the prompt's
    from fold_attention_b200.decode import tail as ptail

    for b in range(2):
        n = c.lens[b]
        for h in range(2):
            bh = b * 2 + h
            rows, slots = _rows(c, b, h, n)
            blk = rows[::64] // 64
            vsum, cnt = ptail.block_sums(vs[b][:, h][None])
            assert torch.allclose(c.tail.vsum[blk], vsum[0], rtol=1e-5, atol=1e-4)
            want = vsum[0] / cnt[:, None].float()
            if rank:
                kint = od.unswizzle(c.ka[rows], slots, 128).float()
                y = ptail.project(kint[None], c.ek[rows][None], c.tail.u[bh][None])
                ysum, _ = ptail.block_sums(y)
                assert torch.allclose(c.tail.ysum[blk], ysum[0], rtol=1e-4, atol=1e-3)
                want = want - (ysum[0] / cnt[:, None].float()) @ c.tail.vr[bh].T
            assert torch.allclose(c.tail.rows[blk].float(), want, rtol=2.0 ** -7, atol=2e-2)


def _serving_errors(mode, depth):
    make, q, k, v, cu, lens = _case(mode, depth=depth)
    errs = {}
    for name, tl in (("auto", "auto"), ("rows", 0), ("mean", None)):
        c = make(tail=tl)
        c.write_prompt(k, v, cu, lens)
        got = c.attend(q)
        G = c.group
        want = torch.stack([
            torch.cat([od.attend_fp32(q[b, h * G:(h + 1) * G].float(), k[int(cu[b]):int(cu[b + 1]), h].float(),
                                      v[int(cu[b]):int(cu[b + 1]), h].float()) for h in range(c.n_kv_heads)])
            for b in range(len(lens))])
        errs[name] = _l2(got, want)
        if name == "auto":
            assert c.tail_rank == 16 and c.kernel == "mma"
        assert c.counts[:, 0].sum().item() < 0.2 * sum(lens) * c.n_kv_heads       # the depth really drops keys
    return errs


def test_serving_with_the_tail_beats_serving_without_it():
    """End to end through FoldKVCache at depth 4 against FP32 attention: where V is its block's
    mean plus a K-linear part plus noise the default tail (rank 16) is far under V's mean, and
    where V is constant inside blocks the block rows alone already are."""
    errs = _serving_errors("mixed", 4.0)
    assert errs["auto"] < 0.5 * errs["mean"], errs
    assert errs["rows"] < 1.05 * errs["mean"], errs
    errs = _serving_errors("blocks", 4.0)
    assert errs["rows"] < 0.6 * errs["mean"], errs
    assert errs["auto"] < 0.6 * errs["mean"], errs


def test_the_tail_is_refused_where_it_cannot_run():
    fa = _fa()
    from fold_attention_b200.decode.launch import prepare_fold_decode

    with pytest.raises(ValueError, match="truncates nothing"):
        fa.FoldKVCache(2, 8, 2, 128, 256, tail=16)
    with pytest.raises(ValueError, match="bf16 V cache"):
        fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, v8=True, tail=16)
    with pytest.raises(ValueError, match="whole blocks"):
        fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, tail=16, page_size=32)
    with pytest.raises(ValueError, match="tail rank"):
        fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, tail=12)
    with pytest.raises(NotImplementedError, match="warp-level"):
        fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, tail=16, kernel="sm100", page_size=128)
    # the policy: rank 16 for these groups on a bf16 V at a finite depth, none otherwise
    assert fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0).tail_rank == 16
    assert fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, v8=True).tail_rank == -1
    assert fa.FoldKVCache(2, 8, 2, 128, 256).tail_rank == -1
    assert fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, page_size=32).tail_rank == -1
    c = fa.FoldKVCache(2, 8, 2, 128, 256, depth=12.0, page_size=128)
    kw = dict(page_table=c.page_table, page_size=128, seq_lens=c.seq_lens, n_kv_heads=2)
    args = (c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut)
    with pytest.raises(ValueError, match="needs truncate"):
        prepare_fold_decode(*args, tail=c.tail, **kw)
    with pytest.raises(ValueError, match="replaces vmean"):
        prepare_fold_decode(*args, tail=c.tail, truncate=True, vmean=c.vmean, **kw)
    with pytest.raises(NotImplementedError, match="warp-level"):
        prepare_fold_decode(*args, tail=c.tail, truncate=True, kernel="sm100", **kw)
    import dataclasses

    bad = dataclasses.replace(c.tail, rows=c.tail.rows[:-1])
    with pytest.raises(ValueError, match="one per 64 pool rows"):
        prepare_fold_decode(*args, tail=bad, truncate=True, **kw)


def test_a_replayed_step_leaves_the_tail_as_it_found_it():
    make, q, k, v, cu, lens = _case("mixed", lens=(640, 300), H=8, HKV=2, depth=8.0)
    c = make()
    c.write_prompt(k, v, cu, lens)
    g = torch.Generator(device="cuda").manual_seed(3)
    kn = torch.randn(2, 2, 128, device="cuda", generator=g).bfloat16()
    vn = torch.randn(2, 2, 128, device="cuda", generator=g).bfloat16()
    qn = torch.randn(2, 8, 128, device="cuda", generator=g).bfloat16()
    step = c.prepare_replay_step(qn, kn, vn)
    first = step()[0].clone()
    for _ in range(3):
        again = step()[0]
    assert torch.equal(first, again)
    # and it is the step the cache itself takes
    got = c.decode(qn, kn, vn)
    assert torch.equal(got.float(), first.float().to(got.dtype).float())
