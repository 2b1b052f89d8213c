"""The tcgen05 split-KV decode kernel (`kernel="sm100"`) against the float64
model of the cache's own planes (oracle/decode.py), against the warp-level
kernel, and against itself (bit-repeatability, batch invariance under a fixed
chunk). Gates are chosen so that each of its paths carries keys: the tensor-core
stream, the whole-quarter plane B of V, and the helper warps (refine-K keys,
sparse refine-V keys, weights past the E5M2 range)."""
import pytest
import torch

from oracle import decode as od
from test_decode_gpu import _cache, _layer, _planes, _rel

pytestmark = pytest.mark.gpu

# (refine_k, refine_v): the defaults' shape, tight gates, plane B of V nearly everywhere
# (whole quarters), no refinement at all (a weight far past 2^8 still has to come out right)
GATES = [(10.0, 10.0), (3.0, 3.0), (2.0, 14.0), (-1e9, 1e9), (-1e9, -1e9)]


def _launch(c, z, *, depth, rk, rv, split, chunk, HKV, ps, kernel):
    from fold_attention_b200.decode.launch import prepare_fold_decode

    return prepare_fold_decode(
        c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, z, c.cut, split=split,
        truncate=depth is not None, refine_k=rk, refine_v=rv, v8=c.v8, v2=c.vb, v_scale=c.v_scale,
        vmean=c.vmean, page_table=c.page_table, page_size=ps, seq_lens=c.seq_lens,
        n_kv_heads=HKV, weight_terms=2, chunk_keys=chunk, kernel=kernel,
    )


@pytest.mark.parametrize("v8", [True, False])
@pytest.mark.parametrize("depth", [None, 16.0, 8.0])
@pytest.mark.parametrize("ps,G,lens,split,chunk", [
    (256, 8, [1500, 700, 64, 2049], 1, 0),
    (256, 8, [1500, 700, 64, 2049], 3, 0),     # ranges without a key: 64 keys over 3 splits
    (128, 4, [300, 1, 129, 1000], 2, 0),
    (256, 1, [513, 2000], 0, 512),
    (256, 2, [5000, 100], 0, 1024),
])
def test_the_tcgen05_kernel_is_the_model(depth, ps, G, lens, split, chunk, v8):
    HKV, D = 2, 128
    B = len(lens)
    q, k, v, cu = _layer(B, HKV * G, HKV, D, lens, seed=2, vmu=0.5)
    c = _cache(B, HKV * G, HKV, D, lens, ps=ps, v8=v8, depth=depth)
    c.write_prompt(k, v, cu, lens)
    c.attend(q)
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    sp = split if not chunk else -(-max(lens) // chunk)
    for rk, rv in GATES:
        run = _launch(c, z, depth=depth, rk=rk, rv=rv, split=sp, chunk=chunk, HKV=HKV, ps=ps, kernel="sm100")
        out, den, counts = run()
        torch.cuda.synchronize()
        assert int(run.status) == 0
        first = (out.clone(), den.clone(), counts.clone())
        for _ in range(8):   # the same bits on every run, whatever the warps' timing
            out, den, counts = run()
            torch.cuda.synchronize()
            assert torch.equal(out, first[0]) and torch.equal(den, first[1]) and torch.equal(counts, first[2])
        ref = _launch(c, z, depth=depth, rk=rk, rv=rv, split=sp, chunk=chunk, HKV=HKV, ps=ps, kernel="mma")
        _, _, counts_mma = ref()
        torch.cuda.synchronize()
        assert torch.equal(counts, counts_mma)
        for b in range(B):
            for h in range(HKV):
                bh = b * HKV + h
                ka, kb, ek, va, vb = _planes(c, b, h, lens[b])
                want, wden, nlive, nref = od.decode_model(
                    c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, va, vb, c.v_scale, z[bh], depth,
                    rk, rv, lens[b], vmean=c.vmean[bh] if depth is not None else None)
                assert counts[bh].tolist() == [nlive, nref], (rk, rv, b, h)
                # weights are 12-bit (four E5M2 terms off an fp16; 16-bit, two bf16 terms, on a bf16 V)
                assert _rel(out[bh], want) < 1e-3, (rk, rv, b, h, _rel(out[bh], want))
                assert ((den[bh].double() - wden).abs() / wden).max().item() < 1e-3


@pytest.mark.parametrize("v8", [True, False])
def test_what_the_pool_holds_past_a_requests_end_changes_no_bit(v8):
    """The kernel reads whole tiles; the rows of a last, partial tile past the request's end hold
    whatever the pool holds. Filled with 0xFF (an E4M3 NaN, a bf16 NaN, -1 in the int8 planes) in
    every plane they must leave every bit of the result as it was: the stream's V rows, the
    plane-B quarters of V and both planes of K are all read there."""
    HKV, G, D, ps = 2, 8, 128, 256
    lens = [1500, 700, 64, 2049, 9000]
    B = len(lens)
    q, k, v, cu = _layer(B, HKV * G, HKV, D, lens, seed=4, vmu=0.5)
    c = _cache(B, HKV * G, HKV, D, lens, ps=ps, v8=v8, depth=16.0)
    c.write_prompt(k, v, cu, lens)
    c.attend(q)
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    lens_now = [int(n) for n in c.seq_lens.tolist()]
    for rk, rv in [(10.0, 10.0), (2.0, 14.0), (14.0, 14.0)]:
        run = _launch(c, z, depth=16.0, rk=rk, rv=rv, split=1, chunk=0, HKV=HKV, ps=ps, kernel="sm100")
        out, den, counts = (t.clone() for t in run())
        torch.cuda.synchronize()
        saved = {}
        for b in range(B):
            n = lens_now[b]
            last = -(-n // ps) * ps            # the end of the request's last page
            if last == n:
                continue
            for h in range(HKV):
                pos = torch.arange(n, last, device="cuda")
                pg = c.page_table[b, pos // ps].long()
                rows = (pg * HKV + h) * ps + pos % ps
                for name in ("ka", "kb", "ek", "va", "vb"):
                    t = getattr(c, name)
                    if t is None:
                        continue
                    raw = t.view(torch.uint8).view(t.shape[0], -1)
                    saved[(b, h, name)] = (rows, raw[rows].clone())
                    raw[rows] = 0xFF
        assert saved
        out2, den2, counts2 = run()
        torch.cuda.synchronize()
        assert int(run.status) == 0
        assert torch.isfinite(out2).all() and torch.isfinite(den2).all()
        assert torch.equal(out2, out) and torch.equal(den2, den) and torch.equal(counts2, counts), (rk, rv)
        for (b, h, name), (rows, old) in saved.items():
            t = getattr(c, name)
            t.view(torch.uint8).view(t.shape[0], -1)[rows] = old


def test_the_cache_serves_through_either_kernel():
    """FoldKVCache with kernel="sm100": append + attend tracks the softmax, a
    request's output under a fixed chunk is the same bits alone and in a batch."""
    lens = [3000, 1000, 5000]
    B, H, HKV, D = len(lens), 16, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=6)
    kw = dict(ps=128, v8=True, depth=16.0, chunk=1024, v_scale=0.03125)
    full = _cache(B, H, HKV, D, lens, kernel="sm100", **kw)
    full.write_prompt(k, v, cu, lens)
    o_full = full.attend(q)
    cnt_full = full.counts.clone()
    other = _cache(B, H, HKV, D, lens, kernel="mma", seed=3, **kw)
    other.write_prompt(k, v, cu, lens)
    o_mma = other.attend(q)
    assert torch.equal(cnt_full, other.counts)
    assert _rel(o_full.float(), o_mma.float()) < 2e-3
    for b in range(B):
        one = _cache(1, H, HKV, D, [lens[b]], seed=b, kernel="sm100", **kw)
        a, e = int(cu[b]), int(cu[b + 1])
        one.write_prompt(k[a:e], v[a:e], torch.tensor([0, lens[b]], device="cuda", dtype=torch.int32), [lens[b]])
        o_one = one.attend(q[b:b + 1])
        assert torch.equal(o_one[0], o_full[b])
        assert torch.equal(one.counts, cnt_full[b * HKV:(b + 1) * HKV])
    # serving steps: the appended token lands in a page the next attend streams
    G = H // HKV
    ks = [k[int(cu[b]):int(cu[b + 1])].float() for b in range(B)]
    vs = [v[int(cu[b]):int(cu[b + 1])].float() for b in range(B)]
    c = _cache(B, H, HKV, D, [n + 8 for n in lens], ps=128, v8=True, depth=16.0, kernel="sm100")
    c.write_prompt(k, v, cu, lens)
    g = torch.Generator(device="cuda").manual_seed(9)
    for step in range(6):
        qn = torch.randn(B, H, D, device="cuda", generator=g).bfloat16()
        kn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
        vn = torch.randn(B, HKV, D, device="cuda", generator=g).bfloat16()
        got = c.decode(qn, kn, vn)
        for b in range(B):
            ks[b] = torch.cat([ks[b], kn[b].float()[None]])
            vs[b] = torch.cat([vs[b], vn[b].float()[None]])
    want = torch.stack([
        torch.cat([od.attend_fp32(qn[b, h * G:(h + 1) * G].float(), ks[b][:, h], vs[b][:, h]) for h in range(HKV)])
        for b in range(B)])
    assert _rel(got.float(), want) < 2.0 ** (-16.0 / 3)   # the bound the depth test uses


def test_what_the_tcgen05_kernel_does_not_take():
    from fold_attention_b200.decode.launch import prepare_fold_decode

    lens = [300]
    q, k, v, cu = _layer(1, 8, 2, 128, lens, seed=1)
    c = _cache(1, 8, 2, 128, lens, ps=64, v8=True)   # pages of 64 keys
    c.write_prompt(k, v, cu, lens)
    c.attend(q)
    with pytest.raises(NotImplementedError, match="multiple of 128"):
        _launch(c, c.z, depth=None, rk=10.0, rv=10.0, split=1, chunk=0, HKV=2, ps=64, kernel="sm100")
    with pytest.raises(ValueError, match="kernel is one of"):
        _launch(c, c.z, depth=None, rk=10.0, rv=10.0, split=1, chunk=0, HKV=2, ps=64, kernel="wgmma")
    # "auto" falls back to the warp-level kernel where the tcgen05 one does not apply
    run = _launch(c, c.z, depth=None, rk=10.0, rv=10.0, split=1, chunk=0, HKV=2, ps=64, kernel="auto")
    run()
    torch.cuda.synchronize()
    assert int(run.status) == 0


def test_a_batch_splits_between_the_kernels_by_request_length():
    """kernel="auto" with mix_kernels under a chunk: the short requests' slots go to
    the warp-level kernel, the long ones' to the tcgen05 kernel, one combine after
    both; every request's output is the bits its own kernel gives it alone."""
    from fold_attention_b200 import FoldKVCache

    lens = [13000, 500, 12288, 1500]
    B, H, HKV, D = len(lens), 16, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=11)
    kw = dict(ps=128, v8=True, depth=16.0, chunk=2048, v_scale=0.03125)
    both = _cache(B, H, HKV, D, lens, kernel="auto", **kw)
    both.mix_kernels = True
    both.write_prompt(k, v, cu, lens)
    o = both.attend(q)
    launch = next(iter(both._launches.values()))
    assert launch.kernel == "sm100+mma" and int(launch.status) == 0
    assert both.order.tolist()[:4] == [2, 3, 6, 7]   # the two short requests' row groups first
    for b in range(B):
        kern = "sm100" if lens[b] >= FoldKVCache.SM100_MIN_KEYS else "mma"
        one = _cache(1, H, HKV, D, [lens[b]], seed=b, kernel=kern, **kw)
        a, e = int(cu[b]), int(cu[b + 1])
        one.write_prompt(k[a:e], v[a:e], torch.tensor([0, lens[b]], device="cuda", dtype=torch.int32), [lens[b]])
        o_one = one.attend(q[b:b + 1])
        assert torch.equal(o_one[0], o[b]), b
        assert torch.equal(one.counts, both.counts[b * HKV:(b + 1) * HKV])
    # a batch of short requests only: the warp-level kernel takes all of it
    short = _cache(2, H, HKV, D, [500, 1500], kernel="auto", **kw)
    short.mix_kernels = True
    short.write_prompt(torch.cat([k[13000:13500], k[-1500:]]), torch.cat([v[13000:13500], v[-1500:]]),
                       torch.tensor([0, 500, 2000], device="cuda", dtype=torch.int32), [500, 1500])
    short.attend(q[[1, 3]])
    assert next(iter(short._launches.values())).kernel == "mma"


@pytest.mark.parametrize("v8", [False, True])
def test_dense_gates_follow_each_requests_length_on_both_kernels(v8):
    """depth=None with the default gates: the kernel moves each request to its own length band
    (edges 5793 and 23170 keys); both kernels count the same refined keys and track the softmax."""
    from test_decode_gpu import _attend_ref

    lens = [3000, 7000, 25000]
    B, H, HKV, D = len(lens), 8, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=21)
    want = torch.stack([_attend_ref(q, k, v, cu, b, HKV, H // HKV) for b in range(B)])
    outs = {}
    for kernel in ("mma", "sm100"):
        c = _cache(B, H, HKV, D, lens, ps=256, v8=v8, kernel=kernel, seed=5)
        assert c._banded()
        c.write_prompt(k, v, cu, lens)
        outs[kernel] = (c.attend(q), c.counts.clone())
        assert next(iter(c._launches.values())).kernel == kernel
        assert _rel(outs[kernel][0], want) < 4e-3, (kernel, _rel(outs[kernel][0], want))
        assert int(c.counts[:, 0].sum()) == sum(lens) * HKV   # every key is live
    assert torch.equal(outs["mma"][1], outs["sm100"][1])
    assert _rel(outs["sm100"][0].float(), outs["mma"][0].float()) < 2e-3


@pytest.mark.parametrize("seed", list(range(10)))
def test_seeded_random_shapes_match_the_model(seed):
    """Group width, page size, lengths, split or chunk, depth, gates and V type drawn from a
    seed: counts equal the model's, outputs within the weight format's error, twice the same."""
    import random

    rng = random.Random(1000 + seed)
    HKV, D = rng.choice([1, 2, 3]), 128
    G = rng.choice([1, 2, 3, 4, 5, 6, 7, 8])
    ps = rng.choice([128, 256, 384, 512])
    B = rng.choice([1, 2, 3, 5])
    lens = [rng.choice([1, 17, 127, 128, 129, 640, 1000, 2304, 3001, 4500]) for _ in range(B)]
    v8 = rng.random() < 0.6
    depth = rng.choice([None, 6.0, 12.0, 16.0, 20.0])
    if rng.random() < 0.5:
        split, chunk = rng.choice([1, 2, 3, 5, 9]), 0
    else:
        split, chunk = 0, rng.choice([128, 384, 1024, 2048])
    rk, rv = rng.choice([(10.0, 12.0), (12.0, 8.0), (4.0, 16.0), (0.0, 0.0), (1e9, 1e9)])
    q, k, v, cu = _layer(B, HKV * G, HKV, D, lens, seed=seed, vmu=rng.choice([0.0, 0.5]))
    c = _cache(B, HKV * G, HKV, D, lens, ps=ps, v8=v8, depth=depth, seed=seed)
    c.write_prompt(k, v, cu, lens)
    c.attend(q)
    z = (torch.ceil(c.z * 16) / 16).contiguous()
    sp = split if not chunk else -(-max(lens) // chunk)
    run = _launch(c, z, depth=depth, rk=rk, rv=rv, split=sp, chunk=chunk, HKV=HKV, ps=ps, kernel="sm100")
    out, den, counts = run()
    torch.cuda.synchronize()
    assert int(run.status) == 0
    first = (out.clone(), den.clone(), counts.clone())
    for _ in range(4):
        out, den, counts = run()
        torch.cuda.synchronize()
        assert torch.equal(out, first[0]) and torch.equal(den, first[1]) and torch.equal(counts, first[2])
    for b in range(B):
        for h in range(HKV):
            bh = b * HKV + h
            ka, kb, ek, va, vb = _planes(c, b, h, lens[b])
            want, wden, nlive, nref = od.decode_model(
                c.qa[bh], c.qb[bh], c.eq[bh], ka, kb, ek, va, vb, c.v_scale, z[bh], depth,
                rk, rv, lens[b], vmean=c.vmean[bh] if depth is not None else None)
            assert counts[bh].tolist() == [nlive, nref], (b, h)
            assert _rel(out[bh], want) < 1e-3, (b, h, _rel(out[bh], want))
            assert ((den[bh].double() - wden).abs() / wden).max().item() < 1e-3


@pytest.mark.parametrize("kernel", ["mma", "sm100"])
def test_an_attend_step_replays_from_a_cuda_graph(kernel):
    """Q's planes, the mass reference, the decode and the combine are stream-ordered launches
    with no host synchronisation between them: a step captured once replays on new queries."""
    lens = [1500, 3000]
    B, H, HKV, D = len(lens), 16, 2, 128
    q, k, v, cu = _layer(B, H, HKV, D, lens, seed=31)
    c = _cache(B, H, HKV, D, lens, ps=128, v8=True, depth=16.0, kernel=kernel)
    c.write_prompt(k, v, cu, lens)
    q_static = q.clone()
    c.attend(q_static)                      # binds the launches and their buffers
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            out_static = c.attend(q_static)
    torch.cuda.synchronize()
    q2 = torch.randn_like(q)
    want = c.attend(q2).clone()
    q_static.copy_(q2)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_static, want)
    q_static.copy_(q)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_static, c.attend(q))


def test_config4_full_size_properties():
    """Config 4 at its own size (dense bf16 V, B128, H32/8, D128, lengths U[1024, 32768], pages
    shuffled): two serving steps through each kernel. The tcgen05 kernel repeats its bits, counts
    the keys the warp-level kernel counts, agrees with it, and sampled requests match FP32
    attention over everything written."""
    from fold_attention_b200 import FoldKVCache

    B, H, HKV, D = 128, 32, 8, 128
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(1024, 32769, (B,), generator=g).tolist()
    gd = torch.Generator(device="cuda").manual_seed(6)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=gd)
    hot = torch.rand(T, 1, 1, device="cuda", generator=gd) < 0.01
    k = torch.where(hot, k * 8, k).bfloat16()
    v = torch.randn(T, HKV, D, device="cuda", generator=gd).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    steps = [tuple(torch.randn(B, h, D, device="cuda", generator=gd).bfloat16() for h in (H, HKV, HKV)) for _ in range(2)]
    outs = {}
    for kernel in ("sm100", "mma"):
        c = FoldKVCache(B, H, HKV, D, max(lens) + 4, device="cuda", kernel=kernel)
        c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).int().view_as(c.page_table))
        c.write_prompt(k, v, cu, lens)
        res = [c.decode(q, kn, vn) for q, kn, vn in steps]
        assert next(iter(c._launches.values())).kernel == kernel
        outs[kernel] = (res, c.counts.clone())
        if kernel == "sm100":
            again = c.attend(steps[-1][0])      # the cache as it stands, the same query
            assert torch.equal(again, res[-1])
            assert int(next(iter(c._launches.values())).status) == 0
            keep = c
    assert torch.equal(outs["sm100"][1], outs["mma"][1])
    for a, b in zip(outs["sm100"][0], outs["mma"][0]):
        assert _rel(a.float(), b.float()) < 2e-3
    G = H // HKV
    q, kn, vn = steps[-1]
    for b in (0, 17, 127):
        a, e = int(cu[b]), int(cu[b + 1])
        for h in (0, 7):
            ks = torch.cat([k[a:e, h], steps[0][1][b, h][None], kn[b, h][None]]).float()
            vs = torch.cat([v[a:e, h], steps[0][2][b, h][None], vn[b, h][None]]).float()
            want = od.attend_fp32(q[b, h * G:(h + 1) * G].float(), ks, vs)
            assert _rel(outs["sm100"][0][-1][b, h * G:(h + 1) * G], want) < 4e-3, (b, h)
    assert keep.lens == [n + 2 for n in lens]


def test_config5_shape_properties():
    """Config 5's shape (v8, depth 16, H64/8, D128, lengths log-uniform in [4096, 131072], 1 % of
    keys x 8, 0.1 % of V entries x 20) at 32 of its 256 requests (the full batch runs in bench.py):
    the tcgen05 kernel repeats its bits, counts the warp-level kernel's live and refined keys,
    agrees with it, and sampled requests stay inside the depth's error bound against FP32
    attention."""
    import math

    from fold_attention_b200 import FoldKVCache

    B, H, HKV, D = 32, 64, 8, 128
    g = torch.Generator().manual_seed(5)
    lens = [int(math.exp(x)) for x in (torch.rand(B, generator=g) * (math.log(131072) - math.log(4096)) + math.log(4096))]
    gd = torch.Generator(device="cuda").manual_seed(6)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=gd)
    hot = torch.rand(T, 1, 1, device="cuda", generator=gd) < 0.01
    k = torch.where(hot, k * 8, k).bfloat16()
    v = torch.randn(T, HKV, D, device="cuda", generator=gd)
    big = torch.rand(T, HKV, D, device="cuda", generator=gd) < 0.001
    v = torch.where(big, v * 20, v).bfloat16()
    del hot, big
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    q, kn, vn = (torch.randn(B, h, D, device="cuda", generator=gd).bfloat16() for h in (H, HKV, HKV))
    outs = {}
    for kernel in ("sm100", "mma"):
        c = FoldKVCache(B, H, HKV, D, max(lens) + 4, depth=16.0, v8=True, device="cuda", kernel=kernel)
        c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).int().view_as(c.page_table))
        c.write_prompt(k, v, cu, lens)
        out = c.decode(q, kn, vn)
        assert next(iter(c._launches.values())).kernel == kernel
        assert torch.equal(c.attend(q), out)
        assert int(next(iter(c._launches.values())).status) == 0
        outs[kernel] = (out, c.counts.clone())
        del c
    assert torch.equal(outs["sm100"][1], outs["mma"][1])
    assert _rel(outs["sm100"][0].float(), outs["mma"][0].float()) < 2e-3
    G = H // HKV
    short = min(range(B), key=lambda b: lens[b])
    for b in (short, 3):
        a, e = int(cu[b]), int(cu[b + 1])
        for h in (0, 5):
            ks = torch.cat([k[a:e, h], kn[b, h][None]]).float()
            vs = torch.cat([v[a:e, h], vn[b, h][None]]).float()
            want = od.attend_fp32(q[b, h * G:(h + 1) * G].float(), ks, vs)
            assert _rel(outs["sm100"][0][b, h * G:(h + 1) * G], want) < 2.0 ** (-16.0 / 3), (b, h)
