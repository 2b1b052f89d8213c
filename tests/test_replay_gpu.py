"""The cache's replay and tuning helpers (src/fold_attention/kv_cache.py:441-570 of the reference):
repeatable launches on private buffers that a benchmark can capture in a CUDA graph, and the
split tuner built on them."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cache(v8=True, depth=16.0, kernel="auto", lens=(1500, 700, 2049, 64), page_size=128):
    import fold_attention_b200 as fa

    B, H, HKV, D = len(lens), 16, 2, 128
    g = torch.Generator(device="cuda").manual_seed(23)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=g).bfloat16()
    v = (torch.randn(T, HKV, D, device="cuda", generator=g) + 0.3).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    c = fa.FoldKVCache(B, H, HKV, D, max(lens) + 16, page_size=page_size, v8=v8, depth=depth, kernel=kernel, tail=None)
    c.write_prompt(k, v, cu, list(lens))
    q, kn, vn = (torch.randn(B, h, D, device="cuda", generator=g).bfloat16() for h in (H, HKV, HKV))
    return c, q, kn, vn


@pytest.mark.parametrize("v8,depth,kernel", [(True, 16.0, "mma"), (False, None, "mma"), (True, 16.0, "sm100")])
def test_a_replayed_step_is_the_real_step_and_leaves_the_lengths_alone(v8, depth, kernel):
    c, q, kn, vn = _cache(v8, depth, kernel)
    lens0 = list(c.lens)
    step = c.prepare_replay_step(q, kn, vn)
    a = [x.clone() for x in step()]
    b = [x.clone() for x in step()]
    assert all(torch.equal(x, y) for x, y in zip(a, b))          # the same bits every replay
    assert c.lens == lens0 and c.seq_lens.tolist() == lens0        # nothing advanced
    vsum0 = c.vsum.clone()
    # from a CUDA graph
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            outs = step()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert all(torch.equal(x, y) for x, y in zip(outs, a))
    assert torch.equal(c.vsum, vsum0)
    # the real step writes the same token to the same slot and sees the same keys
    want = c.decode(q, kn, vn)
    assert torch.equal(a[0].to(want.dtype), want)
    assert c.lens == [n + 1 for n in lens0]
    assert int(step.status) == 0


def test_a_replayed_attention_and_a_replayed_decode_launch():
    c, q, kn, vn = _cache()
    want = c.attend(q)
    att = c.prepare_replay_step(q)                 # no token: attention over the cache as it stands
    assert torch.equal(att()[0].to(want.dtype), want)
    dec = c.prepare_replay_decode(out_dtype=torch.bfloat16)
    o, den, counts = dec()
    assert torch.equal(o.view(want.shape), want) and torch.equal(counts, c.counts)
    other = c.prepare_replay_decode(split=3)
    o3, _, counts3 = other()
    assert torch.equal(counts3, c.counts)          # the verdicts do not depend on the split
    assert ((o3.view(want.shape).float() - want.float()).norm() / want.float().norm()).item() < 1e-2
    with pytest.raises(ValueError, match="both given or both left out"):
        c.prepare_replay_step(q, kn, None)


def test_tune_split_times_every_candidate_and_keeps_the_fastest():
    c, q, kn, vn = _cache(lens=(6000, 5000, 7000, 4096), page_size=128, kernel="mma")
    want = c.attend(q)
    z0 = c.z.clone()
    med = c.tune_split(candidates=(2, 4, 8), rounds=3, reps=3)
    assert {2, 4, 8} <= set(med) and all(t > 0 for t in med.values())
    assert c.split == min(med, key=lambda s: med[s])
    assert torch.equal(c.z, z0)                    # the layer's state is untouched
    got = c.attend(q)                              # and the step still is the function, at the tuned split
    assert ((got.float() - want.float()).norm() / want.float().norm()).item() < 1e-2
    fixed = _cache(lens=(6000, 5000), kernel="mma")[0]
    fixed.chunk = 2048
    with pytest.raises(ValueError, match="nothing to tune"):
        fixed.tune_split()
