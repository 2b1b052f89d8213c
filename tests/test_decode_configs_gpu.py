"""Configs 4 and 5 of the benchmark at their own sizes, as tests.

Config 5: v8, depth 16, 256 requests, GQA 64/8, D128, lengths log-uniform in [4096, 131072],
1 % of key positions x 8, 0.1 % of V entries x 20. Config 4: dense bf16 V, 128 requests, GQA 32/8,
lengths uniform in [1024, 32768], 64 serving steps. Both with the page table shuffled. At full size
the oracle cannot run every key, so the checks are the size-independent ones: the two decode
kernels count the same live and refined keys (the verdicts are exact integer arithmetic under one
reference), they agree with each other, and eight sampled requests per config sit inside the
depth's error bound against dense FP32 attention over everything written."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def _requests(lens, HKV, D, seed):
    T = sum(lens)
    k = torch.empty(T, HKV, D, device="cuda", dtype=torch.bfloat16)
    v = torch.empty(T, HKV, D, device="cuda", dtype=torch.bfloat16)
    at = 0
    for i, n in enumerate(lens):      # request by request: a whole batch's fp32 draws would not fit
        g = torch.Generator(device="cuda").manual_seed(seed * 1000 + i)
        kk = torch.randn(n, HKV, D, device="cuda", generator=g)
        hot = torch.rand(n, 1, 1, device="cuda", generator=g) < 0.01
        k[at:at + n] = torch.where(hot, kk * 8, kk)
        vv = torch.randn(n, HKV, D, device="cuda", generator=g)
        big = torch.rand(n, HKV, D, device="cuda", generator=g) < 0.001
        v[at:at + n] = torch.where(big, vv * 20, vv)
        at += n
    return k, v


def _dense_fp32(q, ks, vs, HKV, G, D):
    qs = q.float().view(HKV, G, D)
    w = torch.softmax(torch.einsum("hgd,shd->hgs", qs, ks.float()) / D**0.5, -1)
    return torch.einsum("hgs,shd->hgd", w, vs.float()).reshape(HKV * G, D)


def _sampled(lens, n=8):
    order = sorted(range(len(lens)), key=lambda b: lens[b])
    B = len(lens)
    return sorted({order[0], order[1], order[B // 8], order[B // 4], order[B // 2], order[3 * B // 4], order[-2], order[-1]})[:n]


def test_config5_at_its_own_batch():
    from fold_attention_b200 import FoldKVCache

    B, H, HKV, D = 256, 64, 8, 128
    G = H // HKV
    g = torch.Generator().manual_seed(5)
    lens = [int(math.exp(x)) for x in (torch.rand(B, generator=g) * (math.log(131072) - math.log(4096)) + math.log(4096))]
    k, v = _requests(lens, HKV, D, seed=7)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    gd = torch.Generator(device="cuda").manual_seed(8)
    q, kn, vn = (torch.randn(B, h, D, device="cuda", generator=gd).bfloat16() for h in (H, HKV, HKV))
    outs = {}
    for kernel in ("sm100", "mma"):
        c = FoldKVCache(B, H, HKV, D, max(lens) + 4, depth=16.0, v8=True, v_scale=2.0 ** -3, device="cuda", kernel=kernel,
                        chunk=8192 if kernel == "mma" else None)
        c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).int().view_as(c.page_table))
        c.write_prompt(k, v, cu, lens)
        out = c.decode(q, kn, vn)
        launch = next(iter(c._launches.values()))
        assert launch.kernel == kernel
        launch.check()
        if kernel == "sm100":
            assert torch.equal(c.attend(q), out)          # the cache as it stands, the same query: the same bits
        outs[kernel] = (out, c.counts.clone())
        del c, launch
        torch.cuda.empty_cache()
    assert torch.equal(outs["sm100"][1], outs["mma"][1])
    live = outs["sm100"][1][:, 0].sum().item() / (sum(lens) + B) / HKV
    assert 0.5 < live < 1.0
    assert _rel(outs["sm100"][0].float(), outs["mma"][0].float()) < 2e-3
    for b in _sampled(lens):
        a, e = int(cu[b]), int(cu[b + 1])
        want = _dense_fp32(q[b], torch.cat([k[a:e], kn[b][None]]), torch.cat([v[a:e], vn[b][None]]), HKV, G, D)
        assert _rel(outs["sm100"][0][b], want) < 2.0 ** (-16.0 / 3), b
        assert _rel(outs["mma"][0][b], want) < 2.0 ** (-16.0 / 3), b


def test_config4_over_its_64_steps():
    from fold_attention_b200 import FoldKVCache

    B, H, HKV, D, STEPS = 128, 32, 8, 128, 64
    G = H // HKV
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(1024, 32769, (B,), generator=g).tolist()
    k, v = _requests(lens, HKV, D, seed=11)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    gd = torch.Generator(device="cuda").manual_seed(12)
    steps = [tuple(torch.randn(B, h, D, device="cuda", generator=gd).bfloat16() for h in (H, HKV, HKV)) for _ in range(STEPS)]
    res = {}
    for kernel in ("sm100", "mma"):
        c = FoldKVCache(B, H, HKV, D, max(lens) + STEPS + 4, device="cuda", kernel=kernel, chunk=4096 if kernel == "mma" else None)
        c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)).int().view_as(c.page_table))
        c.write_prompt(k, v, cu, lens)
        outs, counts = [], []
        for i, (q, kn, vn) in enumerate(steps):
            out = c.decode(q, kn, vn)
            if i in (0, 31, 63):
                outs.append(out.clone())
                counts.append(c.counts.clone())
        for launch in c._launches.values():
            launch.check()
        assert c.lens == [n + STEPS for n in lens]
        res[kernel] = (outs, counts)
        del c
        torch.cuda.empty_cache()
    for a, b in zip(res["sm100"][1], res["mma"][1]):
        assert torch.equal(a, b)                         # live (every key) and refined counts, step by step
    for a, b in zip(res["sm100"][0], res["mma"][0]):
        assert _rel(a.float(), b.float()) < 2e-3
    q = steps[-1][0]
    for b in _sampled(lens):
        a, e = int(cu[b]), int(cu[b + 1])
        ks = torch.cat([k[a:e]] + [s[1][b][None] for s in steps])
        vs = torch.cat([v[a:e]] + [s[2][b][None] for s in steps])
        want = _dense_fp32(q[b], ks, vs, HKV, G, D)
        assert _rel(res["sm100"][0][-1][b], want) < 4e-3, b
        assert _rel(res["mma"][0][-1][b], want) < 4e-3, b
