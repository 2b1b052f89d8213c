"""The backward: is it attention's gradient, and do its bits depend on
anything but the request. Mirrors the reference's tests/test_backward.py with
an FP64 reference as checker; tolerance: rel-L2 <= 3.0e-3 against FP64, the
level the reference publishes for bf16 (worst 2.525e-3 vs FP32)."""

import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import backward as ob  # noqa: E402

TOL = 3.0e-3
KERNELS = ["mma", "sm100"]


def _need(kernel, D, dtype=torch.bfloat16):
    """The tcgen05 kernel serves head_dim 128 (bf16 and fp16); everything runs on mma.sync."""
    if kernel == "sm100" and D != 128:
        pytest.skip("the tcgen05 kernel takes head_dim 128")


def _api():
    import fold_attention_b200 as fa
    from fold_attention_b200.backward import attention_forward, prepare_backward

    return fa, attention_forward, prepare_backward


def _packed(lens, H, HKV, D, seed=0, dtype=torch.bfloat16):
    torch.manual_seed(seed)
    dev = "cuda"
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=dev, dtype=torch.int32)
    T = sum(lens)
    q = torch.randn(T, H, D, device=dev).to(dtype)
    k = torch.randn(T, HKV, D, device=dev).to(dtype)
    v = torch.randn(T, HKV, D, device=dev).to(dtype)
    do = torch.randn(T, H, D, device=dev).to(dtype)
    return q, k, v, do, cu


def _bwd(q, k, v, o, do, lse, cu, S, causal=True, **kw):
    _, _, prepare_backward = _api()
    run = prepare_backward(q, k, v, o, do, lse, causal=causal, cu_seqlens=cu, max_seqlen=S, **kw)
    return tuple(x.clone() for x in run())


def _fwd(q, k, v, cu, S, causal=True):
    _, attention_forward, _ = _api()
    return attention_forward(q, k, v, causal=causal, cu_seqlens=cu, max_seqlen=S)


def _same(a, b):
    return all(torch.equal(x, y) for x, y in zip(a, b))


@pytest.mark.parametrize("H,HKV,D,dtype", [
    (8, 8, 128, torch.bfloat16), (8, 2, 128, torch.bfloat16), (16, 2, 64, torch.bfloat16),
    (8, 8, 96, torch.bfloat16), (8, 2, 128, torch.float16),
])
@pytest.mark.parametrize("kernel", KERNELS)
def test_forward_and_gradient_accuracy(H, HKV, D, dtype, kernel):
    _need(kernel, D, dtype)
    q, k, v, do, cu = _packed([1536], H, HKV, D, dtype=dtype)
    S = 1536
    o, lse = _fwd(q, k, v, cu, S)
    oref, lref = ob.reference_forward(q, k, v)
    assert ob.rel_l2(o, oref) < 4e-3
    assert (lse.double() - lref).abs().max().item() < 2e-3
    ours = _bwd(q, k, v, o, do, lse, cu, S, kernel=kernel)
    ref = ob.reference_grads(q, k, v, do)
    for name, a, r in zip("qkv", ours, ref):
        assert ob.rel_l2(a, r) <= TOL, (name, ob.rel_l2(a, r))


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("kernel", KERNELS)
def test_fp16_packed_sequences_repeat_their_bits(kernel, causal):
    """fp16 keeps the grid's exponent out of P and dS (fp16 has no room for it) and applies it to
    dQ's fp32 sums; the gradients still match FP64 autograd and two runs are the same bits."""
    lens = [300, 129, 1, 640, 77]
    H, HKV, D = 8, 2, 128
    q, k, v, do, cu = _packed(lens, H, HKV, D, seed=11, dtype=torch.float16)
    S = max(lens)
    o, lse = _fwd(q, k, v, cu, S, causal=causal)
    a = _bwd(q, k, v, o, do, lse, cu, S, causal=causal, kernel=kernel)
    b = _bwd(q, k, v, o, do, lse, cu, S, causal=causal, kernel=kernel)
    assert _same(a, b)
    assert all(x.dtype == torch.float16 for x in a)
    for i in range(len(lens)):
        s0, s1 = int(cu[i]), int(cu[i + 1])
        ref = ob.reference_grads(q[s0:s1], k[s0:s1], v[s0:s1], do[s0:s1], causal=causal)
        for name, x, r in zip("qkv", a, ref):
            if r.double().norm().item() > 0:
                assert ob.rel_l2(x[s0:s1], r) <= TOL, (i, name, ob.rel_l2(x[s0:s1], r))


@pytest.mark.parametrize("kernel", KERNELS)
def test_config1_dense_mha_d64_twice(kernel):
    if kernel != "mma":
        pytest.skip("config 1 is head_dim 64: the public API picks the mma.sync kernel")
    """Config 1 of the benchmark: B2 S512 H8/8 D64 causal, N(0,1) inputs; checked
    against FP64 autograd, and two runs are the same bits."""
    fa, _, _ = _api()
    torch.manual_seed(0)
    B, S, H, D = 2, 512, 8, 64
    q, k, v, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(4))
    grads = []
    for _ in range(2):
        qq, kk, vv = (x.clone().requires_grad_() for x in (q, k, v))
        out = fa.fold_attn_func(qq, kk, vv, causal=True)
        out.backward(do)
        grads.append((qq.grad.clone(), kk.grad.clone(), vv.grad.clone()))
    assert _same(grads[0], grads[1])
    for b in range(B):
        ref = ob.reference_grads(q[b], k[b], v[b], do[b])
        for name, a, r in zip("qkv", grads[0], ref):
            assert ob.rel_l2(a[b], r) <= TOL, (name, ob.rel_l2(a[b], r))


@pytest.mark.parametrize("B,H,HKV,S,D,causal", [
    (2, 8, 2, 1024, 128, False), (1, 16, 2, 1000, 64, False), (1, 8, 8, 1000, 96, False),
    (3, 8, 2, 777, 128, True),
])
@pytest.mark.parametrize("kernel", KERNELS)
def test_full_and_ragged_attention(B, H, HKV, S, D, causal, kernel):
    _need(kernel, D)
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(7)
    q, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    o, lse = attention_forward(q, k, v, causal=causal)
    tr = lambda x: x.transpose(1, 2)
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=causal, kernel=kernel)
    ours = tuple(tr(x).clone() for x in run())
    for b in range(B):
        ref = ob.reference_grads(q[b], k[b], v[b], do[b], causal=causal)
        for name, a, r in zip("qkv", ours, ref):
            assert ob.rel_l2(a[b], r) <= TOL, (name, ob.rel_l2(a[b], r))
    assert _same(ours, tuple(tr(x) for x in run()))


@pytest.mark.parametrize("H,HKV,D", [(8, 8, 128), (8, 2, 128), (16, 2, 64), (32, 4, 128)])
@pytest.mark.parametrize("kernel", KERNELS)
def test_a_request_does_not_see_its_batch(H, HKV, D, kernel):
    """A request's gradients alone and packed among others are the same bits."""
    _need(kernel, D)
    lens = [1000, 777, 2048, 64, 1500]
    q, k, v, do, cu = _packed(lens, H, HKV, D)
    S = max(lens)
    o, lse = _fwd(q, k, v, cu, S)
    packed = _bwd(q, k, v, o, do, lse, cu, S, kernel=kernel)
    a, b = int(cu[2]), int(cu[3])
    sl = lambda x: x[a:b].contiguous()
    cu1 = torch.tensor([0, b - a], device="cuda", dtype=torch.int32)
    o1, lse1 = _fwd(sl(q), sl(k), sl(v), cu1, b - a)
    assert torch.equal(o1, sl(o))
    alone = _bwd(sl(q), sl(k), sl(v), o1, sl(do), lse1, cu1, b - a, kernel=kernel)
    assert all(torch.equal(x, sl(y)) for x, y in zip(alone, packed))
    # and in another order, inside another batch
    order = [2, 0, 4]
    parts = [slice(int(cu[i]), int(cu[i + 1])) for i in order]
    cat = lambda x: torch.cat([x[p] for p in parts]).contiguous()
    cu2 = torch.tensor([0] + list(np.cumsum([lens[i] for i in order])), device="cuda", dtype=torch.int32)
    o2, lse2 = _fwd(cat(q), cat(k), cat(v), cu2, S)
    other = _bwd(cat(q), cat(k), cat(v), o2, cat(do), lse2, cu2, S, kernel=kernel)
    assert all(torch.equal(x[: lens[2]], sl(y)) for x, y in zip(other, packed))


@pytest.mark.parametrize("kernel", KERNELS)
def test_repeated_calls_and_short_sequences(kernel):
    _, _, prepare_backward = _api()
    lens = [17, 0, 129, 65, 257, 1, 191]
    q, k, v, do, cu = _packed(lens, 8, 2, 128, seed=5)
    o, lse = _fwd(q, k, v, cu, max(lens))
    run = prepare_backward(q, k, v, o, do, lse, causal=True, cu_seqlens=cu, max_seqlen=max(lens), kernel=kernel)
    first = tuple(x.clone() for x in run())
    for _ in range(3):
        assert _same(first, run())
    off = 0
    for n in lens:
        if n:
            ref = ob.reference_grads(q[off:off + n], k[off:off + n], v[off:off + n], do[off:off + n])
            for name, a, r in zip("qkv", first, ref):
                # a one-token request's dQ and dK are exactly zero
                err = (a[off:off + n].double() - r).norm().item()
                assert err <= 2 * TOL * r.norm().item() + 1e-5 * math.sqrt(r.numel()), (n, name)
        off += n


@pytest.mark.parametrize("kernel", KERNELS)
def test_varlen_is_dense_to_the_bit(kernel):
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(3)
    B, S, H, HKV, D = 3, 640, 8, 2, 128
    q, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)
    dense = tuple(tr(x).clone() for x in prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True, kernel=kernel)())
    cu = torch.arange(B + 1, device="cuda", dtype=torch.int32) * S
    fl = lambda x: x.reshape(B * S, x.shape[2], D)
    lse_p = lse.permute(1, 0, 2).reshape(H, B * S).contiguous()
    packed = _bwd(fl(q), fl(k), fl(v), fl(o), fl(do), lse_p, cu, S, kernel=kernel)
    assert all(torch.equal(fl(a), b) for a, b in zip(dense, packed))


@pytest.mark.parametrize("kernel", KERNELS)
def test_grid_exponent_accumulator_and_postprocess(kernel):
    """The preprocess's maxima and the exponent derived from them are the
    oracle's; the int32 accumulator never nears saturation; dQ is the one
    fp32 multiply of the accumulator the postprocess documents."""
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(11)
    B, S, H, HKV, D = 2, 300, 4, 2, (64 if kernel == "mma" else 128)
    G = H // HKV
    q, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    k[1] *= 6.0
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True, kernel=kernel)
    dq, dk, dv = run()
    torch.cuda.synchronize()
    off_acc, off_dp, off_l2, off_st, rows_p = run.layout[:5]
    ws = run.workspace
    stats = ws[off_st: off_st + B * HKV * 8 * 4].view(torch.float32).view(B, HKV, 8).cpu()
    acc = ws[off_acc: off_acc + H * rows_p * D * 4].view(torch.int32).view(H, rows_p, D)
    S_r = rows_p // B
    for b in range(B):
        st = ob.stats(q[b], k[b], v[b], o[b], do[b], G)
        for h in range(HKV):
            got = stats[b, h]
            assert float(got[0]) == st[h][0] and float(got[1]) == st[h][1]
            assert abs(float(got[2]) - st[h][2]) <= 1e-5 * st[h][2]
            assert abs(float(got[3]) - st[h][3]) <= 1e-4 * max(st[h][3], 1.0)
            s = ob.dq_scale_exp(*[float(x) for x in got[:4]], D)
            for g in range(G):
                a = acc[h * G + g, b * S_r: b * S_r + S]
                assert int(a.abs().max()) < 2**30
                assert int(a.abs().max()) > 2**14
                f = np.float32(np.float32(1.0 / math.sqrt(D)) * np.float32(2.0**-s))
                want = (a.float() * float(f)).bfloat16()
                assert torch.equal(tr(dq)[b, :, h * G + g], want)
    assert int(run.status) == 0


def test_the_two_kernels_agree_and_auto_picks_tcgen05():
    """The tcgen05 and mma.sync main loops are two schedules of one function:
    same grid exponent, gradients equal to within bf16 rounding; "auto" is the
    tcgen05 kernel's bits at head_dim 128."""
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(21)
    B, S, H, HKV, D = 2, 1100, 8, 2, 128
    q, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)
    got = {}
    for kern in ("mma", "sm100", "auto"):
        run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True, kernel=kern)
        got[kern] = tuple(x.clone() for x in run())
        assert int(run.status) == 0
    assert _same(got["auto"], got["sm100"])
    for a, b in zip(got["mma"], got["sm100"]):
        assert ob.rel_l2(a, b.double()) < 1e-3


def test_error_messages():
    fa, _, _ = _api()
    q = torch.randn(2, 64, 8, 128, device="cuda").bfloat16()
    k = torch.randn(2, 64, 3, 128, device="cuda").bfloat16()
    with pytest.raises(ValueError, match="multiple of the KV heads"):
        fa.fold_attn_func(q, k, k)
    with pytest.raises(ValueError, match="bf16 or fp16"):
        fa.fold_attn_func(q.float(), q.float(), q.float())
    q32 = torch.randn(2, 64, 8, 32, device="cuda").bfloat16()
    with pytest.raises(NotImplementedError, match="64, 96 and 128"):
        fa.fold_attn_func(q32.requires_grad_(), q32, q32).sum().backward()


def test_a_shard_of_kv_heads_is_the_full_runs_bits():
    """Multi-GPU sharding unit: the backward of a slice of (request, KV head)
    units, run alone as a rank would, equals the full run's slice bit for bit."""
    from fold_attention_b200 import parallel

    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(31)
    B, S, H, HKV, D = 2, 700, 8, 4, 128
    G = H // HKV
    q, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)
    whole = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True)
    plan = whole.plan          # every rank runs the full call's plan on its slice
    full = tuple(tr(x).clone() for x in whole())
    world = 3
    for rank in range(world):
        for b, (lo, hi) in parallel.backward_units(B, HKV, world, rank).items():
            qs, os_, dos = (x[b:b + 1, :, lo * G:hi * G].contiguous() for x in (q, o, do))
            ks, vs = (x[b:b + 1, :, lo:hi].contiguous() for x in (k, v))
            ls = lse[b:b + 1, lo * G:hi * G].contiguous()
            part = prepare_backward(tr(qs), tr(ks), tr(vs), tr(os_), tr(dos), ls, causal=True, plan=plan)()
            dq, dk, dv = (tr(x) for x in part)
            assert torch.equal(dq, full[0][b:b + 1, :, lo * G:hi * G])
            assert torch.equal(dk, full[1][b:b + 1, :, lo:hi])
            assert torch.equal(dv, full[2][b:b + 1, :, lo:hi])


def test_config2_full_size_repeats_and_matches_a_slice():
    """Config 2 of the benchmark (GQA variant) at full size: B4 S8192 H32/8 D128. Two runs
    are the same bits; one (request, KV head) unit run alone is the full run's
    slice (size-independent property); that unit's gradients match FP32 autograd."""
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(2)
    B, S, H, HKV, D = 4, 8192, 32, 8, 128
    G = H // HKV
    q = (torch.randn(B, S, H, D, device="cuda") / D**0.5).bfloat16()
    do = torch.randn(B, S, H, D, device="cuda").bfloat16()
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True)
    first = tuple(x.clone() for x in run())
    assert _same(first, run())
    assert int(run.status) == 0
    b, hk = 2, 5
    qs, os_, dos = (x[b:b + 1, :, hk * G:(hk + 1) * G].contiguous() for x in (q, o, do))
    ks, vs = (x[b:b + 1, :, hk:hk + 1].contiguous() for x in (k, v))
    ls = lse[b:b + 1, hk * G:(hk + 1) * G].contiguous()
    # the unit alone would plan for one small call: hold the full run's plan, as any comparison across batch sizes must
    dq, dk, dv = prepare_backward(tr(qs), tr(ks), tr(vs), tr(os_), tr(dos), ls, causal=True, plan=run.plan)()
    assert torch.equal(dq, first[0][b:b + 1, hk * G:(hk + 1) * G])
    assert torch.equal(dk, first[1][b:b + 1, hk:hk + 1])
    assert torch.equal(dv, first[2][b:b + 1, hk:hk + 1])
    ref = ob.reference_grads(qs[0, :, :1], ks[0], vs[0], dos[0, :, :1], scale=1.0 / math.sqrt(D), dtype=torch.float32)
    assert ob.rel_l2(tr(dq)[0, :, :1], ref[0]) <= TOL


def test_config2_mha_full_size_repeats_and_matches_a_slice():
    """Config 2's headline variant at full size: B4 S8192 H32/32 D128 (MHA). Two runs are the
    same bits; one (request, head) unit run alone is the full run's slice; that unit's dQ, dK
    and dV match FP32 autograd. (The whole tensor against an FP32 reference would take the CPU
    minutes; the slice property carries the check to every unit.)"""
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(22)
    B, S, H, D = 4, 8192, 32, 128
    q = (torch.randn(B, S, H, D, device="cuda") / D**0.5).bfloat16()
    do = torch.randn(B, S, H, D, device="cuda").bfloat16()
    k, v = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)  # noqa: E731
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True)
    first = tuple(x.clone() for x in run())
    assert _same(first, run())
    assert int(run.status) == 0
    for b, h in ((3, 17), (0, 0)):
        qs, ks, vs, os_, dos = (x[b:b + 1, :, h:h + 1].contiguous() for x in (q, k, v, o, do))
        ls = lse[b:b + 1, h:h + 1].contiguous()
        part = prepare_backward(tr(qs), tr(ks), tr(vs), tr(os_), tr(dos), ls, causal=True, plan=run.plan)()
        for x, y in zip(part, first):
            assert torch.equal(x, y[b:b + 1, h:h + 1])
    ref = ob.reference_grads(qs[0], ks[0], vs[0], dos[0], scale=1.0 / math.sqrt(D), dtype=torch.float32)
    for name, x, r in zip("qkv", part, ref):
        assert ob.rel_l2(tr(x)[0], r) <= TOL, name


def test_varlen_autograd_matches_the_prepared_call_and_the_dense_call():
    """`fold_attn_varlen_func` under autograd (src/fold_attention/interface.py:121-151): its output
    is the library's forward, its gradients are the prepared call's bits on the same packing
    (the reference's tests/test_backward.py:334-343), and a packing of equal lengths is the dense
    `fold_attn_func` bit for bit (:318-332)."""
    fa, attention_forward, prepare_backward = _api()
    lens = [1024, 300, 512, 1]
    H, HKV, D = 8, 2, 128
    q, k, v, do, cu = _packed(lens, H, HKV, D, seed=5)
    qa, ka, va = (x.clone().requires_grad_() for x in (q, k, v))
    out = fa.fold_attn_varlen_func(qa, ka, va, cu, causal=True)
    out.backward(do)
    o, lse = _fwd(q, k, v, cu, max(lens))
    assert torch.equal(out.detach(), o)
    want = _bwd(q, k, v, o, do, lse, cu, max(lens))
    assert all(torch.equal(x.grad, y) for x, y in zip((qa, ka, va), want))
    # given maxima and key-side arguments change nothing; mismatched ones are refused
    qb, kb, vb = (x.clone().requires_grad_() for x in (q, k, v))
    fa.fold_attn_varlen_func(qb, kb, vb, cu, cu.clone(), max(lens), max(lens), None, True).backward(do)
    assert all(torch.equal(x.grad, y.grad) for x, y in zip((qa, ka, va), (qb, kb, vb)))
    with pytest.raises(ValueError, match="max_seqlen_k"):
        fa.fold_attn_varlen_func(q, k, v, cu, max_seqlen_q=1024, max_seqlen_k=512)
    # equal lengths: the packed call is the dense call
    B, L = 3, 640
    q, k, v, do, cu = _packed([L] * B, H, HKV, D, seed=6)
    qa, ka, va = (x.clone().requires_grad_() for x in (q, k, v))
    fa.fold_attn_varlen_func(qa, ka, va, cu, causal=True).backward(do)
    dn = lambda x: x.view(B, L, *x.shape[1:])  # noqa: E731
    qd, kd, vd = (dn(x).clone().requires_grad_() for x in (q, k, v))
    outd = fa.fold_attn_func(qd, kd, vd, causal=True)
    outd.backward(dn(do))
    for x, y in zip((qa, ka, va), (qd, kd, vd)):
        assert torch.equal(dn(x.grad), y.grad)


@pytest.mark.parametrize("causal", [False, True])
def test_dense_autograd_matches_the_forward_and_the_prepared_backward(causal):
    """The dense public call (tests/test_backward.py:346-362 of the reference, with the library's
    own forward where the reference has a third-party one)."""
    fa, attention_forward, prepare_backward = _api()
    B, S, H, HKV, D = 2, 256, 8, 2, 64
    torch.manual_seed(7)
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, HKV, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    do = torch.randn_like(q)
    qa, ka, va = (x.clone().requires_grad_() for x in (q, k, v))
    got = fa.fold_attn_func(qa, ka, va, causal=causal)
    got.backward(do)
    ref, lse = attention_forward(q, k, v, causal=causal)
    assert torch.equal(got.detach(), ref)
    qh, kh, vh, oh, doh = (x.transpose(1, 2) for x in (q, k, v, ref, do))
    want = prepare_backward(qh, kh, vh, oh, doh, lse, causal=causal)()
    for x, y in zip((qa, ka, va), want):
        assert x.grad is not None and torch.equal(x.grad, y.transpose(1, 2))


def test_config3_packed_64k_tokens_invariance():
    """Config 3 of the benchmark: 64K tokens, lengths uniform in [256, 8192], GQA 32/8,
    D128. A sequence's gradients are the same bits packed, alone, and in a
    reversed packing."""
    lens, total = [], 65536
    g = torch.Generator().manual_seed(3)
    while sum(lens) < total:
        lens.append(min(int(torch.randint(256, 8193, (1,), generator=g)), total - sum(lens)))
    H, HKV, D = 32, 8, 128
    q, k, v, do, cu = _packed(lens, H, HKV, D, seed=9)
    S = max(lens)
    o, lse = _fwd(q, k, v, cu, S)
    packed = _bwd(q, k, v, o, do, lse, cu, S)
    assert _same(packed, _bwd(q, k, v, o, do, lse, cu, S))
    i = 3
    a, e = int(cu[i]), int(cu[i + 1])
    sl = lambda x: x[a:e].contiguous()
    cu1 = torch.tensor([0, e - a], device="cuda", dtype=torch.int32)
    o1, lse1 = _fwd(sl(q), sl(k), sl(v), cu1, e - a)
    alone = _bwd(sl(q), sl(k), sl(v), o1, sl(do), lse1, cu1, e - a)
    assert all(torch.equal(x, sl(y)) for x, y in zip(alone, packed))
    order = list(range(len(lens)))[::-1]
    parts = [slice(int(cu[j]), int(cu[j + 1])) for j in order]
    cat = lambda x: torch.cat([x[p] for p in parts]).contiguous()
    cu2 = torch.tensor([0] + list(np.cumsum([lens[j] for j in order])), device="cuda", dtype=torch.int32)
    o2, lse2 = _fwd(cat(q), cat(k), cat(v), cu2, S)
    rev = _bwd(cat(q), cat(k), cat(v), o2, cat(do), lse2, cu2, S)
    pos = sum(lens[j] for j in order[: order.index(i)])
    assert all(torch.equal(x[pos:pos + lens[i]], sl(y)) for x, y in zip(rev, packed))


@pytest.mark.parametrize("kernel", KERNELS)
def test_a_prepared_backward_replays_from_a_cuda_graph(kernel):
    """The three phases are stream-ordered launches over buffers the launch owns (the
    accumulator is zeroed in-stream): captured once, the backward replays on new inputs."""
    _need(kernel, 128, torch.bfloat16)
    _, attention_forward, prepare_backward = _api()
    torch.manual_seed(41)
    B, S, H, HKV, D = 2, 700, 8, 2, 128
    mk = lambda h: torch.randn(B, S, h, D, device="cuda").bfloat16()  # noqa: E731
    q, k, v, do = mk(H), mk(HKV), mk(HKV), mk(H)
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)  # noqa: E731
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True, kernel=kernel)
    want = tuple(x.clone() for x in run())
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            outs = run()
    torch.cuda.synchronize()
    for x in outs:
        x.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert _same(outs, want)
    # new upstream gradient in the bound buffer: the replay follows it
    do2 = mk(H)
    do.copy_(do2)
    g.replay()
    torch.cuda.synchronize()
    got = tuple(x.clone() for x in outs)
    assert _same(got, tuple(x.clone() for x in run()))
    assert not _same(got, want)
    assert int(run.status) == 0


@pytest.mark.parametrize("seed", list(range(8)))
def test_seeded_random_packings_repeat_and_agree_across_kernels(seed):
    """Random packed shapes (ragged lengths around the 128-row tile, MHA/GQA/MQA, both types,
    causal or full): the tcgen05 kernel gives the same bits three times running, raises no
    status, and agrees with the mma.sync kernel within the accuracy tolerance."""
    import random

    _, attention_forward, prepare_backward = _api()
    rng = random.Random(100 + seed)
    HKV = rng.choice([1, 2, 4])
    H = HKV * rng.choice([1, 2, 4])
    lens = [rng.choice([1, 64, 127, 128, 129, 300, 511, 512, 777, 1024, 1500, 2048])
            for _ in range(rng.choice([1, 2, 3, 5]))]
    causal = rng.random() < 0.7
    dtype = torch.bfloat16 if rng.random() < 0.7 else torch.float16
    q, k, v, do, cu = _packed(lens, H, HKV, 128, seed=seed, dtype=dtype)
    S = max(lens)
    o, lse = attention_forward(q, k, v, causal=causal, cu_seqlens=cu, max_seqlen=S)
    outs = []
    for kern in ("sm100", "sm100", "sm100", "mma"):
        run = prepare_backward(q, k, v, o, do, lse, causal=causal, cu_seqlens=cu, max_seqlen=S, kernel=kern)
        outs.append(tuple(x.clone() for x in run()))
        torch.cuda.synchronize()
        assert int(run.status.item()) == 0, kern
    assert _same(outs[0], outs[1]) and _same(outs[0], outs[2])
    for name, a, b in zip("qkv", outs[0], outs[3]):
        if b.double().norm().item() > 0:
            assert ob.rel_l2(a, b.double()) <= 4e-3, (name, lens, H, HKV, causal, dtype)
