"""The library's own forward (O and the log-sum-exp the backward consumes), both
kernels: against FP32 softmax attention, packed against dense to the bit, twice to
the bit. It stands in for the third-party forward the reference calls
(src/fold_attention/interface.py:42-44, 70-81), whose output the reference's tests
only pin as "the same bits as that library" (tests/test_backward.py:340, 358)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_O = 3.0e-3      # rel-L2 of a bf16 output against FP32 attention (the backward tests' level)
TOL_LSE = 1.0e-5    # absolute, nats, on logits of order one


def _fwd():
    from fold_attention_b200.backward import attention_forward

    return attention_forward


def _ref(q, k, v, causal):
    B, S, H, D = q.shape
    G = H // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, 1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3), torch.logsumexp(s, -1)


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()


def _qkv(B, S, H, HKV, D, seed, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return tuple(torch.randn(B, S, h, D, device="cuda", generator=g).to(dtype) for h in (H, HKV, HKV))


@pytest.mark.parametrize("kernel", ["mma", "sm100"])
@pytest.mark.parametrize("B,S,H,HKV,causal", [
    (1, 128, 1, 1, False), (1, 128, 1, 1, True), (2, 384, 4, 2, True), (2, 300, 4, 4, True),
    (1, 1000, 8, 2, False), (2, 2048, 8, 8, True), (3, 1, 2, 1, True), (1, 129, 8, 1, True),
])
def test_forward_is_softmax_attention(kernel, B, S, H, HKV, causal):
    fwd = _fwd()
    q, k, v = _qkv(B, S, H, HKV, 128, S + H)
    o, lse = fwd(q, k, v, causal=causal, kernel=kernel)
    o2, lse2 = fwd(q, k, v, causal=causal, kernel=kernel)
    torch.cuda.synchronize()
    if kernel == "sm100":
        assert int(fwd.last_status) == 0
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    want_o, want_lse = _ref(q, k, v, causal)
    assert o.dtype == q.dtype and lse.dtype == torch.float32 and lse.shape == (B, H, S)
    assert _rel(o, want_o) < TOL_O
    assert (lse - want_lse).abs().max().item() < TOL_LSE * max(1.0, want_lse.abs().max().item())


@pytest.mark.parametrize("kernel", ["mma", "sm100"])
def test_packed_sequences_are_the_dense_bits(kernel):
    """A sequence's O and LSE do not depend on what it is packed with: the tiles are cut from
    the sequence's own start, and what a tile reads past its end meets a zero weight."""
    fwd = _fwd()
    lens = [300, 128, 1000, 77, 1]
    H, HKV, D = 8, 2, 128
    g = torch.Generator(device="cuda").manual_seed(1)
    T = sum(lens)
    q = torch.randn(T, H, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(T, HKV, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(T, HKV, D, device="cuda", generator=g).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    o, lse = fwd(q, k, v, causal=True, cu_seqlens=cu, max_seqlen=max(lens), kernel=kernel)
    assert lse.shape == (H, T)
    for b, n in enumerate(lens):
        a, e = int(cu[b]), int(cu[b + 1])
        o1, lse1 = fwd(q[None, a:e], k[None, a:e], v[None, a:e], causal=True, kernel=kernel)
        assert torch.equal(o1[0], o[a:e]), b
        assert torch.equal(lse1[0], lse[:, a:e]), b


def test_the_two_forwards_agree_and_auto_picks_by_shape():
    fwd = _fwd()
    q, k, v = _qkv(2, 700, 8, 4, 128, 3)
    o_a, lse_a = fwd(q, k, v, causal=True)                    # auto: head_dim 128, bf16 -> tcgen05
    o_s, lse_s = fwd(q, k, v, causal=True, kernel="sm100")
    o_m, lse_m = fwd(q, k, v, causal=True, kernel="mma")
    assert torch.equal(o_a, o_s) and torch.equal(lse_a, lse_s)
    assert _rel(o_s, o_m.float()) < 2e-3 and (lse_s - lse_m).abs().max().item() < 1e-5
    q16, k16, v16 = _qkv(1, 200, 4, 4, 128, 4, torch.float16)
    o16, lse16 = fwd(q16, k16, v16, causal=True)              # fp16, head_dim 128: tcgen05 as well
    o16s, lse16s = fwd(q16, k16, v16, causal=True, kernel="sm100")
    assert o16.dtype == torch.float16 and torch.equal(o16, o16s) and torch.equal(lse16, lse16s)
    q64, k64, v64 = _qkv(1, 200, 4, 4, 64, 5)
    o64, _ = fwd(q64, k64, v64, causal=True)                  # head_dim 64: the warp-level kernel
    assert o64.shape == q64.shape
    with pytest.raises(NotImplementedError, match="head_dim 128"):
        fwd(q64, k64, v64, causal=True, kernel="sm100")
    with pytest.raises(ValueError, match="kernel is one of"):
        fwd(q, k, v, causal=True, kernel="wgmma")


@pytest.mark.parametrize("kernel", ["mma", "sm100"])
@pytest.mark.parametrize("B,S,H,HKV,causal", [(2, 384, 4, 2, True), (1, 1000, 8, 2, False), (1, 129, 8, 1, True)])
def test_fp16_forward_is_softmax_attention(kernel, B, S, H, HKV, causal):
    fwd = _fwd()
    q, k, v = _qkv(B, S, H, HKV, 128, 7 * S + H, torch.float16)
    o, lse = fwd(q, k, v, causal=causal, kernel=kernel)
    torch.cuda.synchronize()
    if kernel == "sm100":
        assert int(fwd.last_status) == 0
    want_o, want_lse = _ref(q, k, v, causal)
    assert o.dtype == torch.float16
    assert _rel(o, want_o) < TOL_O
    assert (lse - want_lse).abs().max().item() < TOL_LSE * max(1.0, want_lse.abs().max().item())


@pytest.mark.parametrize("seed", list(range(6)))
def test_seeded_random_packings_match_fp32_attention(seed):
    import random

    fwd = _fwd()
    rng = random.Random(50 + seed)
    HKV = rng.choice([1, 2, 4])
    H = HKV * rng.choice([1, 2, 4])
    lens = [rng.choice([1, 5, 127, 128, 129, 255, 256, 257, 700, 1300]) for _ in range(rng.choice([1, 2, 4, 6]))]
    causal = rng.random() < 0.7
    T = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(T, H, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(T, HKV, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(T, HKV, 128, device="cuda", generator=g).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    o, lse = fwd(q, k, v, causal=causal, cu_seqlens=cu, max_seqlen=max(lens), kernel="sm100")
    torch.cuda.synchronize()
    assert int(fwd.last_status) == 0
    for b, n in enumerate(lens):
        a, e = int(cu[b]), int(cu[b + 1])
        want_o, want_lse = _ref(q[None, a:e], k[None, a:e], v[None, a:e], causal)
        assert _rel(o[a:e], want_o[0]) < TOL_O, (b, n)
        assert (lse[:, a:e] - want_lse[0]).abs().max().item() < TOL_LSE * max(1.0, want_lse.abs().max().item())
