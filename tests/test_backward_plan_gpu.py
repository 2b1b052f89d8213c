"""Plans of the tcgen05 backward: how a call's work is cut, the work list, and the integer
dK / dV grids a key block's work items meet on when they run in different CTAs.

Mirrors the reference's tests/test_backward.py:195-301 (the packed plan reads head counts only,
the control that two dK/dV reductions are different bits, the dense plan follows the request
shape, dispatch order moves no bit) for B200's own planner."""

import pytest
import torch

from oracle import backward as ob

pytestmark = pytest.mark.gpu

TOL = 3.0e-3


def _api():
    from fold_attention_b200.backward import attention_forward, prepare_backward
    from fold_attention_b200.backward.plan import Plan

    return attention_forward, prepare_backward, Plan


def _dense(B, H, HKV, S, D=128, seed=0, dtype=torch.bfloat16):
    attention_forward, _, _ = _api()
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(B, S, h, D, device="cuda", generator=g).to(dtype)  # noqa: E731
    q, k, v, do = mk(H), mk(HKV), mk(HKV), mk(H)
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)  # noqa: E731
    return (tr(q), tr(k), tr(v), tr(o), tr(do)), lse


def _same(a, b):
    return all(torch.equal(x, y) for x, y in zip(a, b))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_folded_dk_dv_match_the_private_exit_and_dq_never_moves(dtype):
    """Every cut of the same call: dQ is the same bits (each (key block, query block) partial is
    the same integers whoever computes it), dK and dV agree with the private exit to rounding and
    with FP64 autograd within the gradient tolerance, and each plan repeats its own bits."""
    _, prepare_backward, Plan = _api()
    B, H, HKV, S = 2, 8, 2, 1024
    (q, k, v, o, do), lse = _dense(B, H, HKV, S, seed=1, dtype=dtype)
    base = prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(4, 0))
    want = tuple(x.clone() for x in base())
    assert base.dk_acc is None
    refs = [ob.reference_grads(q[b].transpose(0, 1), k[b].transpose(0, 1), v[b].transpose(0, 1), do[b].transpose(0, 1)) for b in range(B)]
    for plan in (Plan(2, 0), Plan(1, 0), Plan(4, 3), Plan(1, 2), Plan(2, 8)):
        run = prepare_backward(q, k, v, o, do, lse, causal=True, plan=plan)
        got = tuple(x.clone() for x in run())
        assert int(run.status) == 0
        assert run.dk_acc is not None and run.dv_acc.dtype == torch.int32   # G * S = 4096: the 30-bit dV grid
        assert torch.equal(got[0], want[0]), plan
        for name, a, b in zip("kv", got[1:], want[1:]):
            assert ob.rel_l2(a, b) < 1e-3, (plan, name, ob.rel_l2(a, b))
        assert _same(got, run()) and _same(got, run())
        for b in range(B):
            for name, a, r in zip("qkv", got, refs[b]):
                assert ob.rel_l2(a[b].transpose(0, 1), r) <= TOL, (plan, name)


def test_the_two_dkv_exits_do_not_agree():
    """The control: the private exit and the integer fold really are different bits somewhere, so a
    plan that silently followed the batch would show in the invariance tests."""
    _, prepare_backward, Plan = _api()
    (q, k, v, o, do), lse = _dense(2, 32, 8, 1024, seed=4)
    private = tuple(x.clone() for x in prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(4, 0))())
    fold = tuple(x.clone() for x in prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(2, 0))())
    assert torch.equal(private[0], fold[0]), "dQ is order-free and must not move"
    assert not torch.equal(private[1], fold[1]) or not torch.equal(private[2], fold[2])


def test_the_wide_dv_grid_and_the_accumulators_stay_in_range():
    """G * S above 16384 moves dV to the 61-bit grid in int64. The accumulators hold what the
    bound promises (|acc| < 2^61, 2^30) and what the postprocess says it converts:
    dK = round16(float(acc) * (scale * 2^-s_dK)) from the oracle's grid exponents."""
    _, prepare_backward, Plan = _api()
    B, H, HKV, S, D = 1, 16, 1, 2048, 128     # G * S = 32768
    (q, k, v, o, do), lse = _dense(B, H, HKV, S, seed=8)
    run = prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(4, 0))
    dq, dk, dv = (x.clone() for x in run())
    assert run.dv_acc.dtype == torch.int64
    assert int(run.dk_acc.abs().max()) < 2**61 and int(run.dv_acc.abs().max()) < 2**61
    assert int(run.dk_acc.abs().max()) > 2**30     # the grid is used, not wasted
    # the exponents from the maxima, restated on the CPU
    st = ob.stats(q[0].transpose(0, 1).cpu(), k[0].transpose(0, 1).cpu(), v[0].transpose(0, 1).cpu(),
                  o[0].transpose(0, 1).cpu(), do[0].transpose(0, 1).cpu(), H // HKV)[0]
    max_doc = float(do.float().abs().max())
    max_q = float(q.float().abs().max())
    rows = float((H // HKV) * S)
    s_k = ob.dk_scale_exp(st[1], st[2], st[3], max_q, rows, D)
    s_v = ob.dv_scale_exp(max_doc, rows, 61)
    scale = 1.0 / D**0.5
    f_k = torch.tensor(scale, dtype=torch.float32) * torch.tensor(2.0 ** -s_k, dtype=torch.float32)
    want_k = (run.dk_acc[0, :S].float() * f_k).bfloat16()
    want_v = (run.dv_acc[0, :S].float() * torch.tensor(2.0 ** -s_v, dtype=torch.float32, device="cuda")).bfloat16()
    # the row norm ||dO_i|| is summed in another order on the device: its maximum may differ in the last
    # bit, which moves the exponent only at a binade edge; the conversion itself is exact to check
    if torch.equal(dk[0, 0], want_k.to(dk.device)):
        assert torch.equal(dv[0, 0], want_v)
    else:
        assert ob.rel_l2(dk[0, 0], want_k) < 1e-2
    ref = ob.reference_grads(q[0].transpose(0, 1), k[0].transpose(0, 1), v[0].transpose(0, 1), do[0].transpose(0, 1))
    for name, a, r in zip("qkv", (dq, dk, dv), ref):
        assert ob.rel_l2(a[0].transpose(0, 1), r) <= TOL, name


def test_the_work_list_covers_the_call_once_longest_first():
    """The device-built list: every (key block, request, KV head, subgroup, record) with work
    appears once, its cost is the tiles it walks, and inside a section costs never rise."""
    _, prepare_backward, Plan = _api()
    B, H, HKV, S = 2, 8, 2, 1536
    (q, k, v, o, do), lse = _dense(B, H, HKV, S, seed=2)
    for plan in (Plan(4, 0), Plan(2, 5), Plan(1, 0)):
        run = prepare_backward(q, k, v, o, do, lse, causal=True, plan=plan)
        run()
        w = run.work.cpu()
        nb = S // 128
        nsub = 4 // plan.subgroup
        nrec = -(-nb // plan.record) if plan.record else 1
        assert w.shape[0] == B * HKV * nsub * nb * nrec
        seen = set()
        total = 0
        for row in w.tolist():
            kb, hkv, b, h0, nh, m_lo, m_hi, cost = row
            first = max(kb, m_lo)
            blocks = max(min(nb, m_hi) - first, 0)
            assert nh == plan.subgroup and cost == blocks * nh
            key = (kb, hkv, b, h0, m_lo)
            assert key not in seen
            seen.add(key)
            total += cost
        assert total == B * H * nb * (nb + 1) // 2
        # one section holds every item of this small call: costs fall from start to end
        costs = w[:, 7].tolist()
        assert costs == sorted(costs, reverse=True)


@pytest.mark.parametrize("B,H,HKV,S,plan", [(1, 8, 2, 1024, (4, 0)), (3, 8, 8, 1536, (1, 0)), (2, 8, 2, 1024, (2, 3))])
def test_dispatch_order_does_not_move_the_bits(B, H, HKV, S, plan):
    """The persistent CTAs claim work from a counter, so which CTA runs an item, and when, changes
    from call to call. Reversing the list moves every item to another CTA and another point in the
    claim order; the bits stay put (private and folded exits alike)."""
    _, prepare_backward, Plan = _api()
    (q, k, v, o, do), lse = _dense(B, H, HKV, S, seed=2)
    run = prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(*plan))
    dq, dk, dv = run()
    ref = tuple(x.clone() for x in (dq, dk, dv))
    for _ in range(3):
        assert _same(ref, run())
    run.run_phase(1)            # preprocess
    run.run_phase(8)            # the list, as the device orders it
    run.work.copy_(run.work.flip(0).clone())
    run.run_phase(2)            # main loop on the reversed list
    run.run_phase(4)
    torch.cuda.synchronize()
    assert _same(ref, (dq, dk, dv))
    assert int(run.status) == 0


def test_the_packed_plan_reads_only_head_counts():
    """Across a growing packed batch the plan and the bits of one request stay put, on the folding
    plan a group of eight takes as well as on a private one."""
    from fold_attention_b200.backward.plan import plan_varlen

    attention_forward, prepare_backward, Plan = _api()
    assert plan_varlen(8, 2) == Plan(4, 0) and plan_varlen(32, 8) == Plan(4, 0)
    assert plan_varlen(64, 8) == Plan(4, 0) and plan_varlen(32, 1) == Plan(4, 0) and plan_varlen(8, 8) == Plan(1, 0)
    D, L = 128, 640
    for H, HKV in ((16, 2), (8, 2)):
        g = torch.Generator(device="cuda").manual_seed(3)
        q1, do1 = (torch.randn(L, H, D, device="cuda", generator=g).bfloat16() for _ in range(2))
        k1, v1 = (torch.randn(L, HKV, D, device="cuda", generator=g).bfloat16() for _ in range(2))
        got, plans = [], []
        for B in (1, 3, 7):
            cu = torch.arange(B + 1, device="cuda", dtype=torch.int32) * L
            q, k, v, do = (x.repeat(B, 1, 1) for x in (q1, k1, v1, do1))
            o, lse = attention_forward(q, k, v, causal=True, cu_seqlens=cu, max_seqlen=L)
            run = prepare_backward(q, k, v, o, do, lse, causal=True, cu_seqlens=cu, max_seqlen=L)
            plans.append(run.plan)
            got.append(tuple(x[-L:].clone() for x in run()))
        assert plans[0] == plans[1] == plans[2] and plans[0].folds(H // HKV) == (H // HKV > 4)
        assert _same(got[0], got[1]) and _same(got[0], got[2])


def test_the_mma_main_loop_refuses_a_folding_plan():
    _, prepare_backward, Plan = _api()
    (q, k, v, o, do), lse = _dense(1, 4, 2, 256, seed=5)
    with pytest.raises(NotImplementedError, match="whole group"):
        prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(1, 0), kernel="mma")
    with pytest.raises(ValueError, match="heads per work item"):
        prepare_backward(q, k, v, o, do, lse, causal=True, plan=Plan(3, 0))


def test_mqa_and_small_batch_shapes_plan_by_default_and_stay_accurate():
    """A shape whose whole-group items cannot balance (B2 H32/1 at S 8192 in the reference's GQA
    sweep) takes a folding plan by default, and B1 H32/8 is where a folding plan (two heads at a
    time) and the private one (the default there) meet; checked here at S 2048 with those plans."""
    from fold_attention_b200.backward.plan import plan_dense

    _, prepare_backward, Plan = _api()
    assert plan_dense(2, 32, 1, 8192, 128, True) == Plan(4, 0)
    assert plan_dense(1, 32, 8, 8192, 128, True) == Plan(4, 0)
    for (B, H, HKV), plan in (((2, 32, 1), Plan(4, 0)), ((1, 32, 8), Plan(2, 0)), ((1, 32, 8), Plan(4, 0))):
        (q, k, v, o, do), lse = _dense(B, H, HKV, 2048, seed=6)
        run = prepare_backward(q, k, v, o, do, lse, causal=True, plan=plan)
        got = tuple(x.clone() for x in run())
        assert _same(got, run())
        ref = ob.reference_grads(q[0].transpose(0, 1)[:, :H // HKV], k[0].transpose(0, 1)[:, :1], v[0].transpose(0, 1)[:, :1],
                                 do[0].transpose(0, 1)[:, :H // HKV])
        assert ob.rel_l2(got[0][0].transpose(0, 1)[:, :H // HKV], ref[0]) <= TOL
        assert ob.rel_l2(got[1][0].transpose(0, 1)[:, :1], ref[1]) <= TOL
        assert ob.rel_l2(got[2][0].transpose(0, 1)[:, :1], ref[2]) <= TOL
