"""Reference gradients and integer-grid exponents of the deterministic
backward. Test infrastructure only.

`reference_grads` is the FP64 autograd statement the reference's tests hold
(tests/test_backward.py:79-92; the FP32 twin is
benchmarks/harness/training.py:124-164). The grid functions restate
src/fold_attention/backward/grid.py:41-100, which exists only as device code in
the reference: pure functions of four maxima, evaluated one rounded fp32
operation at a time, so they are exact; parity with the reference's integer
accumulator *bits* is unpinned (those depend on tensor-core summation order).
"""

from __future__ import annotations

import math

import numpy as np
import torch

F32 = np.float32
DQ_BITS = 30


def root_d(D: int) -> float:
    """sqrt(D) rounded up to a power of two (grid.py:36-38)."""
    return float(2 ** math.ceil(math.log2(math.sqrt(D))))


def pow2_scale_exp(bound, bits: int) -> int:
    """bits - ceil(log2(bound * (1 + 2^-6))), clamped to [-100, 100]; 100 for
    a zero bound (grid.py:41-53)."""
    b = F32(F32(bound) * F32(1.0 + 2.0**-6))
    bb = int(np.array(b, F32).view(np.int32))
    clog = ((bb >> 23) & 0xFF) - 127 + (1 if bb & 0x7FFFFF else 0)
    s = bits - clog
    if not b > 0:
        s = 100
    return max(-100, min(100, s))


def dq_scale_exp(max_k, max_v, max_do_norm, max_delta, D: int) -> int:
    """dQ's grid exponent for one (request, KV head) (grid.py:71-83):
    bound = (||dO||max * C_D * |V|max + |Delta|max) * |K|max."""
    t = F32(F32(max_do_norm) * F32(F32(max_v) * F32(root_d(D))))
    s = F32(t + F32(max_delta))
    return pow2_scale_exp(F32(s * F32(max_k)), DQ_BITS)


DKV_BITS = 61


def dv_scale_exp(max_doc, rows, bits: int) -> int:
    """dV's grid exponent when a key block's dV is summed across CTAs (grid.py:86-90):
    bound = rows * max |dO_id|, rows = G * sequence length bounding the column mass."""
    return pow2_scale_exp(F32(F32(rows) * F32(max_doc)), bits)


def dk_scale_exp(max_v, max_do_norm, max_delta, max_q, rows, D: int) -> int:
    """dK's grid exponent on its 61-bit grid (grid.py:93-100):
    bound = rows * (||dO||max * C_D * |V|max + |Delta|max) * |Q|max."""
    t = F32(F32(max_do_norm) * F32(F32(max_v) * F32(root_d(D))))
    s = F32(t + F32(max_delta))
    return pow2_scale_exp(F32(F32(rows) * F32(s * F32(max_q))), DKV_BITS)


def stats(q, k, v, o, do, G):
    """The preprocess's maxima for one request, (S, H, D) tensors: per KV head
    max|K|, max|V|, max_i ||dO_i||, max_i |Delta_i| over the group's rows
    (preprocess.py:253-309). Row sums in fp32."""
    dn = do.float().pow(2).sum(-1).sqrt()  # (S, H)
    dl = (do.float() * o.float()).sum(-1).abs()
    HKV = k.shape[1]
    out = []
    for h in range(HKV):
        out.append((
            float(k[:, h].float().abs().max()), float(v[:, h].float().abs().max()),
            float(dn[:, h * G:(h + 1) * G].max()), float(dl[:, h * G:(h + 1) * G].max()),
        ))
    return out


def reference_grads(q, k, v, do, causal=True, scale=None, dtype=torch.float64):
    """Gradients of softmax attention for one request, (S, H, D) inputs;
    returns (dq, dk, dv) in `dtype` with dk, dv summed over each GQA group."""
    S, H, D = q.shape
    G = H // k.shape[1]
    sc = 1.0 / math.sqrt(D) if scale is None else scale
    qd = q.to(dtype).requires_grad_()
    kd = k.to(dtype).repeat_interleave(G, 1).requires_grad_()
    vd = v.to(dtype).repeat_interleave(G, 1).requires_grad_()
    s = torch.einsum("shd,thd->hst", qd, kd) * sc
    if causal:
        s = s.masked_fill(torch.ones(S, S, device=q.device, dtype=torch.bool).triu(1), float("-inf"))
    out = torch.einsum("hst,thd->shd", s.softmax(-1), vd)
    out.backward(do.to(dtype))
    return (
        qd.grad,
        kd.grad.view(S, H // G, G, D).sum(2),
        vd.grad.view(S, H // G, G, D).sum(2),
    )


def reference_forward(q, k, v, causal=True, scale=None, dtype=torch.float64):
    """O (S, H, D) and LSE (H, S) in nats for one request."""
    S, H, D = q.shape
    G = H // k.shape[1]
    sc = 1.0 / math.sqrt(D) if scale is None else scale
    kd = k.to(dtype).repeat_interleave(G, 1)
    vd = v.to(dtype).repeat_interleave(G, 1)
    s = torch.einsum("shd,thd->hst", q.to(dtype), kd) * sc
    if causal:
        s = s.masked_fill(torch.ones(S, S, device=q.device, dtype=torch.bool).triu(1), float("-inf"))
    return torch.einsum("hst,thd->shd", s.softmax(-1), vd), torch.logsumexp(s, -1)


def rel_l2(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm()).item()
