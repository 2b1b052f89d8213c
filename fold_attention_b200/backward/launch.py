"""The backward's host side: bind one call's tensors, return the launch.

Mirrors `prepare_backward` of the reference
(src/fold_attention/backward/launch.py:75-117): the launch returns `(dq, dk,
dv)`, the same tensors on every call, and owns its workspace, so two captured
graphs never share one. All device work goes through the C ABI
(`fold_bwd_run`): preprocess, main loop, postprocess on the current stream,
with no host synchronisation.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from .. import _lib
from ..utils import Launch, check_status
from .plan import Plan, plan_dense, plan_varlen, tile_config

P, I, F, Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
_lib.register("fold_bwd_workspace_bytes", [I, I, I, I, I, I, I, I, I], Z)
_lib.register("fold_bwd_workspace_layout", [I, I, I, I, I, I, I, I, I, P])
_lib.register(
    "fold_bwd_run",
    [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, Z, I, I, I, P],
)
_lib.register(
    "fold_bwd_run_phases",
    [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, Z, I, I, I, I, P],
)
_lib.register("fold_bwd_counters", [P, I])
_lib.register("fold_wait_probe", [ctypes.c_longlong, P, P, P])
_lib.register("fold_fwd_run", [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P])
_lib.register("fold_fwd_sm100_supported", [I, I])
_lib.register("fold_fwd_run_sm100", [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P])

KERNELS = {"auto": 0, "mma": 1, "sm100": 2}


@dataclass(eq=False)
class BackwardLaunch(Launch):
    """`prepare_backward`'s result: calling it returns `(dq, dk, dv)`."""

    plan: Plan | None = None
    workspace: torch.Tensor | None = None
    layout: tuple | None = None


def _strides(tensors, varlen):
    """(batch, row, head) element strides of `(B, H, S, D)` views or packed
    `(total, H, D)` tensors, as a host int64 array."""
    out = []
    for t in tensors:
        if t.stride(-1) != 1:
            raise ValueError("the head dim must be contiguous")
        if varlen:
            out += [0, t.stride(0), t.stride(1)]
        else:
            out += [t.stride(0), t.stride(2), t.stride(1)]
    return (ctypes.c_int64 * len(out))(*out)


def prepare_backward(
    q,
    k,
    v,
    o,
    do,
    lse,
    *,
    causal,
    softmax_scale=None,
    cu_seqlens=None,
    max_seqlen=None,
    out_dtype=None,
    plan: Plan | None = None,
    kernel: str = "auto",
):
    """Bind dQ, dK and dV of causal or full self-attention to one call's
    tensors, and return the launch that computes them.

    Dense: `(B, H, S, D)` views and `lse` `(B, H, S)`. Varlen: `(total, H, D)`
    packed by `cu_seqlens` `(B + 1,)` int32, and `lse` `(H, total)`. `lse` is
    in nats. `kernel` picks the main loop: "auto" (tcgen05 where it applies),
    "mma" or "sm100". `plan` cuts the work (`plan_dense` / `plan_varlen` by
    default): the tcgen05 main loop takes any `Plan`, the mma.sync one only
    whole groups over whole query ranges.
    """
    varlen = cu_seqlens is not None
    if varlen:
        total, H, D = q.shape
        H_KV = k.shape[1]
        B = cu_seqlens.shape[0] - 1
        if max_seqlen is None:
            max_seqlen = int(torch.diff(cu_seqlens).max())
        S = int(max_seqlen)
    else:
        B, H, S, D = q.shape
        H_KV = k.shape[1]
        total = B * S
        if k.shape[2] != S:
            raise NotImplementedError("the integer grids assume self-attention")
    if v.shape[-1] != D:
        raise NotImplementedError("the value head dim must equal the key head dim")
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("q, k and v must be bf16 or fp16")
    # the kernels index every tensor by q's sizes: anything that does not match would be read or written past its end
    lead = (total,) if varlen else (B,)
    if k.dim() != q.dim() or tuple(k.shape[:1]) != lead or k.shape[-1] != D or v.shape != k.shape:
        raise ValueError(f"k and v {tuple(k.shape)}, {tuple(v.shape)} do not match q {tuple(q.shape)}")
    if o.shape != q.shape or do.shape != q.shape:
        raise ValueError(f"o and do are q's shape {tuple(q.shape)} (got {tuple(o.shape)}, {tuple(do.shape)})")
    if tuple(lse.shape) != ((H, total) if varlen else (B, H, S)):
        raise ValueError(f"lse is {'(H, total)' if varlen else '(B, H, S)'} (got {tuple(lse.shape)})")
    if any(t.dtype != q.dtype for t in (k, v, o, do)):
        raise ValueError("q, k, v, o and do must be the same 16-bit type")
    if any(t.device != q.device for t in (k, v, o, do, lse)) or any(t.stride(-1) != 1 for t in (q, k, v, o, do)):
        raise ValueError("q, k, v, o, do and lse are on one device, each with a contiguous head dim")
    if varlen and (cu_seqlens.dtype != torch.int32 or cu_seqlens.device != q.device):
        raise ValueError("cu_seqlens is int32 on q's device")
    if H % H_KV:
        raise ValueError("the query heads must be a multiple of the KV heads")
    if D not in (64, 96, 128):
        raise NotImplementedError(f"head_dim {D}: 64, 96 and 128 are supported")
    if out_dtype is not None and out_dtype != q.dtype:
        raise NotImplementedError("gradients are returned in the inputs' dtype")
    dev = q.device
    sm = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    if kernel not in KERNELS:
        raise ValueError(f"kernel is one of {tuple(KERNELS)}")
    G = H // H_KV
    cfg = tile_config(D, kernel)
    if plan is None:
        plan = plan_varlen(H, H_KV, cfg) if varlen else plan_dense(B, H, H_KV, S, D, bool(causal), cfg)
    if plan.subgroup < 1 or G % plan.subgroup or plan.record < 0:
        raise ValueError(f"a plan of {plan.subgroup} heads per work item for groups of {G}")
    if plan.folds(G) and cfg.tile_n != 128:
        raise NotImplementedError(
            "the mma.sync main loop keeps a key block's dK and dV in one CTA: its plan is the whole group over the whole range")
    lse = lse.contiguous()
    if lse.dtype != torch.float32:
        raise ValueError("lse must be fp32")
    dq, dk, dv = (torch.empty_like(x) for x in (q, k, v))
    nbytes = _lib.lib.fold_bwd_workspace_bytes(B, H, H_KV, S, total, D, int(varlen), plan.subgroup, plan.record)
    workspace = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    lay = (ctypes.c_int64 * 11)()
    _lib.call("fold_bwd_workspace_layout", B, H, H_KV, S, total, D, int(varlen), plan.subgroup, plan.record, lay)
    tensors = (q, k, v, o, do, dq, dk, dv)
    strides = _strides(tensors, varlen)
    cu = cu_seqlens
    args = (
        q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ctypes.addressof(strides),
        _lib.ptr(cu), B, H, H_KV, S, total, D, int(bool(causal)),
        int(q.dtype == torch.float16), sm, workspace.data_ptr(), nbytes, KERNELS[kernel],
        plan.subgroup, plan.record,
    )

    def run():
        _lib.call("fold_bwd_run", *args, _lib.stream(dev))
        return dq, dk, dv

    def run_phase(phases):
        """One or more of the backward's phases (1 preprocess, 8 work list,
        2 main loop, 4 postprocess; in that order), for callers that time them
        apart or look at the work list between them."""
        _lib.call("fold_bwd_run_phases", *args, int(phases), _lib.stream(dev))

    held = (q, k, v, o, do, lse, dq, dk, dv, workspace, cu, strides)
    launch = BackwardLaunch(run, held, plan, workspace, tuple(lay))
    launch.run_phase = run_phase
    launch.status = workspace[lay[5]: lay[5] + 4].view(torch.int32)
    # the work list as the device built it (n_items, 8): key block, KV head, request, first head,
    # heads, first / one-past-last query block, cost in tiles; and, for a folding plan, the integer
    # dK and dV accumulators [H_KV, padded rows, D]
    launch.work = workspace[lay[9]: lay[9] + 32 * lay[10]].view(torch.int32).view(-1, 8)
    launch.dk_acc = launch.dv_acc = None
    if lay[8]:
        rows_p = lay[4]
        launch.dk_acc = workspace[lay[6]: lay[6] + 8 * H_KV * rows_p * D].view(torch.int64).view(H_KV, rows_p, D)
        wide = lay[8] == 64
        launch.dv_acc = workspace[lay[7]: lay[7] + (8 if wide else 4) * H_KV * rows_p * D].view(
            torch.int64 if wide else torch.int32).view(H_KV, rows_p, D)
    return launch


def attention_forward(q, k, v, *, causal, softmax_scale=None, cu_seqlens=None, max_seqlen=None, kernel="auto"):
    """O and LSE (nats) of self-attention through the library's own forward.

    Dense: `(B, S, H, D)` tensors, lse `(B, H, S)`. Varlen: `(total, H, D)`,
    lse `(H, total)`. Stands in for the third-party forward the reference
    calls (src/fold_attention/interface.py:42-44,70-81). `kernel`: "mma" (warp-level,
    every head dim), "sm100" (tcgen05; head_dim 128) or
    "auto"."""
    if kernel not in ("auto", "mma", "sm100"):
        raise ValueError('kernel is one of ("auto", "mma", "sm100")')
    varlen = cu_seqlens is not None
    D = q.shape[-1]
    # the kernels index k and v by q's batch, length and head dim: a mismatch would read past them
    if q.dim() != (3 if varlen else 4) or k.dim() != q.dim() or v.shape != k.shape:
        raise ValueError(f"q is {'(total, H, D)' if varlen else '(B, S, H, D)'}, k and v the same with H_KV heads "
                         f"(got q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)})")
    if k.shape[:-2] != q.shape[:-2] or k.shape[-1] != D or q.shape[-2] % k.shape[-2]:
        raise ValueError(f"k and v {tuple(k.shape)} do not match q {tuple(q.shape)}: same leading sizes and head dim, "
                         "and a head count that divides q's")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"q, k and v must be bf16 or fp16, and the same type (got {q.dtype}, {k.dtype}, {v.dtype})")
    if any(t.stride(-1) != 1 for t in (q, k, v)) or k.device != q.device or v.device != q.device:
        raise ValueError("q, k and v are on one device with a contiguous head dim")
    if varlen and (cu_seqlens.dtype != torch.int32 or cu_seqlens.device != q.device):
        raise ValueError("cu_seqlens is int32 on q's device")
    sm = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    o = torch.empty_like(q)
    if varlen:
        total, H, _ = q.shape
        B = cu_seqlens.shape[0] - 1
        if max_seqlen is None:
            max_seqlen = int(torch.diff(cu_seqlens).max())
        S = int(max_seqlen)
        lse = torch.empty((H, total), device=q.device, dtype=torch.float32)
        st = []
        for t in (q, k, v, o):
            st += [0, t.stride(0), t.stride(1)]
    else:
        B, S, H, _ = q.shape
        total = B * S
        lse = torch.empty((B, H, S), device=q.device, dtype=torch.float32)
        st = []
        for t in (q, k, v, o):
            st += [t.stride(0), t.stride(1), t.stride(2)]
    strides = (ctypes.c_int64 * 12)(*st)
    can = bool(_lib.lib.fold_fwd_sm100_supported(D, int(q.dtype == torch.float16)))
    if kernel == "sm100" and not can:
        raise NotImplementedError("the tcgen05 forward takes head_dim 128")
    if can and kernel != "mma":
        status = torch.zeros(1, device=q.device, dtype=torch.int32)
        _lib.call(
            "fold_fwd_run_sm100", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
            ctypes.addressof(strides), _lib.ptr(cu_seqlens), B, H, k.shape[-2], S, total, D,
            int(bool(causal)), int(q.dtype == torch.float16), sm, status.data_ptr(), _lib.stream(q.device),
        )
        attention_forward.last_status = status   # non-zero after a device-side wait ran out
        if attention_forward.check_status:
            check_status(status, "attention_forward")
        return o, lse
    _lib.call(
        "fold_fwd_run", q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
        ctypes.addressof(strides), _lib.ptr(cu_seqlens), B, H, k.shape[-2], S, total, D,
        int(bool(causal)), int(q.dtype == torch.float16), sm, _lib.stream(q.device),
    )
    return o, lse


# The tcgen05 forward's status word of the last call; with `check_status` set every call reads
# it back (one host synchronisation per call) and raises FoldLibraryError when it is raised.
attention_forward.last_status = None
attention_forward.check_status = False
