"""The decode's host side: validation, buffers, the launch closure.

`prepare_fold_decode` mirrors the reference's kernel-level entry
(src/fold_attention/decode/launch.py:380-500) for the single-level paged
decode: already-quantised planes plus an explicit reference (`reference=
"given"`) or the mass estimate (`reference="mass"`). The prepared launch
returns `(out, den, counts)`, the same tensors every call.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..utils import Launch

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_lib.register("fold_mass_z", [P, P, P, P, P, P, P, I, I, I, I, I, I, P, P])
_lib.register(
    "fold_decode_run",
    [P] * 14 + [I] * 10 + [F, F, P, F] + [P, P, P, P, I, P, P, P, P],
)

_lib.register("fold_decode_sm100_supported", [I, I, I, I, I])
_lib.register(
    "fold_decode_run_sm100",
    [P] * 14 + [I] * 9 + [F, F, P, F] + [P, P, P, P, I, P, P, P, P],
)
_lib.register(
    "fold_decode_run_tail",
    [P] * 10 + [I] + [P] * 5 + [I] * 9 + [F] + [P, P, P, P, I, P, P, P, P],
)
_lib.register("fold_decode_combine", [P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P])

_OUT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
KERNELS = ("auto", "mma", "sm100")


class DecodeLaunch(Launch):
    pass


def mass_z(qa, qb, eq, ka, ek, page_table, page_size, seq_lens, n_kv_heads, z):
    """Each query row's estimated log-sum-exp (base 2) into `z` (NBH, G)."""
    NBH, G, D = qa.shape
    _lib.call(
        "fold_mass_z", qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(), ek.data_ptr(),
        page_table.data_ptr(), seq_lens.data_ptr(), NBH, G, n_kv_heads, D, page_table.shape[1],
        int(page_size), z.data_ptr(), _lib.stream(qa.device),
    )
    return z


def prepare_fold_decode(
    qa, qb, eq, ka, kb, ek, v, z, cut, *,
    split=1, truncate=False, refine_k=10.0, refine_v=10.0, v8=False, v2=None, v_scale=1.0,
    vmean=None, page_table, page_size, seq_lens, n_kv_heads, reference="given", weight_terms=1,
    order=None, out_dtype=torch.float32, refine_bands=(), chunk_keys=0, out=None, kernel="mma",
    short_slots=0, tail=None,
):
    """Bind one decode over a paged cache and return its launch.

    `qa`, `qb` int8 `(NBH, G, D)` and `eq` `(NBH, G)` are Q's planes and
    scales; `ka`, `kb`, `ek`, `v`, `v2` the pool; `z` `(NBH, G)` each row's
    reference (written by the launch when `reference="mass"`) and `cut` its
    depth below `z` under which a key is dropped (`truncate`). Calling the
    launch returns `(out (NBH, G, D), den (NBH, G), counts (NBH, 2))`.
    `kernel` picks the split-KV kernel: "mma" (warp-level, every shape), "sm100"
    (tcgen05; D = 128, pages and chunks of a multiple of 128 keys; its weights are
    four E5M2 terms on an 8-bit V and two bf16 terms on a bf16 V, whatever
    `weight_terms` says) or "auto".
    With an `order`, its first `short_slots` slots stay on the warp-level kernel
    when the tcgen05 one takes the rest (requests too short for it to pay), and
    one combine follows both.
    `tail` (a `tail.TailState`, or anything with `rows`, `u`, `vr` and `rank`)
    replaces `vmean` as where dropped mass re-enters: each 64-key block's row
    and, at rank 16, the part of a key's V its K predicts. It needs a
    truncating decode on a bf16 V, pages of a multiple of 64 keys, and the
    warp-level kernel (reference: decode/launch.py:380-500, `tail=`).
    """
    NBH, G, D = qa.shape
    if G > 8:
        raise NotImplementedError(f"a row group of {G} rows: 1..8 are supported")
    if D not in (64, 128):
        raise NotImplementedError(f"head_dim {D}: the decode takes 64 or 128")
    if v8 and v2 is None:
        raise ValueError("an 8-bit V has two planes: pass v2")
    if not v8 and v.dtype != torch.bfloat16:
        raise ValueError("a 16-bit V cache is bf16")
    if reference not in ("given", "mass"):
        raise ValueError("reference is 'given' or 'mass'")
    if chunk_keys % 64:
        raise ValueError(f"chunk={chunk_keys} is not a multiple of 64")
    if kernel not in KERNELS:
        raise ValueError(f"kernel is one of {KERNELS}")
    if tail is not None:
        if not truncate:
            raise ValueError("the tail re-enters truncated mass: it needs truncate")
        if v8:
            raise ValueError("the decode tail needs a bf16 V cache")
        if vmean is not None:
            raise ValueError("a tail replaces vmean: pass one of them")
        if page_size % 64:
            raise ValueError(f"page_size={page_size}: the tail keeps one row per 64 keys, so a page must hold whole blocks")
        if tail.rank not in (0, 16):
            raise ValueError(f"tail rank {tail.rank}: 0 (block rows alone) or 16")
        if tail.rows.dtype != torch.bfloat16 or tail.rows.shape != (ka.shape[0] // 64, D):
            raise ValueError(f"the tail's rows are bf16 ({ka.shape[0] // 64}, {D}): one per 64 pool rows")
        if tail.rank and (tail.u.shape != (NBH, 16, D) or tail.vr.shape != (NBH, D, 16)
                          or tail.u.dtype != torch.int8 or tail.vr.dtype != torch.float32):
            raise ValueError(f"the tail's u is int8 ({NBH}, 16, {D}) and vr fp32 ({NBH}, {D}, 16)")
        if kernel == "sm100":
            raise NotImplementedError("the tail runs on the warp-level kernel: kernel='mma' or 'auto'")
        kernel = "mma"
    can = bool(_lib.lib.fold_decode_sm100_supported(G, D, int(page_size), int(chunk_keys), int(bool(v8))))
    if kernel == "sm100" and not can:
        raise NotImplementedError(
            "the tcgen05 decode takes head_dim 128, pages and chunks of a multiple of 128 keys")
    use_sm100 = can and kernel in ("auto", "sm100")
    dev = qa.device
    split = int(split)
    o_part = torch.empty((NBH * split, G, D), device=dev, dtype=torch.float32)
    den_part = torch.empty((NBH * split, G), device=dev, dtype=torch.float32)
    cnt_part = torch.empty((NBH * split, 2), device=dev, dtype=torch.int32)
    out_t = torch.empty((NBH, G, D), device=dev, dtype=out_dtype) if out is None else out
    den = torch.empty((NBH, G), device=dev, dtype=torch.float32)
    counts = torch.empty((NBH, 2), device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    bands = (ctypes.c_float * 6)(*refine_bands) if refine_bands else None
    fixed = (
        qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(), kb.data_ptr(), ek.data_ptr(),
        v.data_ptr(), _lib.ptr(v2) if v8 else None, _lib.ptr(vmean) if truncate else None,
        z.data_ptr(), cut.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), _lib.ptr(order),
        NBH, G, int(n_kv_heads), D, page_table.shape[1], int(page_size), split, int(chunk_keys),
        int(bool(truncate)), int(weight_terms), float(refine_k), float(refine_v),
        ctypes.addressof(bands) if bands is not None else None, float(v_scale),
        o_part.data_ptr(), den_part.data_ptr(), cnt_part.data_ptr(),
    )
    short_slots = int(short_slots) if (use_sm100 and order is not None) else 0
    if not 0 <= short_slots <= NBH:
        raise ValueError(f"short_slots={short_slots} of {NBH} slots")
    if short_slots == NBH:
        use_sm100, short_slots = False, 0

    def args(first, count, sm100, o):
        """One call's arguments over `count` slots from slot `first`; `o` None: partials only."""
        a = list(fixed)
        if first or count != NBH:
            a[13] = order.data_ptr() + 4 * first
            a[14] = count
        if sm100:
            del a[23]   # the tcgen05 kernel has no weight_terms
        a += [o.data_ptr() if o is not None else None, _OUT[out_t.dtype] if o is None else _OUT[o.dtype],
              den.data_ptr(), counts.data_ptr(), status.data_ptr(), _lib.stream(dev)]
        return a

    def tail_args(o):
        return [
            qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(), kb.data_ptr(), ek.data_ptr(), v.data_ptr(),
            tail.rows.data_ptr(), _lib.ptr(tail.u), _lib.ptr(tail.vr), tail.rank, z.data_ptr(), cut.data_ptr(),
            page_table.data_ptr(), seq_lens.data_ptr(), _lib.ptr(order), NBH, G, int(n_kv_heads), D,
            page_table.shape[1], int(page_size), split, int(chunk_keys), int(weight_terms), float(refine_k),
            o_part.data_ptr(), den_part.data_ptr(), cnt_part.data_ptr(), o.data_ptr(), _OUT[o.dtype],
            den.data_ptr(), counts.data_ptr(), status.data_ptr(), _lib.stream(dev),
        ]

    def run(out=None):
        o = out_t if out is None else out
        if reference == "mass":
            mass_z(qa, qb, eq, ka, ek, page_table, page_size, seq_lens, n_kv_heads, z)
        if tail is not None:
            _lib.call("fold_decode_run_tail", *tail_args(o))
        elif use_sm100 and short_slots:
            _lib.call("fold_decode_run_sm100", *args(short_slots, NBH - short_slots, True, None))
            _lib.call("fold_decode_run", *args(0, short_slots, False, None))
            _lib.call(
                "fold_decode_combine", o_part.data_ptr(), den_part.data_ptr(), cnt_part.data_ptr(),
                seq_lens.data_ptr(), o.data_ptr(), _OUT[o.dtype], den.data_ptr(), counts.data_ptr(), NBH, G, D,
                int(n_kv_heads), split, int(chunk_keys), float(v_scale), _lib.stream(dev),
            )
        elif use_sm100:
            _lib.call("fold_decode_run_sm100", *args(0, NBH, True, o))
        else:
            _lib.call("fold_decode_run", *args(0, NBH, False, o))
        return o, den, counts

    launch = DecodeLaunch(
        run,
        (qa, qb, eq, ka, kb, ek, v, v2, vmean, z, cut, page_table, seq_lens, order, o_part,
         den_part, cnt_part, out_t, den, counts, status, bands, tail),
    )
    launch.z = z
    launch.status = status
    launch.kernel = ("sm100+mma" if short_slots else "sm100") if use_sm100 else "mma"
    return launch
