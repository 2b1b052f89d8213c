"""The decode's host side: validation, buffers, the launch closure.

`prepare_fold_decode` mirrors the reference's kernel-level entry
(src/fold_attention/decode/launch.py:380-500) for the single-level paged
decode: already-quantised planes plus an explicit reference (`reference=
"given"`) or the mass estimate (`reference="mass"`). The prepared launch
returns `(out, den, counts)`, the same tensors every call.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import _lib
from ..utils import Launch
from .rows import pack_tree

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
_lib.register(
    "fold_decode_run_ex",
    [P] * 14 + [I] * 10 + [F, F, P, F] + [P, P, P, P, I, P, P, P] + [P, I, P, I, I, I, I, P, I, P],
)
_lib.register("fold_mass_z_ex", [P, P, P, P, P, P, P, I, I, I, I, I, I, P, P, I, P, I, P])
_lib.register("fold_decode_counters", [P, I])
_lib.register("fold_decode_combine", [P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, P])

_OUT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
KERNELS = ("auto", "mma", "sm100")


class DecodeLaunch(Launch):
    pass


@dataclass
class SharedPrefix:
    """One shared level of a cascade: a prefix cache that several requests
    attend before their own keys, whose partials the combine adds to the
    unique level's under the rows' one reference.

    `ka`, `kb`, `ek`, `v` (and `v2`, V's second e4m3 plane) are the prefix's own
    paged pool in the cache's format, `page_table` `(n_prefixes, pages)` and
    `seq_lens` `(n_prefixes,)` its pages and lengths, read when the launch is
    prepared (a prefix does not grow). `req_map` `(requests,)` int32 names the
    prefix each request holds (-1: none; None: every request holds prefix 0).
    `vmean` `(n_prefixes * H_KV, D)` is the prefix's dropped-mass direction,
    given exactly when the unique level has one. Both levels share V's scale.

    The reference's `SharedPrefix` (src/fold_attention/decode/launch.py:48-80)
    names the requests' stacked rows (`cascade_rows`) and reads a prefix once
    for up to 64 of them; here every request's row group reads its prefix
    itself (the pages are the same, so L2 serves the repeats), which keeps a
    request's result independent of the requests it shares the prefix with.
    """

    ka: torch.Tensor
    kb: torch.Tensor
    ek: torch.Tensor
    v: torch.Tensor
    page_table: torch.Tensor
    seq_lens: torch.Tensor
    page_size: int
    req_map: torch.Tensor | None = None
    v2: torch.Tensor | None = None
    vmean: torch.Tensor | None = None
    split: int = 1


def mass_z(qa, qb, eq, ka, ek, page_table, page_size, seq_lens, n_kv_heads, z, *, req_map=None, tree=None, draft_len=0):
    """Each query row's estimated log-sum-exp (base 2) into `z` (NBH, G).
    A group of 16, 24 or 32 rows is estimated as groups of 8; `req_map` reads
    another cache's rows (a cascade's shared level), `tree` with `draft_len`
    hides the draft nodes a row does not see."""
    NBH, G, D = qa.shape
    gsub = 1 if G <= 8 else G // 8
    if G > 8 and (G % 8 or G > 32):
        raise NotImplementedError(f"a row group of {G} rows: 1..8, 16, 24 or 32 are supported")
    if gsub > 1 or req_map is not None or tree is not None:
        _lib.call(
            "fold_mass_z_ex", qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(), ek.data_ptr(),
            page_table.data_ptr(), seq_lens.data_ptr(), NBH * gsub, G // gsub, n_kv_heads, D, page_table.shape[1],
            int(page_size), z.data_ptr(), _lib.ptr(req_map), gsub, _lib.ptr(tree), int(draft_len) if tree is not None else 0,
            _lib.stream(qa.device),
        )
        return z
    _lib.call(
        "fold_mass_z", qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(), ek.data_ptr(),
        page_table.data_ptr(), seq_lens.data_ptr(), NBH, G, n_kv_heads, D, page_table.shape[1],
        int(page_size), z.data_ptr(), _lib.stream(qa.device),
    )
    return z


def prepare_fold_decode(
    qa, qb, eq, ka, kb, ek, v, z, cut, *,
    split=1, truncate=False, refine_k=10.0, refine_v=10.0, v8=False, v2=None, v_scale=1.0,
    vmean=None, page_table=None, page_size=0, seq_lens=None, n_kv_heads=1, reference="given", weight_terms=1,
    order=None, out_dtype=torch.float32, refine_bands=(), chunk_keys=0, out=None, kernel="mma",
    short_slots=0, tail=None, draft_len=1, causal=False, mask=None, shared=None, group_cut="auto", sound=False,
):
    """Bind one decode over a paged cache and return its launch.

    `qa`, `qb` int8 `(NBH, G, D)` and `eq` `(NBH, G)` are Q's planes and
    scales; `ka`, `kb`, `ek`, `v`, `v2` the pool; `z` `(NBH, G)` each row's
    reference (written by the launch when `reference="mass"`) and `cut` its
    depth below `z` under which a key is dropped (`truncate`). Calling the
    launch returns `(out (NBH, G, D), den (NBH, G), counts (NBH, 2))`.
    Without a `page_table` the cache is contiguous: `ka`, `kb`, `v` `(NBH, S, D)`
    and `ek` `(NBH, S)`, every row group `S` keys long unless `seq_lens` `(NBH,)`
    says otherwise (S a multiple of 64).
    `kernel` picks the split-KV kernel: "mma" (warp-level, every shape), "sm100"
    (tcgen05; D = 128, pages and chunks of a multiple of 128 keys; its weights are
    four E5M2 terms on an 8-bit V and two bf16 terms on a bf16 V, whatever
    `weight_terms` says) or "auto".
    With an `order`, its first `short_slots` slots stay on the warp-level kernel
    when the tcgen05 one takes the rest (requests too short for it to pay), and
    one combine follows both.
    `draft_len` with `causal` or `mask` verifies a draft: a row group is
    `G // draft_len` query heads at `draft_len` positions (`rows.pack_rows`),
    the draft's keys are the cache's last `draft_len`, and a row sees the nodes
    its word names (`rows.pack_tree`, `rows.draft_mask`). `shared` is a
    cascade: a `SharedPrefix` or a list of them. `group_cut` lets a gathered key
    enter every row of its group at its true weight; "auto" takes it for a
    single-level step and not for drafts and cascades, where each row keeps its
    own cut (reference: launch.py:602-640). Groups of 16, 24 or 32 rows run
    as groups of 8 on one KV head (an `order` then names those: `NBH * G / 8`
    slots). `sound` shifts the cut by the bound on what K's second plane can
    still add to a row's logit, so the screen drops only keys the full logit
    would drop too; `vmean` may be `(NBH, G, D)`, a direction per query row
    (single level). All of these run on the warp-level kernel.
    `tail` (a `tail.TailState`, or anything with `rows`, `u`, `vr` and `rank`)
    replaces `vmean` as where dropped mass re-enters: each 64-key block's row
    and, at rank 16, the part of a key's V its K predicts. It needs a
    truncating decode on a bf16 V, pages of a multiple of 64 keys, and the
    warp-level kernel (reference: decode/launch.py:380-500, `tail=`).
    """
    NBH, G, D = qa.shape
    if page_table is None:
        # a contiguous cache `(NBH, S, D)` is a paged one whose pages are the row groups themselves
        if ka.dim() != 3 or ka.shape[0] != NBH:
            raise ValueError(f"without a page table K's planes are ({NBH}, S, {D}) (got {tuple(ka.shape)})")
        S = ka.shape[1]
        if S % 64 and S not in (16, 32):
            raise NotImplementedError(f"a contiguous cache of {S} keys a row group: a multiple of 64 (or 16, 32); page it otherwise")
        page_table = torch.arange(NBH, device=qa.device, dtype=torch.int32).view(NBH, 1)
        page_size, n_kv_heads = S, 1
        if seq_lens is None:
            seq_lens = torch.full((NBH,), S, device=qa.device, dtype=torch.int32)
        elif seq_lens.numel() != NBH:
            raise ValueError(f"a contiguous cache's seq_lens has one length per row group ({NBH})")
        ka, kb, ek, v = ka.reshape(NBH * S, D), kb.reshape(NBH * S, D), ek.reshape(NBH * S), v.reshape(NBH * S, D)
        if v2 is not None:
            v2 = v2.reshape(NBH * S, D)
    elif seq_lens is None or page_size <= 0:
        raise ValueError("a paged cache is ragged: pass seq_lens and page_size")
    if G > 8 and (G % 8 or G > 32):
        raise NotImplementedError(f"a row group of {G} rows: 1..8, 16, 24 or 32 are supported")
    gsub = 1 if G <= 8 else G // 8
    q_len = int(draft_len)
    if q_len < 1:
        raise ValueError("draft_len is the number of draft positions per query head")
    if G % q_len:
        raise ValueError(f"G={G} is not a multiple of draft_len={q_len}: a row group is G // draft_len query heads at "
                         "draft_len positions each, row g * draft_len + t (see rows.pack_rows)")
    if causal and mask is not None:
        raise ValueError("causal=True and mask= are two answers to one question: put the chain in the bits or drop the mask")
    if q_len > 1 and gsub > 1:
        raise NotImplementedError("a draft's rows share one group of at most 8")
    levels = [] if shared is None else (list(shared) if isinstance(shared, (list, tuple)) else [shared])
    for lv in levels:
        if not isinstance(lv, SharedPrefix):
            raise TypeError("shared is a SharedPrefix or a list of them")
        if (lv.vmean is None) != (vmean is None):
            raise ValueError("vmean for both levels or neither")
        if (lv.v2 is None) != (not v8):
            raise ValueError("a shared level's V has the unique level's format")
        if lv.page_size < 16 or lv.page_size % 16 or (lv.page_size % 64 and 64 % lv.page_size):
            raise ValueError(f"a shared level's page_size={lv.page_size}: a multiple of 64, or 16 or 32")
    vmean_rows = vmean is not None and vmean.dim() == 3
    if vmean is not None and (vmean.dtype != torch.float32 or not vmean.is_contiguous()
                              or tuple(vmean.shape) not in ((NBH, D), (NBH, G, D))):
        raise ValueError(f"vmean is contiguous fp32 ({NBH}, {D}), a direction per KV head, or ({NBH}, {G}, {D}), one per query row")
    if vmean_rows and levels:
        raise NotImplementedError("a cascade's levels each take one direction per KV head")
    if group_cut == "auto":
        group_cut = bool(truncate) and G > 1 and q_len == 1 and not levels
    if group_cut not in (0, 1, False, True):
        raise ValueError('group_cut is True, False or "auto"')
    row_cut = bool(truncate) and not bool(group_cut) and G > 1
    tree = pack_tree(mask, bool(causal), q_len, G, NBH, qa.device) if (q_len > 1 and (causal or mask is not None)) else None
    sound = bool(sound) and bool(truncate)
    ex = gsub > 1 or tree is not None or bool(levels) or row_cut or sound or vmean_rows
    bound = torch.empty((NBH, G), device=qa.device, dtype=torch.float32) if sound else None
    if ex and (tail is not None or kernel == "sm100" or short_slots):
        raise NotImplementedError("drafts, cascades, wide row groups and a row's own cut run on the warp-level kernel "
                                  "(kernel='mma' or 'auto'), without a tail")
    if ex and levels and chunk_keys:
        raise ValueError("a cascade's levels interleave their splits: no fixed chunk")
    if ex and any(not t.is_contiguous() for t in (qa, qb, eq, z, cut)):
        raise ValueError("qa, qb, eq, z and cut are contiguous (NBH, G, ...) tensors")
    if gsub > 1 and order is not None and order.numel() != NBH * gsub:
        raise ValueError(f"an order over groups of {G} rows names the {NBH * gsub} groups of 8 they run as")
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
    use_sm100 = can and kernel in ("auto", "sm100") and not ex
    dev = qa.device
    split = int(split)
    slots = split + sum(int(lv.split) for lv in levels)
    o_part = torch.empty((NBH * slots, G, D), device=dev, dtype=torch.float32)
    den_part = torch.empty((NBH * slots, G), device=dev, dtype=torch.float32)
    cnt_part = torch.empty((NBH * gsub * slots, 2), device=dev, dtype=torch.int32)
    out_t = torch.empty((NBH, G, D), device=dev, dtype=out_dtype) if out is None else out
    den = torch.empty((NBH, G), device=dev, dtype=torch.float32)
    counts = torch.empty((NBH * gsub, 2), device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    bands = (ctypes.c_float * 6)(*refine_bands) if refine_bands else None
    fixed = (
        qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(), kb.data_ptr(), ek.data_ptr(),
        v.data_ptr(), _lib.ptr(v2) if v8 else None, _lib.ptr(vmean) if truncate else None,
        z.data_ptr(), cut.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), _lib.ptr(order),
        NBH * gsub, G // gsub, int(n_kv_heads), D, page_table.shape[1], int(page_size), split, int(chunk_keys),
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

    # ---- the layouts beyond the single-level step (fold_decode_run_ex) ----
    keep = []           # tensors the level calls read
    # the shared levels' key counts, the same tensor every call (the launch's closure must not hold the
    # launch itself: a reference cycle would keep a cache's pools alive until the collector runs)
    counts_shared = torch.zeros((NBH * gsub, 2), device=dev, dtype=torch.int32) if levels else None
    level_calls = []
    if ex:
        off = split
        for lv in levels:
            n_pre = lv.page_table.shape[0]
            rm = lv.req_map if lv.req_map is not None else torch.zeros(NBH // n_kv_heads, device=dev, dtype=torch.int32)
            # a request that holds no prefix reads an empty one appended to the level's tables
            pt = torch.cat([lv.page_table, torch.zeros_like(lv.page_table[:1])]).contiguous()
            sl = torch.cat([lv.seq_lens.to(torch.int32), torch.zeros(1, device=dev, dtype=torch.int32)]).contiguous()
            rm = torch.where(rm < 0, torch.full_like(rm, n_pre), rm).to(torch.int32).contiguous()
            vm = None
            if truncate and lv.vmean is not None:      # the empty prefix's direction: it has no mass to send there
                vm = torch.cat([lv.vmean.float(), torch.zeros((int(n_kv_heads), D), device=dev)]).contiguous()
            if rm.numel() != NBH // int(n_kv_heads) or int(rm.max()) > n_pre:
                raise ValueError(f"req_map names a prefix (or -1) for each of the {NBH // int(n_kv_heads)} requests")
            keep += [pt, sl, rm, vm, lv]
            level_calls.append((
                qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), lv.ka.data_ptr(), lv.kb.data_ptr(), lv.ek.data_ptr(),
                lv.v.data_ptr(), _lib.ptr(lv.v2) if v8 else None, _lib.ptr(vm),
                z.data_ptr(), cut.data_ptr(), pt.data_ptr(), sl.data_ptr(), None,
                NBH * gsub, G // gsub, int(n_kv_heads), D, pt.shape[1], int(lv.page_size), int(lv.split), 0,
                int(bool(truncate)), int(weight_terms), float(refine_k), float(refine_v),
                ctypes.addressof(bands) if bands is not None else None, float(v_scale),
                o_part.data_ptr(), den_part.data_ptr(), cnt_part.data_ptr(), None, 0, den.data_ptr(), counts.data_ptr(),
                status.data_ptr(), rm.data_ptr(), gsub, None, 0, slots, off, int(row_cut), _lib.ptr(bound), 0, _lib.stream(dev),
            ))
            off += int(lv.split)

    def ex_args(o):
        """The unique level: combined in the call when it is the only level."""
        a = list(fixed)
        a += [o.data_ptr() if not levels else None, _OUT[o.dtype], den.data_ptr(), counts.data_ptr(), status.data_ptr(),
              None, gsub, _lib.ptr(tree), q_len if tree is not None else 0, slots, 0, int(row_cut), _lib.ptr(bound),
              int(vmean_rows), _lib.stream(dev)]
        return a

    def run_mass():
        mass_z(qa, qb, eq, ka, ek, page_table, page_size, seq_lens, n_kv_heads, z, tree=tree, draft_len=q_len)
        for lv, call in zip(levels, level_calls):
            zl = torch.empty_like(z)
            _lib.call("fold_mass_z_ex", qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), lv.ka.data_ptr(), lv.ek.data_ptr(),
                      call[11], call[12], NBH * gsub, G // gsub, int(n_kv_heads), D, call[18], int(lv.page_size), zl.data_ptr(),
                      call[36], gsub, None, 0, _lib.stream(dev))
            z.copy_(torch.logaddexp2(z, zl))      # the rows' mass over both levels

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
            run_mass()
        if sound:   # the planes are this step's: the bound is too
            bound.copy_(eq * (qa.float().abs().sum(-1) * 128.0 + qb.float().abs().sum(-1) * 0.5))
        if ex:
            _lib.call("fold_decode_run_ex", *ex_args(o))
            if levels:
                for call in level_calls:
                    _lib.call("fold_decode_run_ex", *call)
                _lib.call(
                    "fold_decode_combine", o_part.data_ptr(), den_part.data_ptr(), cnt_part.data_ptr(),
                    seq_lens.data_ptr(), o.data_ptr(), _OUT[o.dtype], den.data_ptr(), counts.data_ptr(), NBH * gsub, G // gsub, D,
                    int(n_kv_heads) * gsub, slots, 0, float(v_scale), _lib.stream(dev),
                )
                # the combine counted every level's keys: keep the unique level's, and the shared levels' apart
                per = cnt_part.view(NBH * gsub, slots, 2)
                counts_shared.copy_(per[:, split:].sum(1, dtype=torch.int32))
                counts.copy_(per[:, :split].sum(1, dtype=torch.int32))
        elif tail is not None:
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
         den_part, cnt_part, out_t, den, counts, status, bands, tail, tree, keep, bound),
    )
    launch.counts_shared = counts_shared
    launch.z = z
    launch.status = status
    launch.kernel = ("sm100+mma" if short_slots else "sm100") if use_sm100 else "mma"
    launch.tree = tree
    return launch


def fold_decode(qa, qb, eq, ka, kb, ek, v, z, cut, **kw):
    """One decode step: `prepare_fold_decode(...)()`, returning `(out, den, counts)`
    (reference: decode/launch.py:503-506)."""
    return prepare_fold_decode(qa, qb, eq, ka, kb, ek, v, z, cut, **kw)()


def capture_decode(launch, warmup=3):
    """A prepared decode captured in a CUDA graph; the returned launch replays it.

    The replay reads and writes the tensors `launch` was bound to: their
    contents may change between replays, the tensors themselves may not. A
    launch that was bound with `sound=True` or a cascade under the mass
    reference runs a few torch kernels of its own, which are captured too
    (reference: decode/launch.py:1333-1360)."""
    for _ in range(int(warmup)):
        launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            result = launch()
    torch.cuda.synchronize()

    def replay(out=None):
        if out is not None:
            raise ValueError("a captured decode writes the output it was captured with")
        graph.replay()
        return result

    captured = DecodeLaunch(replay, (launch, side, graph))
    for name in ("z", "status", "kernel", "tree", "counts_shared"):
        setattr(captured, name, getattr(launch, name, None))
    return captured
