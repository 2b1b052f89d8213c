"""The decode through the library's built-in scratch, for hosts that may not
allocate device memory while a step runs (a serving plugin given a fixed
amount of memory, a process whose device allocator belongs to another runtime).

`decode_static` takes the same planes as `prepare_fold_decode`, but the split
partials live in a fixed 4 MiB array inside libfold_b200 instead of in torch
buffers, so the call itself allocates nothing: the caller passes the inputs
and the outputs `out`, `den`, `counts`, `status`. Calls on one device share
that array, so they must be stream-ordered (calls on two streams or from two
threads race on it); a call too large for it raises ValueError. `order`, if
given, must be a permutation of all the call's row groups: the array has room
for those and no others, and a slot that points elsewhere sets `status` to 1
on the device instead of writing. The first call on a device resolves the array's address and
should come before any stream capture starts.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib

P, I, F, Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
_lib.register("fold_decode_static_scratch_needed", [I, I, I, I], Z)
_lib.register("fold_decode_run_static", [P] * 14 + [I] * 10 + [F, F, P, F] + [P, I, P, P, P, P])

SCRATCH_BYTES = 4 << 20
_OUT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def scratch_needed(n_groups, group, head_dim, split):
    return _lib.lib.fold_decode_static_scratch_needed(n_groups, group, head_dim, split)


def decode_static(
    qa, qb, eq, ka, kb, ek, v, z, cut, out, den, counts, status, *, split, truncate, refine_k,
    refine_v, v2=None, v_scale=1.0, vmean=None, page_table, page_size, seq_lens, n_kv_heads,
    weight_terms=1, order=None, refine_bands=(), chunk_keys=0,
):
    """One decode + combine into the caller's `out` (NBH, G, D), `den`
    (NBH, G) and `counts` (NBH, 2); `status` is an int32[1] device tensor."""
    NBH, G, D = qa.shape
    bands = (ctypes.c_float * 6)(*refine_bands) if refine_bands else None
    _lib.call(
        "fold_decode_run_static", qa.data_ptr(), qb.data_ptr(), eq.data_ptr(), ka.data_ptr(),
        kb.data_ptr(), ek.data_ptr(), v.data_ptr(), _lib.ptr(v2), _lib.ptr(vmean) if truncate else None,
        z.data_ptr(), cut.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), _lib.ptr(order),
        NBH, G, int(n_kv_heads), D, page_table.shape[1], int(page_size), int(split), int(chunk_keys),
        int(bool(truncate)), int(weight_terms), float(refine_k), float(refine_v),
        ctypes.addressof(bands) if bands is not None else None, float(v_scale),
        out.data_ptr(), _OUT[out.dtype], den.data_ptr(), counts.data_ptr(), status.data_ptr(),
        _lib.stream(qa.device),
    )
    return out, den, counts
