"""Every write into the serving cache: a prompt's, and a decode step's Q and
new token. Host side of `fold_cache_write_prompt` and `fold_step_append`;
mirrors `write_prompt` and `step` of the reference
(src/fold_attention/decode/write.py:676-724, 931-1009)."""

from __future__ import annotations

import torch

from .. import _lib

# A prompt's reductions run over fixed chunks counted from its request's start
# and are summed in order, so its V sum is its own bits whatever the batch.
CHUNK = 256


def chunk_table(lens):
    """The prompt writer's chunk table as a host int32 tensor:
    first[batch + 1] padded to four entries, then (request, first token,
    first position, count) per 256-token chunk."""
    first, rows, t0 = [0], [], 0
    for b, n in enumerate(lens):
        for p0 in range(0, n, CHUNK):
            rows += (b, t0 + p0, p0, min(CHUNK, n - p0))
        first.append(len(rows) // 4)
        t0 += n
    first += [0] * (-len(first) % 4)
    return torch.tensor(first + rows, dtype=torch.int32), len(rows) // 4


def write_prompt(
    k, v, lens, page_table, page_size, ka, kb, va, vb, ek, vsum, vmean, *, v_headroom, v_scale
):
    """Quantise packed prompts `(total, H_KV, D)` of host lengths `lens` into
    the paged cache, each key's scale into the pool `ek`, and each row
    group's V sum and mean. Returns V's scale as a one-element device tensor;
    nothing here waits on the device."""
    total, HKV, D = k.shape
    if k.dtype not in (torch.bfloat16, torch.float16) or v.dtype != k.dtype:
        raise ValueError("k and v must be bf16 or fp16")
    if sum(lens) != total:
        raise ValueError(f"lens sum to {sum(lens)} but k holds {total} tokens")
    k, v = k.contiguous(), v.contiguous()
    dev = k.device
    meta, nc = chunk_table(lens)
    meta = meta.pin_memory().to(dev, non_blocking=True) if dev.type == "cuda" else meta
    scratch = torch.empty(nc * HKV * (D + 1) + 1, device=dev, dtype=torch.float32)
    v8 = vb is not None
    vfix = (float(v_scale) if v_scale is not None else 0.0) if v8 else 1.0
    _lib.call(
        "fold_cache_write_prompt", k.data_ptr(), v.data_ptr(), int(k.dtype == torch.float16),
        meta.data_ptr(), nc, len(lens), page_table.data_ptr(), page_table.shape[1],
        int(page_size), HKV, D, ka.data_ptr(), kb.data_ptr(), va.data_ptr(), _lib.ptr(vb),
        ek.data_ptr(), vsum.data_ptr(), vmean.data_ptr(), scratch.data_ptr(),
        float(v_headroom), vfix, _lib.stream(dev),
    )
    return scratch[-1:]


def step(
    q, k, v, qa, qb, eq, ek, page_table, page_size, lens, ka, kb, va, vb, v_scale, vsum, vmean,
    lens_out,
):
    """One step's writes: Q's planes (`q` `(B*H, D)`), and/or one token per
    request appended at `lens` (`k`, `v` `(B, H_KV, D)`), `lens_out = lens + 1`."""
    x = q if q is not None else k
    # one kernel reads all three as the same 16-bit type: anything else would be read as garbage
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t is None:
            continue
        if t.dtype not in (torch.bfloat16, torch.float16) or t.dtype != x.dtype:
            raise ValueError(f"q, k and v must be bf16 or fp16, and the same type ({name} is {t.dtype}, "
                             f"{'q' if q is not None else 'k'} is {x.dtype})")
        if t.device != lens.device:
            raise ValueError(f"{name} is on {t.device}, the cache on {lens.device}")
    B = lens.shape[0]
    D = x.shape[-1]
    HKV = k.shape[1] if k is not None else vsum.shape[0] // B
    heads = q.shape[0] // B if q is not None else HKV
    if q is not None:
        q = q.contiguous()
    if k is not None:
        k, v = k.contiguous(), v.contiguous()
    _lib.call(
        "fold_step_append", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), int(x.dtype == torch.float16),
        B, heads, HKV, D, page_table.data_ptr(), page_table.shape[1], int(page_size),
        lens.data_ptr(), lens_out.data_ptr(), _lib.ptr(qa), _lib.ptr(qb), _lib.ptr(eq),
        ka.data_ptr(), kb.data_ptr(), va.data_ptr(), _lib.ptr(vb), ek.data_ptr(), float(v_scale),
        vsum.data_ptr(), vmean.data_ptr(), _lib.stream(x.device),
    )


def tail_append(v, tail, ka, ek, page_table, page_size, lens, back):
    """The tail's share of an append, after `step` on the same stream: the token
    of each request (at `lens - back`) joins its 64-key block's sums and row
    (`tail` a `TailState`; reference: decode/write.py:193-300, `append_row`)."""
    if v.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"v must be bf16 or fp16 (it is {v.dtype})")
    B, HKV, D = v.shape
    v = v.contiguous()
    _lib.call(
        "fold_tail_append", v.data_ptr(), int(v.dtype == torch.float16), B, HKV, D, page_table.data_ptr(),
        page_table.shape[1], int(page_size), lens.data_ptr(), int(back), ka.data_ptr(), ek.data_ptr(),
        _lib.ptr(tail.u), _lib.ptr(tail.vr), tail.vsum.data_ptr(), _lib.ptr(tail.ysum), tail.rows.data_ptr(),
        tail.rank, _lib.stream(v.device),
    )
