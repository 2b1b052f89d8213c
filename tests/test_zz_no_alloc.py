"""The decode entry point that allocates nothing (`fold_decode_run_static`):
its split partials live in a fixed array inside the library, for hosts that
may not allocate device memory while a step runs. Called through the C ABI on
the same inputs as the allocating entry point, twice in a row (the array
keeps the previous call's contents), its outputs must be the same bits.
Collected last so a failure here cannot hide another test's."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(v8, depth, seed):
    import fold_attention_b200 as fa

    lens = [1500, 700, 64, 2049]
    B, H, HKV, D, PS = len(lens), 16, 2, 128, 64
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = sum(lens)
    k = torch.randn(T, HKV, D, device="cuda", generator=g).bfloat16()
    v = (torch.randn(T, HKV, D, device="cuda", generator=g) + 0.4).bfloat16()
    q = torch.randn(B, H, D, device="cuda", generator=g).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    c = fa.FoldKVCache(B, H, HKV, D, max(lens) + 8, page_size=PS, v8=v8, depth=depth)
    c.page_table.copy_(torch.randperm(c.page_table.numel(), device="cuda", generator=g).int().view_as(c.page_table))
    c.write_prompt(k, v, cu, lens)
    c.attend(q)  # Q planes and the reference Z
    return c, lens


@pytest.mark.parametrize("v8,depth,split,chunk", [(True, 16.0, 3, 0), (False, None, 1, 0), (True, 12.0, 0, 512)])
def test_the_static_scratch_entry_point_is_the_allocating_ones_bits(v8, depth, split, chunk):
    from fold_attention_b200.decode.launch import prepare_fold_decode
    from fold_attention_b200.decode.static_scratch import SCRATCH_BYTES, decode_static, scratch_needed

    c, lens = _case(v8, depth, seed=17)
    sp = split if not chunk else -(-max(lens) // chunk)
    kw = dict(split=sp, truncate=depth is not None, refine_k=10.0, refine_v=10.0, v2=c.vb,
              v_scale=c.v_scale, vmean=c.vmean, page_table=c.page_table, page_size=c.page_size,
              seq_lens=c.seq_lens, n_kv_heads=c.n_kv_heads, weight_terms=2, chunk_keys=chunk)
    want = [x.clone() for x in prepare_fold_decode(
        c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, v8=v8, **kw)()]
    NBH, G, D = c.qa.shape
    assert scratch_needed(NBH, G, D, sp) <= SCRATCH_BYTES
    for _ in range(2):  # the second call finds the first call's partials in the array
        out = torch.full((NBH, G, D), float("nan"), device="cuda")
        den = torch.full((NBH, G), float("nan"), device="cuda")
        counts = torch.full((NBH, 2), -1, device="cuda", dtype=torch.int32)
        status = torch.zeros(1, device="cuda", dtype=torch.int32)
        decode_static(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, out, den, counts, status, **kw)
        torch.cuda.synchronize()
        assert int(status) == 0
        assert torch.equal(out, want[0]) and torch.equal(den, want[1]) and torch.equal(counts, want[2])


def test_a_call_too_large_for_the_array_is_refused():
    from fold_attention_b200.decode.static_scratch import SCRATCH_BYTES, decode_static, scratch_needed

    c, lens = _case(True, 16.0, seed=18)
    NBH, G, D = c.qa.shape
    split = 4096
    assert scratch_needed(NBH, G, D, split) > SCRATCH_BYTES
    out = torch.empty((NBH, G, D), device="cuda")
    den = torch.empty((NBH, G), device="cuda")
    counts = torch.empty((NBH, 2), device="cuda", dtype=torch.int32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    with pytest.raises(ValueError, match="built-in scratch holds"):
        decode_static(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, out, den, counts, status,
                      split=split, truncate=True, refine_k=10.0, refine_v=10.0, v2=c.vb, v_scale=c.v_scale,
                      vmean=c.vmean, page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens,
                      n_kv_heads=c.n_kv_heads, weight_terms=2)


def _outputs(NBH, G, D):
    out = torch.full((NBH, G, D), float("nan"), device="cuda")
    den = torch.full((NBH, G), float("nan"), device="cuda")
    counts = torch.full((NBH, 2), -1, device="cuda", dtype=torch.int32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    return out, den, counts, status


def test_a_permuted_order_gives_the_allocating_entry_points_bits():
    """`order` maps grid slots to row groups (longest first, say). The built-in array is laid out
    for exactly the call's row groups, so a permutation of all of them is what this entry takes."""
    from fold_attention_b200.decode.launch import prepare_fold_decode
    from fold_attention_b200.decode.static_scratch import decode_static

    c, lens = _case(True, 16.0, seed=19)
    NBH, G, D = c.qa.shape
    g = torch.Generator(device="cuda").manual_seed(3)
    order = torch.randperm(NBH, device="cuda", generator=g).int()
    kw = dict(split=3, truncate=True, refine_k=10.0, refine_v=10.0, v2=c.vb, v_scale=c.v_scale, vmean=c.vmean,
              page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=c.n_kv_heads,
              weight_terms=2, order=order)
    want = [x.clone() for x in prepare_fold_decode(
        c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, v8=True, **kw)()]
    for _ in range(2):
        out, den, counts, status = _outputs(NBH, G, D)
        decode_static(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, out, den, counts, status, **kw)
        torch.cuda.synchronize()
        assert int(status) == 0
        assert torch.equal(out, want[0]) and torch.equal(den, want[1]) and torch.equal(counts, want[2])


def test_an_order_that_leaves_the_array_is_refused_on_the_device():
    """A slot mapped to a row group the array has no room for must not write anywhere: the CTA
    raises the status word (FOLD_ERR_ARGUMENT = 1) and returns; the call itself returns normally."""
    from fold_attention_b200.decode.static_scratch import decode_static

    c, lens = _case(True, 16.0, seed=20)
    NBH, G, D = c.qa.shape
    order = torch.arange(NBH, device="cuda", dtype=torch.int32)
    order[1] = NBH + 5
    out, den, counts, status = _outputs(NBH, G, D)
    decode_static(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, out, den, counts, status,
                  split=3, truncate=True, refine_k=10.0, refine_v=10.0, v2=c.vb, v_scale=c.v_scale, vmean=c.vmean,
                  page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=c.n_kv_heads,
                  weight_terms=2, order=order)
    torch.cuda.synchronize()
    assert int(status) == 1
    # the next, well-formed call is unaffected
    out, den, counts, status = _outputs(NBH, G, D)
    decode_static(c.qa, c.qb, c.eq, c.ka, c.kb, c.ek, c.va, c.z, c.cut, out, den, counts, status,
                  split=3, truncate=True, refine_k=10.0, refine_v=10.0, v2=c.vb, v_scale=c.v_scale, vmean=c.vmean,
                  page_table=c.page_table, page_size=c.page_size, seq_lens=c.seq_lens, n_kv_heads=c.n_kv_heads,
                  weight_terms=2)
    torch.cuda.synchronize()
    assert int(status) == 0 and bool(torch.isfinite(out).all())


def test_a_call_without_outputs_is_refused():
    """The partials never leave the library, so a call that asks for partials only (out NULL, which
    the allocating entry point allows) is an argument error here."""
    import ctypes

    from fold_attention_b200 import _lib
    from fold_attention_b200.decode import static_scratch  # noqa: F401  (registers the signature)

    c, lens = _case(False, None, seed=21)
    NBH, G, D = c.qa.shape
    _, den, counts, status = _outputs(NBH, G, D)
    rc = _lib.lib.fold_decode_run_static(
        c.qa.data_ptr(), c.qb.data_ptr(), c.eq.data_ptr(), c.ka.data_ptr(), c.kb.data_ptr(), c.ek.data_ptr(),
        c.va.data_ptr(), None, None, c.z.data_ptr(), c.cut.data_ptr(), c.page_table.data_ptr(),
        c.seq_lens.data_ptr(), None, NBH, G, c.n_kv_heads, D, c.page_table.shape[1], c.page_size, 2, 0, 0, 2,
        ctypes.c_float(10.0), ctypes.c_float(10.0), None, ctypes.c_float(1.0), None, 0, den.data_ptr(),
        counts.data_ptr(), status.data_ptr(), _lib.stream(c.qa.device))
    assert rc == 1
    assert b"out, den and counts must be given" in _lib.lib.fold_last_error()
