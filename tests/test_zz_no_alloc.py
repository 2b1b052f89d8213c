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
