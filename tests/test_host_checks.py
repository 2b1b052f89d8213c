"""Host-side argument checks that need no GPU: they raise before any launch."""

import pytest
import torch


def _step_args(q, k, v):
    from fold_attention_b200.decode import write

    B, H, HKV, D = 2, 4, 2, 64
    z8 = torch.zeros(8, D, dtype=torch.int8)
    lens = torch.zeros(B, dtype=torch.int32)
    return write.step, (q, k, v, z8, z8, torch.zeros(8), torch.zeros(8, dtype=torch.bfloat16),
                        torch.zeros(B, 1, dtype=torch.int32), 64, lens, z8, z8, z8, None, 1.0,
                        torch.zeros(B * HKV, D), torch.zeros(B * HKV, D), lens)


@pytest.mark.parametrize("qd,kd,vd", [
    (torch.float32, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.float16, torch.float16),
    (torch.float16, torch.float16, torch.bfloat16),
    (None, torch.float32, torch.float32),
])
def test_a_step_refuses_mixed_or_wide_dtypes(qd, kd, vd):
    """The step kernel reads q, k and v as one 16-bit type (the reference binds its step per
    dtype, src/fold_attention/decode/write.py:565-673): anything else is refused on the host."""
    B, H, HKV, D = 2, 4, 2, 64
    q = None if qd is None else torch.zeros(B * H, D, dtype=qd)
    k, v = torch.zeros(B, HKV, D, dtype=kd), torch.zeros(B, HKV, D, dtype=vd)
    step, args = _step_args(q, k, v)
    with pytest.raises(ValueError, match="must be bf16 or fp16"):
        step(*args)


def test_status_text():
    from fold_attention_b200 import _lib
    from fold_attention_b200.utils import check_status

    check_status(None, "x")
    check_status(torch.zeros(1, dtype=torch.int32), "x")
    with pytest.raises(_lib.FoldLibraryError, match="x: a device-side wait ran out"):
        check_status(torch.tensor([3], dtype=torch.int32), "x")
    with pytest.raises(_lib.FoldLibraryError, match="refused its arguments"):
        check_status(torch.tensor([1], dtype=torch.int32), "x")


def test_the_forward_and_backward_refuse_tensors_that_do_not_match_q():
    """The kernels index k, v, o, do and lse by q's sizes, so a mismatch is refused on the host
    (CPU tensors here: the checks come before any launch)."""
    from fold_attention_b200.backward.launch import attention_forward, prepare_backward

    B, S, H, HKV, D = 2, 16, 4, 2, 64
    q = torch.zeros(B, S, H, D, dtype=torch.bfloat16)
    k = torch.zeros(B, S, HKV, D, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="do not match q"):
        attention_forward(q, k[:, :8], k[:, :8], causal=True)          # a shorter k: would be read past its end
    with pytest.raises(ValueError, match="do not match q"):
        attention_forward(q.transpose(1, 2), k, k, causal=True)        # (B, H, S, D) passed where (B, S, H, D) goes
    with pytest.raises(ValueError, match="H_KV heads"):
        attention_forward(q, k, k[:, :, :1], causal=True)
    with pytest.raises(ValueError, match="same type"):
        attention_forward(q, k.half(), k.half(), causal=True)
    with pytest.raises(ValueError, match="contiguous head dim"):
        attention_forward(q.transpose(-1, -2).contiguous().transpose(-1, -2), k, k, causal=True)
    with pytest.raises(ValueError, match="int32"):
        attention_forward(q[0], k[0], k[0], causal=True, cu_seqlens=torch.tensor([0, 16]), max_seqlen=16)

    qb, kb = q.transpose(1, 2), k.transpose(1, 2)                      # the backward's (B, H, S, D) views
    lse = torch.zeros(B, H, S)
    with pytest.raises(ValueError, match="do not match q"):
        prepare_backward(qb, kb[:1], kb[:1], qb, qb, lse, causal=True)
    with pytest.raises(ValueError, match="o and do are q's shape"):
        prepare_backward(qb, kb, kb, qb[:, :2], qb, lse, causal=True)
    with pytest.raises(ValueError, match=r"lse is \(B, H, S\)"):
        prepare_backward(qb, kb, kb, qb, qb, lse[:, :, :8], causal=True)
    with pytest.raises(ValueError, match="same 16-bit type"):
        prepare_backward(qb, kb, kb, qb.half(), qb, lse, causal=True)
    with pytest.raises(NotImplementedError, match="self-attention"):
        prepare_backward(qb, kb[:, :, :8], kb[:, :, :8], qb, qb, lse, causal=True)


def test_a_decode_launch_binds_on_the_host_for_every_layout():
    """`prepare_fold_decode` validates and binds without touching the GPU: every layout it takes
    builds a launch from CPU tensors (nothing is run), and the mismatches are refused."""
    from fold_attention_b200.decode.launch import prepare_fold_decode

    def planes(NBH, G, D=128):
        return (torch.zeros(NBH, G, D, dtype=torch.int8), torch.zeros(NBH, G, D, dtype=torch.int8), torch.ones(NBH, G),
                torch.zeros(1024, D, dtype=torch.int8), torch.zeros(1024, D, dtype=torch.int8), torch.zeros(1024, dtype=torch.bfloat16),
                torch.zeros(1024, D, dtype=torch.bfloat16), torch.zeros(NBH, G), torch.full((NBH, G), 8.0))

    kw = dict(page_table=torch.zeros(2, 4, dtype=torch.int32), page_size=64, seq_lens=torch.zeros(2, dtype=torch.int32), n_kv_heads=2)
    assert prepare_fold_decode(*planes(4, 8), truncate=True, vmean=torch.zeros(4, 128), **kw).kernel in ("mma", "sm100")
    assert prepare_fold_decode(*planes(4, 8), truncate=True, vmean=torch.zeros(4, 128), draft_len=4, causal=True, **kw).tree.shape == (4, 8)
    assert prepare_fold_decode(*planes(4, 8), truncate=True, vmean=torch.zeros(4, 8, 128), **kw).kernel == "mma"
    assert prepare_fold_decode(*planes(4, 8), truncate=True, vmean=torch.zeros(4, 128), sound=True, **kw).kernel == "mma"
    assert prepare_fold_decode(*planes(4, 8), truncate=True, vmean=torch.zeros(4, 128), group_cut=False, **kw).kernel == "mma"
    assert prepare_fold_decode(*planes(4, 32), split=2, **kw).kernel == "mma"      # 16 groups of 8 on the warp-level kernel
    with pytest.raises(ValueError, match="one per query row"):
        prepare_fold_decode(*planes(4, 8), truncate=True, vmean=torch.zeros(4, 4, 128), **kw)
    with pytest.raises(NotImplementedError, match="16, 24 or 32"):
        prepare_fold_decode(*planes(4, 12), **kw)
    with pytest.raises(NotImplementedError, match="one group of at most 8"):
        prepare_fold_decode(*planes(4, 16), draft_len=2, causal=True, **kw)
    with pytest.raises(ValueError, match="names the 16 groups of 8"):
        prepare_fold_decode(*planes(4, 32), order=torch.arange(4, dtype=torch.int32), **kw)
