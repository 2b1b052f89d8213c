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
