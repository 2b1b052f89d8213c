"""The device status word reaches the host as an exception.

Every wait inside the tcgen05 kernels is bounded: when one runs out the kernel raises a status
word and returns. Nothing here makes a real kernel time out (and nothing faults): the library's
`fold_wait_probe` runs that same wait on a barrier nobody arrives at, with a limit of about a
millisecond, and the host-side checks are exercised on the word it leaves and on words set by
hand."""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_raises_the_status_word_and_returns():
    from fold_attention_b200 import _lib
    from fold_attention_b200.backward import launch  # noqa: F401  (registers the signature)
    from fold_attention_b200.utils import check_status

    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    torch.cuda.synchronize()
    t0 = time.time()
    _lib.call("fold_wait_probe", 2_000_000, status.data_ptr(), flag.data_ptr(), _lib.stream(status.device))
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert int(status) == 3           # FOLD_ERR_TIMEOUT
    assert int(flag) == 1             # the CTA-wide flag that makes every other role stop waiting
    assert dt < 1.0                   # ~1 ms of SM clocks, not the production limit of about a second
    with pytest.raises(_lib.FoldLibraryError, match="wait ran out"):
        check_status(status, "probe")
    # the context is intact: the next kernel runs
    x = torch.arange(8, device="cuda").sum()
    assert int(x) == 28
    with pytest.raises(ValueError, match="limit"):
        _lib.call("fold_wait_probe", 0, status.data_ptr(), None, _lib.stream(status.device))


def test_prepared_launches_check_and_clear_their_status():
    from fold_attention_b200 import FoldKVCache, _lib
    from fold_attention_b200.backward import attention_forward, prepare_backward

    torch.manual_seed(3)
    B, S, H, HKV, D = 1, 256, 4, 2, 128
    q, do = (torch.randn(B, S, H, D, device="cuda").bfloat16() for _ in range(2))
    k, v = (torch.randn(B, S, HKV, D, device="cuda").bfloat16() for _ in range(2))
    attention_forward.check_status = True
    try:
        o, lse = attention_forward(q, k, v, causal=True)
    finally:
        attention_forward.check_status = False
    tr = lambda x: x.transpose(1, 2)  # noqa: E731
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True)
    run()
    run.check()                        # a clean run: nothing raised
    run.status.fill_(3)                # what a kernel that gave up a wait would leave
    with pytest.raises(_lib.FoldLibraryError, match="BackwardLaunch.*wait ran out"):
        run.check()
    run()                              # the next call's preprocess clears the word in-stream
    run.check()

    c = FoldKVCache(2, H, HKV, D, 512, page_size=128, depth=16.0, v8=True)
    cu = torch.tensor([0, 300, 377], device="cuda", dtype=torch.int32)
    c.write_prompt(torch.randn(377, HKV, D, device="cuda").bfloat16(), torch.randn(377, HKV, D, device="cuda").bfloat16(), cu, [300, 77])
    c.check_status = True
    qd = torch.randn(2, H, D, device="cuda").bfloat16()
    out = c.attend(qd)
    launch = next(iter(c._launches.values()))
    launch.status.fill_(3)
    with pytest.raises(_lib.FoldLibraryError, match="DecodeLaunch"):
        c.attend(qd)
    launch.clear_status()
    assert torch.equal(c.attend(qd), out)


def test_the_public_training_call_checks_when_asked():
    import fold_attention_b200 as fa
    from fold_attention_b200 import interface

    torch.manual_seed(4)
    q, k, v = (torch.randn(1, 256, 2, 128, device="cuda").bfloat16().requires_grad_() for _ in range(3))
    interface.check_status = True
    try:
        fa.fold_attn_func(q, k, v, causal=True).backward(torch.ones(1, 256, 2, 128, device="cuda").bfloat16())
    finally:
        interface.check_status = False
    assert q.grad is not None and bool(torch.isfinite(q.grad.float()).all())
