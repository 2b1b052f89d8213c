"""Host-side helpers shared by the backward and the decode."""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass

import torch

# Every decode weight is exp2(s - Z), so Q is scaled by LOG2E / sqrt(D) before
# it is quantised (reference: src/fold_attention/utils.py:13-15).
LOG2E = 1.4426950408889634


@dataclass(eq=False)
class Launch:
    """A prepared launch: calling it calls `run`. Kernels take the bound
    tensors by address, so `held` keeps them alive as long as the launch
    (reference: src/fold_attention/utils.py:21-30)."""

    run: Callable
    held: tuple = ()

    def __call__(self, *args, **kwargs):
        return self.run(*args, **kwargs)


def require_sm100(device):
    """The kernels are built for sm_100a only (the reference gates on SM90,
    src/fold_attention/interface.py:35-36)."""
    major, _ = torch.cuda.get_device_capability(device)
    if major != 10:
        raise ValueError("fold_attention_b200 requires an SM100 (B200) GPU")
