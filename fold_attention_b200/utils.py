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

    def check(self):
        """Read the launch's device status word (this waits for the device) and
        raise if a kernel of the last call gave up a bounded wait or refused
        its arguments: its outputs are then incomplete. The word stays raised
        until `clear_status`."""
        check_status(getattr(self, "status", None), type(self).__name__)

    def clear_status(self):
        status = getattr(self, "status", None)
        if status is not None:
            status.zero_()


_STATUS_TEXT = {
    1: "a kernel refused its arguments (status 1)",
    2: "a kernel could not lay out its shared memory (status 2)",
    3: "a device-side wait ran out: a kernel returned early and its outputs are incomplete (status 3)",
}


def check_status(status, what):
    """Raise `FoldLibraryError` if the int32 device status word is non-zero."""
    if status is None:
        return
    code = int(status.item())
    if code:
        from ._lib import FoldLibraryError

        raise FoldLibraryError(f"{what}: {_STATUS_TEXT.get(code, f'status {code}')}")


def require_sm100(device):
    """The kernels are built for sm_100a only (the reference gates on SM90,
    src/fold_attention/interface.py:35-36)."""
    major, _ = torch.cuda.get_device_capability(device)
    if major != 10:
        raise ValueError("fold_attention_b200 requires an SM100 (B200) GPU")
