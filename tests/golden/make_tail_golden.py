"""Generate tests/golden/tail_model.npz from the reference's own `tail_model`.

    python tests/golden/make_tail_golden.py /path/to/reference

`src/fold_attention/decode/cache.py` is pure torch and is imported by file path
(as `make_cache_golden.py` does). Seeded keys with a low-rank K -> V relation
plus noise go through the reference's `quantize_k` and `tail_model` on the CPU;
the file stores plane A (swizzled, as the cache holds it), the key scales, V,
and the model's `vblk`, `u`, `vr` at ranks 0 and 16.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from make_cache_golden import load_reference  # noqa: E402


def main(root):
    c = load_reference(root)
    out = {}
    g = torch.Generator().manual_seed(2025)
    for tag, (N, S, D) in dict(d64=(2, 200, 64), d128=(2, 330, 128)).items():
        k = torch.randn(N, S, D, generator=g)
        a = torch.randn(N, D, 6, generator=g) / D ** 0.5
        b = torch.randn(N, 6, D, generator=g)
        blk = torch.randn(N, -(-S // 64), D, generator=g).repeat_interleave(64, 1)[:, :S]
        v = (blk + k @ a @ b + 0.3 * torch.randn(N, S, D, generator=g)).bfloat16()
        ka, _kb, ek = c.quantize_k(k.bfloat16())
        out[f"{tag}_ka"] = ka.numpy()
        out[f"{tag}_ek"] = ek.float().numpy()
        out[f"{tag}_v"] = v.float().numpy()
        for rank in (0, 16):
            t = c.tail_model(ka, ek, v, rank=rank)
            out[f"{tag}_r{rank}_vblk"] = t.vblk.float().numpy()
            if rank:
                out[f"{tag}_r{rank}_u"] = t.u.numpy()
                out[f"{tag}_r{rank}_vr"] = t.vr.numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tail_model.npz")
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
