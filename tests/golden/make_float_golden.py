"""Generate tests/golden/float_models.npz from the reference's own float models.

    python tests/golden/make_float_golden.py /path/to/reference

The oracle's float64 / fp32 models (`oracle/decode.py`, `oracle/backward.py`) restate functions
that, in the reference, live in its benchmark harness and its test files. This script runs the
reference's own text of those functions on the CPU, on seeded inputs, and stores inputs and
outputs, so `tests/test_oracle_float_models.py` can hold the oracle to them:

* `benchmarks/harness/training.py`: `reference_grads` (FP32 gradients per request and head);
* `tests/test_decode.py`: `_fma`, `_coarse` (the coarse logit, one fused multiply-add under a
  given reference), `_mass_model` (the mass reference's estimate), `_ref` (truncated softmax) and
  `_s16` (the four-term logit liveness is defined on).

The two source files import GPU-only packages at module level, so the functions are taken out
of the files' text (by name, with `ast`) and compiled beside the reference's pure-torch cache
module, which is imported by file path as `make_cache_golden.py` does.
"""

from __future__ import annotations

import ast
import dataclasses
import itertools
import math
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from make_cache_golden import load_reference  # noqa: E402


def functions_of(path, names, env):
    """Compile the named top-level functions of `path` into `env`."""
    tree = ast.parse(open(path).read())
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in keep} == set(names), (path, names)
    code = compile(ast.Module(body=keep, type_ignores=[]), path, "exec")
    exec(code, env)
    return env


@dataclasses.dataclass
class Inputs:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    o: torch.Tensor
    do: torch.Tensor
    lse: torch.Tensor
    causal: bool
    scale: float
    lens: list
    cu: torch.Tensor | None = None

    @property
    def varlen(self):
        return self.cu is not None


def main(root):
    c = load_reference(root)
    out = {}
    # ---- training: FP32 gradients ----
    env = dict(torch=torch, itertools=itertools, math=math, Inputs=Inputs)
    functions_of(os.path.join(root, "benchmarks", "harness", "training.py"), ["_segments", "reference_grads"], env)
    g = torch.Generator().manual_seed(77)
    for tag, (B, S, H, HKV, D, causal) in dict(mha=(2, 96, 2, 2, 32, True), gqa=(1, 130, 4, 2, 64, True),
                                                full=(1, 64, 4, 1, 32, False)).items():
        q = (torch.randn(B, S, H, D, generator=g) / D**0.5).bfloat16()
        k, v = (torch.randn(B, S, HKV, D, generator=g).bfloat16() for _ in range(2))
        do = torch.randn(B, S, H, D, generator=g).bfloat16()
        inp = Inputs(q, k, v, None, do, None, causal, 1.0 / math.sqrt(D), [S] * B)
        dq, dk, dv = env["reference_grads"](inp)
        for n, t in dict(q=q, k=k, v=v, do=do, dq=dq, dk=dk, dv=dv).items():
            out[f"train_{tag}_{n}"] = t.float().numpy()
        out[f"train_{tag}_causal"] = np.array(int(causal))
    # packed: two sequences in one call
    lens = [70, 33]
    T, H, HKV, D = sum(lens), 4, 2, 32
    q = (torch.randn(T, H, D, generator=g) / D**0.5).bfloat16()
    k, v = (torch.randn(T, HKV, D, generator=g).bfloat16() for _ in range(2))
    do = torch.randn(T, H, D, generator=g).bfloat16()
    inp = Inputs(q, k, v, None, do, None, True, 1.0 / math.sqrt(D), lens, torch.tensor([0, 70, 103]))
    dq, dk, dv = env["reference_grads"](inp)
    for n, t in dict(q=q, k=k, v=v, do=do, dq=dq, dk=dk, dv=dv).items():
        out[f"train_packed_{n}"] = t.float().numpy()
    out["train_packed_lens"] = np.array(lens)

    # ---- decode: the test file's float models ----
    env = dict(torch=torch, math=math, KBR=c.KBR, swizzle_rows=c.swizzle_rows, quantize_kq=c.quantize_kq,
               key_planes=c.key_planes)
    functions_of(os.path.join(root, "tests", "test_decode.py"), ["_fma", "_coarse", "_mass_model", "_ref", "_s16"], env)
    LOG2E = 1.4426950408889634
    for tag, (NBH, S, G, D) in dict(a=(2, 400, 8, 128), b=(1, 300, 4, 64), c=(2, 64, 1, 128)).items():
        qs = torch.randn(NBH, G, D, generator=g) * (LOG2E / math.sqrt(D)) * 3.0
        k = torch.randn(NBH, S, D, generator=g)
        k[:, ::97] *= 6.0
        v = torch.randn(NBH, S, 16, generator=g)   # the truncated softmax's values: 16 channels are enough
        qq = c.quantize_kq(qs)       # CPU division for the scale: inputs and outputs both stored
        kk = c.quantize_k(k)         # swizzled planes, padded bf16 scales
        ek = kk[2][:, :S]
        z = torch.randn(NBH, G, generator=g) * 2 + 8
        sc = env["_coarse"](qq, (kk[0], kk[1], kk[2]), S)
        sz = env["_coarse"](qq, (kk[0], kk[1], kk[2]), S, z)
        mass = torch.stack([env["_mass_model"](sc[b], S) for b in range(NBH)])
        mass_short = torch.stack([env["_mass_model"](sc[b], min(S, 50)) for b in range(NBH)])
        s16 = env["_s16"](qs, k)
        cut = z - 6.0
        o, p = env["_ref"](s16.double(), z.double(), v.double(), cut.double())
        out.update({
            f"dec_{tag}_qa": qq[0].numpy(), f"dec_{tag}_qb": qq[1].numpy(), f"dec_{tag}_eq": qq[2].numpy(),
            f"dec_{tag}_ka_unswizzled": c.swizzle_rows(kk[0])[:, :S].numpy(), f"dec_{tag}_kb_unswizzled": c.swizzle_rows(kk[1])[:, :S].numpy(),
            f"dec_{tag}_ek": ek.float().numpy(), f"dec_{tag}_z": z.numpy(), f"dec_{tag}_v": v.numpy(),
            f"dec_{tag}_coarse": sc.numpy(), f"dec_{tag}_coarse_z": sz.numpy(), f"dec_{tag}_mass": mass.numpy(),
            f"dec_{tag}_mass50": mass_short.numpy(), f"dec_{tag}_s16": s16.numpy(), f"dec_{tag}_cut": cut.numpy(),
            f"dec_{tag}_ref_out": o.numpy(), f"dec_{tag}_ref_psum": p.sum(-1).numpy(),
        })
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "float_models.npz")
    np.savez_compressed(path, **out)
    print(path, len(out), "arrays", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
