"""Generate tests/golden/cache_format.npz from the reference's own torch code.

Run once in a container that has the reference checked out:

    python tests/golden/make_cache_golden.py /path/to/reference

It imports the reference's pure-torch cache quantisers by file path
(`src/fold_attention/decode/cache.py`, `src/fold_attention/utils.py`; no GPU
and no package import needed), feeds them seeded inputs and stores inputs and
outputs. The one deviation, needed because the reference's tests compare on a
GPU: the query scale is `amax * fp32(1/127)` (what CUDA torch and the device
quantiser evaluate for `amax / 127.0`, decode/quant.py:137), not the true
division CPU torch performs for cache.py:92.
"""

from __future__ import annotations

import importlib.util
import math
import os
import sys
import types

import numpy as np
import torch

LOG2E = 1.4426950408889634


def load_reference(root):
    src = os.path.join(root, "src", "fold_attention")

    def load(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        return m

    pkg = types.ModuleType("fold_attention")
    pkg.__path__ = [src]
    sys.modules["fold_attention"] = pkg
    sub = types.ModuleType("fold_attention.decode")
    sub.__path__ = [os.path.join(src, "decode")]
    sys.modules["fold_attention.decode"] = sub
    load("fold_attention.utils", os.path.join(src, "utils.py"))
    load("fold_attention.decode.config", os.path.join(src, "decode", "config.py"))
    return load("fold_attention.decode.cache", os.path.join(src, "decode", "cache.py"))


def main(root):
    c = load_reference(root)
    from fold_attention.utils import hadamard

    out = {}
    g = torch.Generator().manual_seed(1234)
    for D in (64, 128):
        for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16")):
            k = (torch.randn(96, D, generator=g) * 2).to(dt)
            k[5] = 0
            k[7, 3] = 40.0  # an outlier channel
            pa, pb, e = c.key_planes(k.float())
            out[f"key_{D}_{tag}_in"] = k.float().numpy()
            out[f"key_{D}_{tag}_pa"] = pa.numpy()
            out[f"key_{D}_{tag}_pb"] = pb.numpy()
            out[f"key_{D}_{tag}_e"] = e.numpy()
            out[f"had_{D}_{tag}"] = hadamard(k.float()).numpy()
            q = (torch.randn(40, D, generator=g) * 3).to(dt)
            q[3] = 0
            x = hadamard(q.float() * (LOG2E / math.sqrt(D)))
            eq = x.abs().amax(-1, keepdim=True).clamp_min(1e-30) * c.INV127
            qa, qb = c._int8_planes(x, eq)
            out[f"q_{D}_{tag}_in"] = q.float().numpy()
            out[f"q_{D}_{tag}_pa"] = qa.numpy()
            out[f"q_{D}_{tag}_pb"] = qb.numpy()
            out[f"q_{D}_{tag}_e"] = eq.squeeze(-1).numpy()

    # every e4m3 value, every midpoint between neighbours, both zeros
    # (tests/test_write.py:207-239), at scale 0.5 and through bf16 as there
    allv = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    allv = allv[torch.isfinite(allv)].unique()
    vals = torch.cat([allv, (allv[1:] + allv[:-1]) / 2, torch.tensor([-0.0, 0.0])])
    v = (vals * 0.5).bfloat16().float()
    pa, pb = c._e4m3_planes(v, 0.5)
    out["e4m3_in"] = v.numpy()
    out["e4m3_pa"] = pa.view(torch.uint8).numpy()
    out["e4m3_pb"] = pb.view(torch.uint8).numpy()
    v2 = (torch.randn(64, 128, generator=g) * 1.3 + 1).bfloat16().float()
    v2[3, 7] = 60.0
    pa, pb = c._e4m3_planes(v2, 0.25)
    out["e4m3r_in"] = v2.numpy()
    out["e4m3r_pa"] = pa.view(torch.uint8).numpy()
    out["e4m3r_pb"] = pb.view(torch.uint8).numpy()
    qa, qb, ev = c.quantize_v(v2)
    out["e4m3r_ev"] = np.float32(ev)

    # a paged append (cache.py:340-367; tests/test_write.py:93-135)
    for v8 in (False, True):
        B, HKV, D, PS, ppr = 6, 4, 128, 64, 8
        rows = B * ppr * HKV * PS
        k = (torch.randn(B, HKV, D, generator=g) * 2).bfloat16()
        vv = (torch.randn(B, HKV, D, generator=g) + 1).bfloat16()
        lens = torch.randint(1, ppr * PS - 1, (B,), generator=g)
        pt = torch.randperm(B * ppr, generator=g).int().view(B, ppr)
        ka = torch.zeros(rows, D, dtype=torch.int8)
        kb = torch.zeros_like(ka)
        ek = torch.zeros(rows, dtype=torch.bfloat16)
        if v8:
            va = torch.zeros(rows, D, dtype=torch.float8_e4m3fn)
            vb = torch.zeros_like(va)
        else:
            va, vb = torch.zeros(rows, D, dtype=torch.bfloat16), None
        ev = 0.25 if v8 else 1.0
        if v8:
            c.write_kv(ka, kb, ek, va, vb, k, vv, ev, pt, lens, PS, HKV)
        else:
            pos = lens
            row = (pt[torch.arange(B), pos // PS].long()[:, None] * HKV + torch.arange(HKV)) * PS
            row = row + (pos % PS)[:, None]
            c.write_rows(ka, kb, ek, va, None, k, vv, ev, row, pos % PS)
        t = "v8" if v8 else "bf"
        nz = ka.abs().sum(-1).nonzero().flatten()
        out[f"app_{t}_k"] = k.float().numpy()
        out[f"app_{t}_v"] = vv.float().numpy()
        out[f"app_{t}_lens"] = lens.int().numpy()
        out[f"app_{t}_pt"] = pt.numpy()
        out[f"app_{t}_rows"] = nz.numpy()
        out[f"app_{t}_ka"] = ka[nz].numpy()
        out[f"app_{t}_kb"] = kb[nz].numpy()
        out[f"app_{t}_ek"] = ek[nz].float().numpy()
        out[f"app_{t}_va"] = va[nz].view(torch.uint8).numpy() if v8 else va[nz].float().numpy()
        if v8:
            out[f"app_{t}_vb"] = vb[nz].view(torch.uint8).numpy()

    # a prompt written through write_rows (tests/test_write.py:242-290), D=64
    lens, H, PS, D, ppr = [300, 1, 256, 77], 2, 64, 64, 8
    N, B = sum(lens), len(lens)
    k = (torch.randn(N, H, D, generator=g) * 3).bfloat16()
    vv = (torch.randn(N, H, D, generator=g) + 1).bfloat16()
    pt = torch.randperm(B * ppr, generator=g).int().view(B, ppr)
    rows = B * ppr * H * PS
    ka = torch.zeros(rows, D, dtype=torch.int8)
    kb = torch.zeros_like(ka)
    ek = torch.zeros(rows, dtype=torch.bfloat16)
    va = torch.zeros(rows, D, dtype=torch.float8_e4m3fn)
    vb = torch.zeros_like(va)
    evs = 2.0 ** math.ceil(math.log2(float(vv.abs().amax()) * 2.0 / 448.0))
    req = torch.repeat_interleave(torch.arange(B), torch.tensor(lens))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)))
    pos = torch.arange(N) - cu[req]
    row = (pt[req, pos // PS].long()[:, None] * H + torch.arange(H)) * PS + (pos % PS)[:, None]
    c.write_rows(ka, kb, ek, va, vb, k, vv, evs, row, pos % PS)
    out["pr_k"], out["pr_v"] = k.float().numpy(), vv.float().numpy()
    out["pr_lens"], out["pr_pt"] = np.array(lens, np.int32), pt.numpy()
    out["pr_evs"] = np.float32(evs)
    out["pr_ka"], out["pr_kb"] = ka.numpy(), kb.numpy()
    out["pr_ek"] = ek.float().numpy()
    out["pr_va"], out["pr_vb"] = va.view(torch.uint8).numpy(), vb.view(torch.uint8).numpy()

    # swizzle_rows (cache.py:53-69)
    x = torch.randint(-128, 128, (2, 40, 128), generator=g).to(torch.int8)
    out["swz_in"] = x.numpy()
    out["swz_out"] = c.swizzle_rows(x).numpy()
    x = torch.randint(-128, 128, (1, 24, 64), generator=g).to(torch.int8)
    out["swz64_in"] = x.numpy()
    out["swz64_out"] = c.swizzle_rows(x).numpy()

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cache_format.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
