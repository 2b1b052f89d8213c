"""Benchmark of the deterministic causal attention backward (and, as extra
keys, the paged decode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout. A step is one backward (preprocess, work list, main
loop, postprocess) over the headline configuration (config 2): batch 4, seqlen
8192, 32 query / 32 KV heads, head_dim 128, bf16, causal; inputs iid N(0,1)
with 1/sqrt(D) on q, O and LSE from the library's own forward, computed before
the timed region. At N > 1 every rank runs that workload on its own shard (weak
scaling; the path shards over batch x KV head with no collective on the data
path), and the extra keys add the same work sharded: config 2's (request, KV
head) units split over the ranks, and config 5's 256 requests partitioned by
length.

Timing: `value` is the mean of K steps inside one region bracketed by barriers
and synchronisation (the contract of this file); `extra.timing` repeats the
measurement the way the reference's harness does (CUDA-graph replays, 21 rounds
after dropped warm-ups, median: benchmarks/harness/timing.py:117-170) and over
a region of at least two seconds, each with the SM clock sampled while it ran.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import re
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

CFG = dict(B=4, S=8192, H=32, HKV=32, D=128)
WORKLOAD = "config2 causal det. backward B{B} S8192 H32/32 D128 bf16"
METRIC = "det. causal bwd TFLOP/s"
KERNELS_PER_STEP = 5   # preprocess, its finalize pass, work list, main loop, dQ postprocess


def flops(B, S, H, D):
    """5 GEMMs of the causal half: 5 * B * H * S^2 * D (FA convention)."""
    return 5.0 * B * H * S * S * D


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(bf16=d["bf16_tflops_sustained"], bf16_burst=d["bf16_tflops"], hbm=d["hbm_gbs"],
                    which="measured")
    return dict(bf16=1400.0, bf16_burst=1590.0, hbm=6650.0, which="fallback")


def profiled(name, key, default):
    """A number kept in a tracked ncu summary (`profiles/<name>`), written there as `key = value`."""
    try:
        text = open(os.path.join(ROOT, "profiles", name)).read()
        m = re.search(rf"^\s*{re.escape(key)}\s*=\s*([0-9.eE+-]+)", text, flags=re.M)
        return float(m.group(1)) if m else default
    except OSError:
        return default


class Clocks:
    """Sample SM clocks and throttle reasons with nvidia-smi while timing."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def window(self, t0, t1):
        rows = [r for ts, r in self.rows if t0 - 0.02 <= ts <= t1 + 0.05] or [r for _, r in self.rows[-3:]]
        if not rows:
            return None
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return dict(sm_mhz=mhz[len(mhz) // 2] if mhz else None,
                    sm_max_mhz=int(rows[0][1]) if rows[0][1].isdigit() else None,
                    reasons=reasons, samples=len(rows))

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return None
        time.sleep(0.1)
        self.proc.terminate()
        return self.window(t0, t1) if t0 is not None else None


def make_inputs(cfg, device, seed):
    B, S, H, HKV, D = (cfg[k] for k in ("B", "S", "H", "HKV", "D"))
    g = torch.Generator(device=device).manual_seed(seed)
    q = (torch.randn(B, S, H, D, device=device, generator=g) / D**0.5).bfloat16()
    k = torch.randn(B, S, HKV, D, device=device, generator=g).bfloat16()
    v = torch.randn(B, S, HKV, D, device=device, generator=g).bfloat16()
    do = torch.randn(B, S, H, D, device=device, generator=g).bfloat16()
    return q, k, v, do


def tr(x):
    return x.transpose(1, 2)


def prepare(cfg, device, seed, plan=None):
    from fold_attention_b200.backward import attention_forward, prepare_backward

    q, k, v, do = make_inputs(cfg, device, seed)
    o, lse = attention_forward(q, k, v, causal=True)
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True, plan=plan)
    return (q, k, v, o, do, lse, run)


def time_backward(state, steps, warmup, dist):
    """(ms per step, main-kernel ms per launch, host window): K steps in one region, the three
    phases of each between events on the launching stream."""
    run = state[-1]
    for _ in range(warmup):
        run()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    t0 = time.time()
    for i in range(steps):
        ev[i][0].record()
        run.run_phase(1)
        ev[i][1].record()
        run.run_phase(8 | 2)   # the work list, then the main loop
        ev[i][2].record()
        run.run_phase(4)
        ev[i][3].record()
    torch.cuda.synchronize()
    t1 = time.time()
    if dist is not None:
        dist.barrier()
    total = ev[0][0].elapsed_time(ev[-1][3]) / steps
    main = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    return total, main, (t0, t1)


def time_protocols(state, device, clocks, ms_hint):
    """The same step the way the reference's harness times a kernel, and over a long region.

    graph: the whole step captured once in a CUDA graph; 3 dropped warm-up replays, then 21
    replays each between its own events; median. long: back-to-back steps for at least two
    seconds of device time (where the SM clock settles under the power limit). Each carries the
    SM clock sampled while it ran and TFLOP/s per GHz, so burst and sustained read off one line."""
    run = state[-1]
    fl = flops(CFG["B"], CFG["S"], CFG["H"], CFG["D"])
    out = {}
    side = torch.cuda.Stream(device)
    g = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            run()
    torch.cuda.synchronize()
    for _ in range(3):
        g.replay()
    rounds = 21
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(rounds)]
    torch.cuda.synchronize()
    t0 = time.time()
    for a, b in ev:
        a.record()
        g.replay()
        b.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = sorted(a.elapsed_time(b) for a, b in ev)
    med = ms[rounds // 2]
    ck = clocks.window(t0, t1) or {}
    out["graph_median"] = dict(ms_per_step=med, tflops=fl / med / 1e9, rounds=rounds, dropped=3, min_ms=ms[0], max_ms=ms[-1],
                               sm_mhz=ck.get("sm_mhz"), tflops_per_ghz=(fl / med / 1e9) / (ck["sm_mhz"] / 1e3) if ck.get("sm_mhz") else None)
    n = max(8, int(math.ceil(2200.0 / max(ms_hint, 1e-3))))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.time()
    e0.record()
    for _ in range(n):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    msl = e0.elapsed_time(e1) / n
    ck = clocks.window(t0 + 0.5, t1) or {}
    out["long_region"] = dict(ms_per_step=msl, tflops=fl / msl / 1e9, steps=n, seconds=e0.elapsed_time(e1) / 1e3,
                              sm_mhz=ck.get("sm_mhz"), reasons=ck.get("reasons"),
                              tflops_per_ghz=(fl / msl / 1e9) / (ck["sm_mhz"] / 1e3) if ck.get("sm_mhz") else None)
    del g
    return out


def headline_check(state, device):
    """One (request, head) unit of the timed workload against FP32 autograd attention in plain
    torch on the GPU (outside every timed region): rel-L2 of dQ, dK, dV."""
    q, k, v, o, do, lse, run = state
    dq, dk, dv = run()
    b, h = CFG["B"] - 1, 17 % CFG["H"]
    hk = h * CFG["HKV"] // CFG["H"]
    S, D = CFG["S"], CFG["D"]
    qs = q[b, :, h].float().requires_grad_()
    ks = k[b, :, hk].float().requires_grad_()
    vs = v[b, :, hk].float().requires_grad_()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        s = (qs @ ks.T) / D**0.5
        s = s.masked_fill(torch.ones(S, S, device=device, dtype=torch.bool).triu(1), float("-inf"))
        (s.softmax(-1) @ vs).backward(do[b, :, h].float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    rel = lambda a, r: ((a.double() - r.double()).norm() / r.double().norm()).item()  # noqa: E731
    out = dict(unit=[b, h], reference="torch fp32 autograd on the GPU", status=int(run.status), dq=rel(dq[b, h], qs.grad))
    if CFG["H"] == CFG["HKV"]:   # an MHA unit's dK, dV are that head's alone
        out.update(dk=rel(dk[b, hk], ks.grad), dv=rel(dv[b, hk], vs.grad))
    return out


def time_e2e(cfg, device, steps, state):
    """The same metric through the public launch with HOST buffers: every step
    copies q, k, v, o, dO and lse from pinned memory, runs the backward and
    copies dq, dk, dv back. Steps are pipelined the way a host that feeds the
    GPU would run them: two sets of device buffers, the copies in and out on
    their own streams, so step i+1's inputs travel while step i computes and
    step i-1's gradients leave. Timed with events from before the first copy in
    to after the last copy out."""
    from fold_attention_b200.backward import prepare_backward

    q, k, v, o, do, lse, run0 = state
    host_in = [t.detach().cpu().pin_memory() for t in (q, k, v, o, do, lse)]
    slots = []
    for i in range(2):
        dev = (q, k, v, o, do, lse) if i == 0 else tuple(torch.empty_like(t) for t in (q, k, v, o, do, lse))
        run = run0 if i == 0 else prepare_backward(tr(dev[0]), tr(dev[1]), tr(dev[2]), tr(dev[3]), tr(dev[4]), dev[5], causal=True)
        outs = run()
        slots.append(dict(dev=dev, run=run, host_out=[torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs],
                          in_ready=torch.cuda.Event(), comp_done=torch.cuda.Event(), out_done=torch.cuda.Event()))
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in slots[0]["host_out"])
    s_in, s_c, s_out = (torch.cuda.Stream(device) for _ in range(3))

    def step(i):
        sl = slots[i % 2]
        with torch.cuda.stream(s_in):
            s_in.wait_event(sl["comp_done"])      # the step two back has read these inputs
            for d, h in zip(sl["dev"], host_in):
                d.copy_(h, non_blocking=True)
            sl["in_ready"].record(s_in)
        with torch.cuda.stream(s_c):
            s_c.wait_event(sl["in_ready"])
            s_c.wait_event(sl["out_done"])        # and its gradients have left
            res = sl["run"]()
            sl["comp_done"].record(s_c)
        with torch.cuda.stream(s_out):
            s_out.wait_event(sl["comp_done"])
            for h, d in zip(sl["host_out"], res):
                h.copy_(d, non_blocking=True)
            sl["out_done"].record(s_out)

    torch.cuda.synchronize()
    for sl in slots:
        for name in ("in_ready", "comp_done", "out_done"):
            sl[name].record()
    for i in range(2):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(s_in)
    for i in range(steps):
        step(i)
    s_out.wait_stream(s_c)
    e1.record(s_out)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    del slots
    return ms, h2d, d2h


def copy_bandwidth(device, dist):
    """Pinned host <-> device copy bandwidth of this rank with every rank copying at once (what the
    end-to-end leg leans on): GB/s in and out, 1 GiB each way."""
    n = 1 << 30
    host = torch.empty(n, dtype=torch.uint8).pin_memory()
    dev = torch.empty(n, dtype=torch.uint8, device=device)
    dev.copy_(host, non_blocking=True)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    res = []
    for src, dst in ((host, dev), (dev, host)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        res.append(3 * n / e0.elapsed_time(e1) / 1e6)
    return res


def bwd_shape_extra(device, B, H, HKV, steps=4, plan=None, seed=99):
    """Another shape of the same backward (GQA, MQA, small batch): whole step, with the plan it ran."""
    cfg = dict(CFG, B=B, H=H, HKV=HKV)
    state = prepare(cfg, device, seed, plan)
    run = state[-1]
    for _ in range(3):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    fl = flops(B, cfg["S"], H, cfg["D"])
    out = dict(workload=f"B{B} S8192 H{H}/{HKV} D128 causal", ms_per_step=ms, tflops=fl / ms / 1e9,
               plan=[run.plan.subgroup, run.plan.record], folds=run.dk_acc is not None, status=int(run.status))
    del state
    torch.cuda.empty_cache()
    return out


def train_extra(device, steps=3):
    """Forward + backward through the public operator (`fold_attn_func` under autograd) on the
    shape the reference publishes its "train" row for: B2 S8192 H32/8 D128, causal."""
    import fold_attention_b200 as fa

    B, S, H, HKV, D = 2, 8192, 32, 8, 128
    g = torch.Generator(device=device).manual_seed(7)
    q = (torch.randn(B, S, H, D, device=device, generator=g) / D**0.5).bfloat16().requires_grad_()
    k = torch.randn(B, S, HKV, D, device=device, generator=g).bfloat16().requires_grad_()
    v = torch.randn(B, S, HKV, D, device=device, generator=g).bfloat16().requires_grad_()
    do = torch.randn(B, S, H, D, device=device, generator=g).bfloat16()

    def step():
        q.grad = k.grad = v.grad = None
        fa.fold_attn_func(q, k, v, causal=True).backward(do)

    for _ in range(2):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    fl = 3.5 * 2 * B * H * S * S * D / 2   # 2 forward + 5 backward GEMMs, causal half
    return dict(workload="forward + backward, fold_attn_func, B2 S8192 H32/8 D128 causal", ms_per_step=ms,
                tflops=fl / ms / 1e9)


def varlen_extra(device, steps=3):
    """Config 3: packed causal backward, GQA 32/8, D128, 64K tokens in sequences
    of length uniform in [256, 8192] (last truncated), int32 cu_seqlens on device."""
    from fold_attention_b200.backward import attention_forward, prepare_backward

    H, HKV, D, total = 32, 8, 128, 65536
    g = torch.Generator().manual_seed(3)
    lens = []
    while sum(lens) < total:
        lens.append(min(int(torch.randint(256, 8193, (1,), generator=g)), total - sum(lens)))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=device, dtype=torch.int32)
    gd = torch.Generator(device=device).manual_seed(4)
    q = (torch.randn(total, H, D, device=device, generator=gd) / D**0.5).bfloat16()
    k = torch.randn(total, HKV, D, device=device, generator=gd).bfloat16()
    v = torch.randn(total, HKV, D, device=device, generator=gd).bfloat16()
    do = torch.randn(total, H, D, device=device, generator=gd).bfloat16()
    o, lse = attention_forward(q, k, v, causal=True, cu_seqlens=cu, max_seqlen=max(lens))
    run = prepare_backward(q, k, v, o, do, lse, causal=True, cu_seqlens=cu, max_seqlen=max(lens))
    for _ in range(3):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    fl = 5.0 * H * D * sum(n * n for n in lens)
    return dict(workload=f"config3 packed causal backward H32/8 D128 {len(lens)} sequences, {total} tokens",
                ms_per_step=ms, tflops=fl / ms / 1e9, status=int(run.status))


def cpu_reference_tflops(seconds_limit=12.0):
    """The reference's CPU arithmetic for this path: FP32 gradients of causal
    softmax attention per request and head (its benchmarks/harness/training.py
    :124-164), here the oracle's restatement, on the host cores. A bounded
    sample: batch 1, 4 heads, seqlen 2048, head_dim 128, scaled by FLOPs."""
    from oracle import backward as ob

    S, H, D = 2048, 4, 128
    torch.manual_seed(0)
    q, k, v, do = (torch.randn(S, H, D).bfloat16().float() for _ in range(4))
    ob.reference_grads(q[:256], k[:256], v[:256], do[:256], dtype=torch.float32)
    n, t0 = 0, time.time()
    while True:
        ob.reference_grads(q, k, v, do, dtype=torch.float32)
        n += 1
        if time.time() - t0 > seconds_limit or n >= 8:
            break
    dt = (time.time() - t0) / n
    return flops(1, S, H, D) / dt / 1e12, f"B1 H4 S{S} D{D} causal FP32 autograd x{n}, scaled by FLOPs"


# ---- the decode extras ---------------------------------------------------------------------

def decode_lengths(kind, B, seed=5):
    """The config's request lengths: config 5 log-uniform in [4096, 131072], config 4 uniform in
    [1024, 32768]; one seeded draw, so every rank of a sharded run sees the same batch."""
    g = torch.Generator().manual_seed(seed)
    if kind == "config4":
        return torch.randint(1024, 32769, (B,), generator=g).tolist()
    return [int(math.exp(x)) for x in (torch.rand(B, generator=g) * (math.log(131072) - math.log(4096)) + math.log(4096))]


def request_kv(n, HKV, D, device, seed, tail=False, structured=False):
    """One request's prompt K, V from its own seed (a rank can draw any request alone): N(0,1),
    1 % of key positions x 8, 0.1 % of V entries x 20. `tail`: a heavy-tailed key distribution in
    place of the x 8 keys (2 % of positions far above the rest: few live keys at depth 16, as on
    the model captures the reference publishes its decode rows for). `structured`: V drifts from
    one 64-key block to the next and carries a rank-6 image of K, under N(0, 0.5) noise: the
    structure a decode tail can use, and iid V cannot show."""
    g = torch.Generator(device=device).manual_seed(seed)
    kk = torch.randn(n, HKV, D, device=device, generator=g)
    if tail:
        boost = torch.rand(n, 1, 1, device=device, generator=g)
        kk = kk * torch.where(boost < 0.02, 8.0, 0.15)
    else:
        hot = torch.rand(n, 1, 1, device=device, generator=g) < 0.01
        kk = torch.where(hot, kk * 8, kk)
    vv = torch.randn(n, HKV, D, device=device, generator=g)
    if structured:
        nb = -(-n // 64)
        drift = torch.randn(nb, HKV, D, device=device, generator=g).repeat_interleave(64, 0)[:n]
        a = torch.randn(HKV, D, 6, device=device, generator=g) / D**0.5
        b = torch.randn(HKV, 6, D, device=device, generator=g)
        vv = 0.5 * vv + drift + torch.einsum("shd,hdr,hre->she", kk, a, b)
    out = torch.rand(n, HKV, D, device=device, generator=g) < 0.001
    return kk.bfloat16(), torch.where(out, vv * 20, vv).bfloat16()


def decode_extra(device, kind="config5", ids=None, steps=64, kernel="auto", tail=False, with_e2e=True, B=None, seed=5,
                 tail_rank="auto"):
    """A decode config end to end: cache write, then `steps` serving steps (one token appended per
    request per step, then attention), timed as one region; us/step is the mean over the steps.

    config5: v8, depth 16, GQA 64/8, D128, 256 requests; config4: bf16 V, depth None, GQA 32/8,
    128 requests; bf16depth: bf16 V at depth 12 with the decode tail `tail_rank` ("auto": rank 16;
    0: block rows; None: V's mean), GQA 64/8, config 5's lengths, a structured V (`request_kv`).
    `ids` picks a subset of the batch's requests (a rank's shard). Returns the step
    time, the kernel's own counts, the roofline on algorithmic bytes, the clocks while it ran, the
    error of sampled requests against dense FP32 attention, and `e2e`: the same steps through
    `fold_attn_with_kvcache` with q, k, v in pinned host memory and the output copied back."""
    import fold_attention_b200 as fa
    from fold_attention_b200 import FoldKVCache

    dense = kind == "config4"
    deep = kind == "bf16depth"
    H, HKV, D = (32, 8, 128) if dense else (64, 8, 128)
    full = B or (128 if dense else 64 if deep else 256)
    lens_all = decode_lengths(kind, full, seed)
    ids = list(range(full)) if ids is None else list(ids)
    lens = [lens_all[i] for i in ids]
    Bn = len(lens)
    kw = dict(device=device, kernel=kernel)
    if dense:
        c = FoldKVCache(Bn, H, HKV, D, max(lens) + 2 * steps + 16, chunk=4096 if kernel == "mma" else None, **kw)
    elif deep:
        c = FoldKVCache(Bn, H, HKV, D, max(lens) + 2 * steps + 16, depth=12.0, tail=tail_rank,
                        chunk=8192 if kernel == "mma" or tail_rank is not None else None, **kw)
    else:
        # a fixed V scale, as every shard of a sharded layer must use (2^-3 covers |v| <= 56 at 448 / 8)
        c = FoldKVCache(Bn, H, HKV, D, max(lens) + 2 * steps + 16, depth=16.0, v8=True, v_scale=2.0 ** -3,
                        chunk=8192 if kernel == "mma" else None, **kw)
    gd = torch.Generator(device=device).manual_seed(seed + 1)
    pages = c.page_table.shape[1]
    c.page_table.copy_(torch.randperm(Bn * pages, device=device, generator=gd).int().view(Bn, pages))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=device, dtype=torch.int32)
    T = sum(lens)
    k = torch.empty(T, HKV, D, device=device, dtype=torch.bfloat16)
    v = torch.empty(T, HKV, D, device=device, dtype=torch.bfloat16)
    at = 0
    for i, n in zip(ids, lens):   # request by request: the fp32 draws of a whole batch would not fit beside the pool
        k[at:at + n], v[at:at + n] = request_kv(n, HKV, D, device, 1000 * seed + i, tail, structured=deep)
        at += n
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c.write_prompt(k, v, cu, lens)
    torch.cuda.synchronize()
    e0.record()
    c.write_prompt(k, v, cu, lens)
    e1.record()
    torch.cuda.synchronize()
    write_us = e0.elapsed_time(e1) * 1e3
    order = sorted(range(Bn), key=lambda b: lens[b])
    picks = sorted({order[0], order[1 % Bn], order[Bn // 8], order[Bn // 4], order[Bn // 2], order[(3 * Bn) // 4], order[-2 % Bn],
                    order[-1]})
    sample = {b: (k[int(cu[b]):int(cu[b + 1])].clone(), v[int(cu[b]):int(cu[b + 1])].clone()) for b in picks}
    del k, v
    torch.cuda.empty_cache()
    q = torch.randn(Bn, H, D, device=device, generator=gd).bfloat16()
    kn = torch.randn(Bn, HKV, D, device=device, generator=gd).bfloat16()
    vn = torch.randn(Bn, HKV, D, device=device, generator=gd).bfloat16()
    for _ in range(3):
        c.decode(q, kn, vn)
    clocks = Clocks(device.index or 0)
    torch.cuda.synchronize()
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        out = c.decode(q, kn, vn)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ck = clocks.stop(t0, t1)
    us = e0.elapsed_time(e1) / steps * 1e3
    done = 3 + steps
    # the last step against dense FP32 attention over everything written (rel-L2 per sampled request)
    G, errs = H // HKV, []
    for b, (kp, vp) in sample.items():
        ks = torch.cat([kp, kn[b][None].expand(done, -1, -1)]).float()
        vs = torch.cat([vp, vn[b][None].expand(done, -1, -1)]).float()
        qs = q[b].float().view(HKV, G, D)
        w = torch.softmax(torch.einsum("hgd,shd->hgs", qs, ks) / D**0.5, -1)
        want = torch.einsum("hgs,shd->hgd", w, vs).reshape(H, D)
        errs.append(((out[b].float() - want).norm() / want.norm()).item())
    keys = sum(c.lens) * HKV
    live = c.counts[:, 0].sum().item() / keys
    refk = c.counts[:, 1].sum().item() / keys
    vb = 2 * D if dense or deep else D
    byts = keys * (D + 2 + D * refk + vb * live + (2 * D / 64 if c.tail is not None else 0))
    pk = peaks()
    launch_kernels = sorted({l.kernel for l in c._launches.values()})
    status = max(int(l.status) for l in c._launches.values())
    ratio = profiled("decode_sm100_kernel_configs4_5.md", "dram_bytes_over_algorithmic_bytes_" + ("bf16" if dense else "v8"), None)
    res = dict(
        workload=(f"config4 decode bf16 dense B{Bn} H32/8 D128 lens U[1024,32768]" if dense else
                  f"decode bf16 V depth12 tail rank {c.tail_rank} B{Bn} H64/8 D128 lens logU[4096,131072] structured V" if deep else
                  f"config5 decode v8 depth16 B{Bn} H64/8 D128 lens logU[4096,131072]") + (" heavy-tailed keys" if tail else "")
                 + f", {steps} steps, page 256 shuffled",
        kernel="/".join(launch_kernels), us_per_step=us, steps=steps, keys=keys, live_fraction=live, refined_fraction=refk,
        rel_l2_vs_fp32=max(errs), rel_l2_requests=len(errs), status=status, write_prompt_us=write_us, tokens_written=T,
        roofline=dict(bound="hbm", achieved=byts / us / 1e3, peak=pk["hbm"], unit="GB/s", frac=byts / us / 1e3 / pk["hbm"],
                      traffic=(ratio * byts if ratio else None),
                      note=f"algorithmic bytes per step from the kernel's own counts, of {pk['which']} copy bandwidth; traffic = "
                           "the ncu DRAM/algorithmic ratio of a small capture (profiles/) times the step's algorithmic bytes"),
        clocks=ck, gpu_launches=(5 if c.tail is not None else 4) * steps,   # append + Q planes (+ the tail's append), mass reference, decode, combine
    )
    res["algorithmic_gbs"], res["hbm_frac"] = res["roofline"]["achieved"], res["roofline"]["frac"]
    if with_e2e:
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, kn, vn))
        ho = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        dq_, dk_, dv_ = (torch.empty_like(t) for t in (q, kn, vn))
        n2 = max(4, steps // 4)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n2):
            dq_.copy_(hq, non_blocking=True)
            dk_.copy_(hk, non_blocking=True)
            dv_.copy_(hv, non_blocking=True)
            ho.copy_(fa.fold_attn_with_kvcache(dq_, c, dk_, dv_), non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        res["e2e"] = dict(value=e0.elapsed_time(e1) / n2 * 1e3, unit="us/step",
                          h2d_bytes_per_step=sum(t.numel() * t.element_size() for t in (hq, hk, hv)),
                          d2h_bytes_per_step=ho.numel() * ho.element_size(), steps=n2)
    del c, sample
    torch.cuda.empty_cache()
    return res


def levels_extra(device, B=64, steps=20):
    """The decode's layouts beyond the single-level step, timed on the warp-level kernel that
    runs them (CUDA events around `steps` launches of mass reference + decode + combine): a
    two-position draft verified against a bf16 cache (GQA 32/8: 4 query heads x 2 positions a row
    group), the same cache's single-token step beside it, and a cascade of `B` requests sharing
    one 16384-key prefix before 2048 keys of their own, beside the same keys as one flat cache per
    request. Each with the error of sampled rows against FP32 attention over the keys they see."""
    from fold_attention_b200 import FoldKVCache
    from fold_attention_b200.decode import write
    from fold_attention_b200.decode.launch import SharedPrefix, prepare_fold_decode
    from fold_attention_b200.decode.rows import pack_rows

    H, HKV, D = 32, 8, 128
    G = H // HKV
    g = torch.Generator(device=device).manual_seed(31)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(run):
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps * 1e3

    def filled(lens, seed):
        c = FoldKVCache(len(lens), H, HKV, D, max(lens) + 8, device=device, kernel="mma")
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=device, dtype=torch.int32)
        k = torch.empty(sum(lens), HKV, D, device=device, dtype=torch.bfloat16)
        v = torch.empty_like(k)
        at = 0
        for i, n in enumerate(lens):
            k[at:at + n], v[at:at + n] = request_kv(n, HKV, D, device, seed + i)
            at += n
        c.write_prompt(k, v, cu, lens)
        return c, k, v, cu

    def quantise(c, rows):
        qa = torch.zeros(rows.shape, device=device, dtype=torch.int8)
        qb, eq = torch.zeros_like(qa), torch.ones(rows.shape[:2], device=device, dtype=torch.float32)
        write.step(rows.reshape(-1, D).contiguous(), None, None, qa.view(-1, D), qb.view(-1, D), eq.view(-1), c.ek, c.page_table,
                   c.page_size, c.seq_lens, c.ka, c.kb, c.va, c.vb, 1.0, c.vsum, c.vmean, c.seq_lens)
        return qa, qb, eq

    def attend(q, kk, vv):
        w = torch.softmax((q.float() @ kk.float().T) / D**0.5, -1)
        return w @ vv.float()

    res = {}
    # ---- a two-position draft on config 4's lengths ----
    lens = decode_lengths("config4", B, 7)
    c, k, v, cu = filled(lens, 7000)
    q = torch.randn(B, 2, H, D, device=device, generator=g).bfloat16()
    common = dict(split=c._auto_split(), refine_k=10.0, refine_v=10.0, v_scale=1.0, page_table=c.page_table, page_size=c.page_size,
                  seq_lens=c.seq_lens, n_kv_heads=HKV, reference="mass", weight_terms=2, kernel="mma")
    qa, qb, eq = quantise(c, pack_rows(q, HKV, 2))
    z = torch.empty((B * HKV, 2 * G), device=device)
    draft = prepare_fold_decode(qa, qb, eq, c.ka, c.kb, c.ek, c.va, z, torch.full_like(z, 1e4), draft_len=2, causal=True, **common)
    qa1, qb1, eq1 = quantise(c, pack_rows(q[:, 1:], HKV, 1))
    z1 = torch.empty((B * HKV, G), device=device)
    single = prepare_fold_decode(qa1, qb1, eq1, c.ka, c.kb, c.ek, c.va, z1, torch.full_like(z1, 1e4), **common)
    us_d, us_s = timed(draft), timed(single)
    out = draft()[0]
    errs = []
    for b in (0, B // 2, B - 1):
        a, n = int(cu[b]), lens[b]
        for t in range(2):
            want = attend(q[b, t, :G], k[a:a + n - 1 + t, 0], v[a:a + n - 1 + t, 0])
            errs.append(((out[b * HKV, t::2].float() - want).norm() / want.norm()).item())
    res["draft"] = dict(workload=f"bf16 dense B{B} H32/8 D128 lens U[1024,32768], 2 draft positions (8 rows a group), warp-level kernel",
                        us_per_step=us_d, single_token_us_per_step=us_s, keys=sum(lens) * HKV, rel_l2_vs_fp32=max(errs),
                        status=int(draft.status))
    del c, k, v, draft, single
    torch.cuda.empty_cache()
    # ---- a cascade: one 16384-key prefix, 2048 keys of each request's own ----
    PL, UL = 16384, 2048
    P, kp, vp, _ = filled([PL], 8000)
    U, ku, vu, cuu = filled([UL] * B, 8100)
    F, kf, vf, _ = filled([PL + UL] * 8, 8200)          # the flat comparison at B8: the same keys per request, eight copies
    q = torch.randn(B, H, D, device=device, generator=g).bfloat16()
    qa, qb, eq = quantise(U, pack_rows(q[:, None], HKV, 1))
    z = torch.empty((B * HKV, G), device=device)
    level = SharedPrefix(P.ka, P.kb, P.ek, P.va, P.page_table, P.seq_lens, P.page_size, split=8)
    common.update(page_table=U.page_table, page_size=U.page_size, seq_lens=U.seq_lens, split=2)
    casc = prepare_fold_decode(qa, qb, eq, U.ka, U.kb, U.ek, U.va, z, torch.full_like(z, 1e4), shared=level, **common)
    qa8, qb8, eq8 = quantise(F, pack_rows(q[:8, None], HKV, 1))
    z8 = torch.empty((8 * HKV, G), device=device)
    common.update(page_table=F.page_table, page_size=F.page_size, seq_lens=F.seq_lens, split=F._auto_split())
    flat = prepare_fold_decode(qa8, qb8, eq8, F.ka, F.kb, F.ek, F.va, z8, torch.full_like(z8, 1e4), **common)
    us_c, us_f = timed(casc), timed(flat)
    out = casc()[0]
    errs = []
    for b in (0, B - 1):
        a = int(cuu[b])
        want = attend(q[b, :G], torch.cat([kp[:, 0], ku[a:a + UL, 0]]), torch.cat([vp[:, 0], vu[a:a + UL, 0]]))
        errs.append(((out[b * HKV].float() - want).norm() / want.norm()).item())
    res["cascade"] = dict(workload=f"bf16 dense B{B} H32/8 D128: one shared prefix of {PL} keys + {UL} own keys a request, warp-level kernel",
                          us_per_step=us_c, keys_attended=B * HKV * (PL + UL), keys_stored=HKV * (PL + B * UL),
                          flat_b8_us_per_step=us_f, flat_b8_keys=8 * HKV * (PL + UL), rel_l2_vs_fp32=max(errs), status=int(casc.status),
                          note="every request's row group reads the prefix itself; its pages are shared, so the repeats are L2 hits")
    return res


def write_prompt_extra(device):
    """The prompt writer on the shape the reference publishes a row for (235 us on H100, eager, with
    host planning: 32 prompts of 2048 tokens, 4 KV heads, D128, 8-bit V)."""
    from fold_attention_b200 import FoldKVCache

    B, L, H, HKV, D = 32, 2048, 32, 4, 128
    c = FoldKVCache(B, H, HKV, D, L + 8, depth=16.0, v8=True, page_size=128, device=device)
    g = torch.Generator(device=device).manual_seed(12)
    k = torch.randn(B * L, HKV, D, device=device, generator=g).bfloat16()
    v = torch.randn(B * L, HKV, D, device=device, generator=g).bfloat16()
    cu = torch.arange(B + 1, device=device, dtype=torch.int32) * L
    lens = [L] * B
    for _ in range(3):
        c.write_prompt(k, v, cu, lens)
    torch.cuda.synchronize()
    t0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    n = 20
    for _ in range(n):
        c.write_prompt(k, v, cu, lens)
    e1.record()
    torch.cuda.synchronize()
    wall = (time.time() - t0) / n * 1e6
    us = e0.elapsed_time(e1) / n * 1e3
    byts = B * L * HKV * (2 * D * 2 + 4 * D + 2)   # k, v read (bf16); four planes and a scale written
    return dict(workload="write_prompt 8-bit V, 32 x 2048 tokens, 4 KV heads, D128", us_device=us, us_wall_with_host_planning=wall,
                gbs=byts / us / 1e3, hbm_frac=byts / us / 1e3 / peaks()["hbm"])


# ---- sharded extras (N > 1) ------------------------------------------------------------------

def sharded_backward_extra(device, dist, world, rank, steps=4):
    """Config 2's (request, KV head) units split over the ranks (`parallel.backward_units`): every
    rank draws the same seeded workload and runs its own slice under the full call's plan; the step
    time is the slowest rank's. One unit is then gathered to rank 0 and compared, bit for bit, with
    that unit run alone there."""
    from fold_attention_b200 import parallel
    from fold_attention_b200.backward import attention_forward, prepare_backward
    from fold_attention_b200.backward.plan import plan_dense

    cfg = dict(CFG, HKV=8)      # the GQA variant: 32 units of four heads
    B, S, H, HKV, D = (cfg[k] for k in ("B", "S", "H", "HKV", "D"))
    G = H // HKV
    plan = plan_dense(B, H, HKV, S, D, True)
    units = parallel.backward_units(B, HKV, world, rank)
    q, k, v, do = make_inputs(cfg, device, 4321)      # the same on every rank
    runs = []
    for b, (lo, hi) in units.items():
        qs, dos = (x[b:b + 1, :, lo * G:hi * G].contiguous() for x in (q, do))
        ks, vs = (x[b:b + 1, :, lo:hi].contiguous() for x in (k, v))
        os_, ls = attention_forward(qs, ks, vs, causal=True)
        runs.append((b, lo, hi, prepare_backward(tr(qs), tr(ks), tr(vs), tr(os_), tr(dos), ls, causal=True, plan=plan)))
    for _ in range(2):
        for r in runs:
            r[3]()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for _ in range(steps):
        for r in runs:
            r[3]()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # the unit (request B-1, KV head HKV-1) lives on the last rank: its dK travels to rank 0
    b, h = B - 1, HKV - 1
    got = torch.empty(1, 1, S, D, device=device, dtype=torch.bfloat16)
    if rank == world - 1:
        own = [r for r in runs if r[0] == b and r[1] <= h < r[2]][0]
        got.copy_(own[3]()[1][:, h - own[1]:h - own[1] + 1])
    dist.broadcast(got, src=world - 1)
    same = None
    if rank == 0:
        qs, dos = (x[b:b + 1, :, h * G:(h + 1) * G].contiguous() for x in (q, do))
        ks, vs = (x[b:b + 1, :, h:h + 1].contiguous() for x in (k, v))
        os_, ls = attention_forward(qs, ks, vs, causal=True)
        alone = prepare_backward(tr(qs), tr(ks), tr(vs), tr(os_), tr(dos), ls, causal=True, plan=plan)()
        same = bool(torch.equal(alone[1], got))
    ms = t.item()
    return dict(workload=f"config2 GQA B4 S8192 H32/8: {B * HKV} (request, KV head) units over {world} ranks, strong scaling",
                ms_per_step=ms, tflops=flops(B, S, H, D) / ms / 1e9, units_this_rank=sum(hi - lo for lo, hi in units.values()),
                gathered_unit_equals_single_gpu_run=same)


def sharded_decode_extra(device, dist, world, rank, steps=64):
    """Config 5's 256 requests (one seeded batch), partitioned over the ranks by length
    (`parallel.balance`); the step time is the slowest rank's."""
    from fold_attention_b200 import parallel

    lens = decode_lengths("config5", 256)
    part = parallel.balance(lens, world)[rank]
    try:
        d = decode_extra(device, "config5", ids=part, steps=steps, with_e2e=False)
        t = torch.tensor([d["us_per_step"], 0.0], device=device, dtype=torch.float64)
        u = torch.tensor([d["keys"], d["roofline"]["achieved"] * d["us_per_step"]], device=device, dtype=torch.float64)
    except Exception as e:   # a rank that cannot hold its shard must not hang the others
        d = dict(error=repr(e))
        t = torch.tensor([float("inf"), 1.0], device=device, dtype=torch.float64)
        u = torch.zeros(2, device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    if t[1].item() != 0.0:
        return d if "error" in d else dict(error="a rank failed")
    us = t[0].item()
    return dict(workload=f"config5 decode, the same 256 requests over {world} ranks balanced by length, {steps} steps",
                kernel=d["kernel"], us_per_step=us, keys=int(u[0].item()), algorithmic_gbs=u[1].item() / us,
                hbm_frac_per_gpu=u[1].item() / us / world / peaks()["hbm"], requests_this_rank=len(part))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm may use every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    val, sample = cpu_reference_tflops(20.0)
    cores = torch.get_num_threads()
    line = dict(
        impl="reference", metric=METRIC, value=val, unit="TFLOP/s", n_gpus=args.gpus, steps=args.steps,
        warmup=args.warmup, ms_per_step=flops(**{k: CFG[k] for k in ("B", "S", "H", "D")}) / val / 1e9,
        higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
        config=dict(workload=WORKLOAD.format(B=CFG["B"])),
        cpu_baseline=dict(value=val, unit="TFLOP/s", cores=cores, kind="port", sample=sample),
        e2e=dict(value=val, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
    )
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-extra", action="store_true", help="skip the extra keys")
    ap.add_argument("--batch", type=int, default=CFG["B"],
                    help="batch of the backward workload (config 2 is 4; 1 gives the small case ncu captures)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--decode-only", action="store_true", help="run only one decode extra and print its dict")
    ap.add_argument("--decode-batch", type=int, default=None)
    ap.add_argument("--decode-steps", type=int, default=64)
    ap.add_argument("--decode-kernel", default="auto", choices=("auto", "mma", "sm100"))
    ap.add_argument("--decode-dense", action="store_true", help="config 4's shape instead of config 5's")
    ap.add_argument("--decode-tail", action="store_true", help="heavy-tailed keys: few live keys at depth 16")
    ap.add_argument("--decode-levels", action="store_true", help="run only the draft / cascade extra and print its dict")
    ap.add_argument("--decode-bf16-depth", default=None, choices=("auto", "rows", "mean"),
                    help="the bf16-V depth-12 extra instead: with the rank-16 tail, the block rows alone, or V's mean")
    args = ap.parse_args()
    CFG["B"] = args.batch
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.decode_levels:
        torch.cuda.set_device(0)
        print(json.dumps(levels_extra(torch.device("cuda", 0))), flush=True)
        return
    if args.decode_only:
        torch.cuda.set_device(0)
        kind = "bf16depth" if args.decode_bf16_depth else "config4" if args.decode_dense else "config5"
        print(json.dumps(decode_extra(torch.device("cuda", 0), kind,
                                      steps=max(2, args.decode_steps), B=args.decode_batch, kernel=args.decode_kernel,
                                      tail=args.decode_tail, with_e2e=False,
                                      tail_rank={"auto": "auto", "rows": 0, "mean": None, None: "auto"}[args.decode_bf16_depth])), flush=True)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    clocks = Clocks(local)
    state = prepare(CFG, device, 1234 + rank)
    ms, main_ms, (t0, t1) = time_backward(state, args.steps, args.warmup, dist)
    ck = clocks.window(t0, t1)
    fl = flops(CFG["B"], CFG["S"], CFG["H"], CFG["D"])
    t = torch.tensor([ms, main_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, main_max = t.tolist()
    timing = time_protocols(state, device, clocks, ms) if (rank == 0 and not args.no_extra) else None
    check = headline_check(state, device) if (rank == 0 and not args.no_extra) else None
    clocks.stop()
    if args.no_e2e:
        e2e_ms, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_ms, h2d, d2h = time_e2e(CFG, device, max(2, args.steps // 3), state)
    t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_max = t.item()
    plan = state[-1].plan
    del state
    torch.cuda.empty_cache()
    pk = peaks()
    achieved = fl / main_max / 1e9
    traffic1 = profiled("bwd_main_sm100_config2.md", "dram_bytes_per_launch_batch1", None)
    line = dict(
        metric=METRIC, value=world * fl / ms_max / 1e9, unit="TFLOP/s", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=ms_max, higher_is_better=True, scaling="weak", vs_baseline=None,
        dtype="bf16", data="synthetic",
        config=dict(workload=WORKLOAD.format(B=CFG["B"]), l2="inputs (1.3 GB) larger than L2", shard="batch x KV head, one workload per rank"),
        e2e=dict(value=world * fl / e2e_max / 1e9, unit="TFLOP/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
        gpu_launches=KERNELS_PER_STEP * args.steps,
        clocks=ck,
        roofline=dict(bound="tensor", achieved=achieved, peak=pk["bf16_burst"], unit="TFLOP/s",
                      frac=achieved / pk["bf16_burst"], frac_of_sustained=achieved / pk["bf16"],
                      frac_of_nominal_2250=achieved / 2250.0,
                      # dram__bytes_read + write of one main-loop launch in the batch-1 ncu capture kept in
                      # profiles/, times the batch (the traffic is per request)
                      traffic=(traffic1 * CFG["B"] if traffic1 else None),
                      note=f"main-loop kernel (work list included); peak = {pk['which']} burst bf16 GEMM (the timed region is "
                           f"short: the clock has not settled under the power limit), sustained {pk['bf16']}; traffic in bytes "
                           "per launch = the batch-1 ncu capture in profiles/ times the batch"),
    )
    extra = dict(plan=[plan.subgroup, plan.record], headline_check=check)
    if timing:
        extra["timing"] = timing
    if rank == 0 and world == 1 and not args.no_e2e:
        val, sample = cpu_reference_tflops()
        line["cpu_baseline"] = dict(value=val, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port", sample=sample)
    if rank == 0 and world == 1 and not args.no_extra:
        for key, fn in (("gqa_32_8", lambda: bwd_shape_extra(device, 4, 32, 8)),
                        ("mqa_b2_32_1", lambda: bwd_shape_extra(device, 2, 32, 1)),
                        ("small_batch_b1_32_8", lambda: bwd_shape_extra(device, 1, 32, 8)),
                        ("varlen_config3", lambda: varlen_extra(device)),
                        ("train_fwd_bwd", lambda: train_extra(device)),
                        ("write_prompt", lambda: write_prompt_extra(device)),
                        ("decode_config5", lambda: decode_extra(device, "config5")),
                        ("decode_config4", lambda: decode_extra(device, "config4")),
                        ("decode_config5_few_live_keys", lambda: decode_extra(device, "config5", B=64, tail=True, with_e2e=False)),
                        ("decode_levels", lambda: levels_extra(device)),
                        ("decode_bf16_depth12_tail16", lambda: decode_extra(device, "bf16depth", with_e2e=False)),
                        ("decode_bf16_depth12_vmean", lambda: decode_extra(device, "bf16depth", with_e2e=False, tail_rank=None, kernel="mma"))):
            try:
                extra[key] = fn()
            except Exception as e:  # the headline stands on its own
                extra[key] = dict(error=repr(e))
            torch.cuda.empty_cache()
    if world > 1 and not args.no_extra:
        for key, fn in (("sharded_backward", lambda: sharded_backward_extra(device, dist, world, rank)),
                        ("decode_config5", lambda: sharded_decode_extra(device, dist, world, rank))):
            try:
                extra[key] = fn()
            except Exception as e:
                extra[key] = dict(error=repr(e))
            torch.cuda.empty_cache()
        bw = torch.tensor(copy_bandwidth(device, dist), device=device, dtype=torch.float64)
        allbw = [torch.zeros_like(bw) for _ in range(world)]
        dist.all_gather(allbw, bw)
        extra["pinned_copy_gbs_per_rank"] = dict(h2d=[round(x[0].item(), 1) for x in allbw], d2h=[round(x[1].item(), 1) for x in allbw],
                                                 note="every rank copying 1 GiB each way at once")
    line["extra"] = extra
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
