"""Benchmark of the deterministic causal attention backward (and, as extra
keys, the paged decode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout. A step is one backward (preprocess + main loop +
postprocess) over the headline configuration (config 2): batch 4, seqlen 8192, 32 query / 32 KV
heads, head_dim 128, bf16, causal; inputs iid N(0,1) with 1/sqrt(D) on q, O and
LSE from the library's own forward, computed before the timed region. At
N > 1 every rank runs that workload on its own shard (weak scaling; the path
shards over batch x KV head with no collective on the data path).
"""

from __future__ import annotations

import argparse
import json
import os
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

    def stop(self, t0, t1):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for ts, r in self.rows if t0 - 0.05 <= ts <= t1 + 0.15] or [r for _, r in self.rows[-3:]]
        if not rows:
            return None
        mhz = sorted(int(r[0]) for r in rows if r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return dict(sm_mhz=mhz[len(mhz) // 2] if mhz else None,
                    sm_max_mhz=int(rows[0][1]) if rows[0][1].isdigit() else None,
                    reasons=reasons, samples=len(rows))


def make_inputs(cfg, device, seed):
    B, S, H, HKV, D = (cfg[k] for k in ("B", "S", "H", "HKV", "D"))
    g = torch.Generator(device=device).manual_seed(seed)
    q = (torch.randn(B, S, H, D, device=device, generator=g) / D**0.5).bfloat16()
    k = torch.randn(B, S, HKV, D, device=device, generator=g).bfloat16()
    v = torch.randn(B, S, HKV, D, device=device, generator=g).bfloat16()
    do = torch.randn(B, S, H, D, device=device, generator=g).bfloat16()
    return q, k, v, do


def time_backward(cfg, device, steps, warmup, seed, dist):
    """(ms per step, main-kernel ms per launch, launches per step, run)."""
    from fold_attention_b200.backward import attention_forward, prepare_backward

    q, k, v, do = make_inputs(cfg, device, seed)
    o, lse = attention_forward(q, k, v, causal=True)
    tr = lambda x: x.transpose(1, 2)  # noqa: E731
    run = prepare_backward(tr(q), tr(k), tr(v), tr(o), tr(do), lse, causal=True)
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
    total = ev[0][0].elapsed_time(ev[-1][3]) / steps
    main = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    # per step: the statistics' memset, preprocess, its finalize pass, main loop, postprocess
    return total, main, 5, (q, k, v, o, do, lse, run), (t0, t1)


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
    tr = lambda x: x.transpose(1, 2)  # noqa: E731
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
                ms_per_step=ms, tflops=fl / ms / 1e9)


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


def decode_extra(device, steps=8, B=32, dense=False, kernel="auto", seed=5):
    """Config 5's decode (extra keys, not the headline; B=256 is the config's own batch):
    v8, depth 16, GQA 64/8, D128, lengths log-uniform in [4096, 131072]; or with
    `dense` config 4's shape: bf16 V, depth None, GQA 32/8, lengths uniform in
    [1024, 32768]."""
    import math

    from fold_attention_b200 import FoldKVCache

    H, HKV, D = (32, 8, 128) if dense else (64, 8, 128)
    # the pool is sized by the longest request for every request: halve the batch until the pool and
    # the prompt tensors fit beside what is already on the device
    free = torch.cuda.mem_get_info(device)[0]
    top = 32768 if dense else 131072
    while B > 8 and B * (top + 256) * HKV * (642 if dense else 514) * 1.30 + (6 << 30) > free:
        B //= 2
    g = torch.Generator().manual_seed(seed)
    if dense:
        lens = torch.randint(1024, 32769, (B,), generator=g).tolist()
        c = FoldKVCache(B, H, HKV, D, max(lens) + steps + 2, device=device, kernel=kernel,
                        chunk=4096 if kernel == "mma" else None)
    else:
        lens = [int(math.exp(x)) for x in (torch.rand(B, generator=g) * (math.log(131072) - math.log(4096)) + math.log(4096))]
        c = FoldKVCache(B, H, HKV, D, max(lens) + steps + 2, depth=16.0, v8=True, device=device, kernel=kernel,
                        chunk=8192 if kernel == "mma" else None)
    gd = torch.Generator(device=device).manual_seed(seed + 1)
    pages = c.page_table.shape[1]
    perm = torch.randperm(B * pages, device=device, generator=gd).int().view(B, pages)
    c.page_table.copy_(perm)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=device, dtype=torch.int32)
    T = sum(lens)
    # request by request: the fp32 draws of a whole large batch would not fit beside the pool
    k = torch.empty(T, HKV, D, device=device, dtype=torch.bfloat16)
    v = torch.empty(T, HKV, D, device=device, dtype=torch.bfloat16)
    at = 0
    for n in lens:
        kk = torch.randn(n, HKV, D, device=device, generator=gd)
        hot = torch.rand(n, 1, 1, device=device, generator=gd) < 0.01
        k[at:at + n] = torch.where(hot, kk * 8, kk)
        vv = torch.randn(n, HKV, D, device=device, generator=gd)
        out = torch.rand(n, HKV, D, device=device, generator=gd) < 0.001
        v[at:at + n] = torch.where(out, vv * 20, vv)
        at += n
    del kk, vv, hot, out
    c.write_prompt(k, v, cu, lens)
    # the two shortest and the longest request's prompts, kept to check the steps' output afterwards
    order = sorted(range(B), key=lambda b: lens[b])
    sample = {b: (k[int(cu[b]):int(cu[b + 1])].clone(), v[int(cu[b]):int(cu[b + 1])].clone()) for b in order[:2] + order[-1:]}
    del k, v
    q = torch.randn(B, H, D, device=device, generator=gd).bfloat16()
    kn = torch.randn(B, HKV, D, device=device, generator=gd).bfloat16()
    vn = torch.randn(B, HKV, D, device=device, generator=gd).bfloat16()
    for _ in range(2):
        c.decode(q, kn, vn)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        out = c.decode(q, kn, vn)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / steps * 1e3
    # the last step against dense FP32 attention over everything written (rel-L2, worst sampled request)
    G, err = H // HKV, 0.0
    for b, (kp, vp) in sample.items():
        ks = torch.cat([kp, kn[b][None].expand(2 + steps, -1, -1)]).float()
        vs = torch.cat([vp, vn[b][None].expand(2 + steps, -1, -1)]).float()
        qs = q[b].float().view(HKV, G, D)
        w = torch.softmax(torch.einsum("hgd,shd->hgs", qs, ks) / D**0.5, -1)
        want = torch.einsum("hgs,shd->hgd", w, vs).reshape(H, D)
        err = max(err, ((out[b].float() - want).norm() / want.norm()).item())
    del sample
    keys = sum(c.lens) * HKV
    live = c.counts[:, 0].sum().item() / keys
    refk = c.counts[:, 1].sum().item() / keys
    vb = 2 * D if dense else D
    byts = keys * (D + 2 + D * refk + vb * live)
    name = (f"config4-shaped decode bf16 dense B{B} H32/8 D128 lens U[1024,32768] " +
            ("chunk4096" if kernel == "mma" else "default split") if dense else
            f"config5-shaped decode v8 depth16 B{B} H64/8 D128 lens logU[4096,131072] " +
            ("chunk8192" if kernel == "mma" else "default split"))
    return dict(workload=name, kernel="/".join(sorted({l.kernel for l in c._launches.values()})),
                us_per_step=us, keys=keys, live_fraction=live, refined_fraction=refk, rel_l2_vs_fp32=err,
                algorithmic_gbs=byts / us / 1e3, hbm_frac=byts / us / 1e3 / peaks()["hbm"])


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
    ap.add_argument("--no-extra", action="store_true", help="skip the decode extra keys")
    ap.add_argument("--batch", type=int, default=CFG["B"],
                    help="batch of the backward workload (config 2 is 4; 1 gives the small case ncu captures)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--decode-only", action="store_true",
                    help="run only the config-5-shaped decode (extra keys) and print its dict")
    ap.add_argument("--decode-batch", type=int, default=32)
    ap.add_argument("--decode-kernel", default="auto", choices=("auto", "mma", "sm100"))
    ap.add_argument("--decode-dense", action="store_true", help="config 4's shape instead of config 5's")
    args = ap.parse_args()
    CFG["B"] = args.batch
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.decode_only:
        torch.cuda.set_device(0)
        print(json.dumps(decode_extra(torch.device("cuda", 0), steps=max(2, args.steps), B=args.decode_batch,
                                      dense=args.decode_dense, kernel=args.decode_kernel)), flush=True)
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
    ms, main_ms, launches, state, (t0, t1) = time_backward(CFG, device, args.steps, args.warmup, 1234 + rank, dist)
    ck = clocks.stop(t0, t1)
    fl = flops(CFG["B"], CFG["S"], CFG["H"], CFG["D"])
    t = torch.tensor([ms, main_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, main_max = t.tolist()
    if args.no_e2e:
        e2e_ms, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_ms, h2d, d2h = time_e2e(CFG, device, max(2, args.steps // 3), state)
    t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_max = t.item()
    del state
    torch.cuda.empty_cache()
    pk = peaks()
    line = dict(
        metric=METRIC, value=world * fl / ms_max / 1e9, unit="TFLOP/s", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=ms_max, higher_is_better=True, scaling="weak", vs_baseline=None,
        dtype="bf16", data="synthetic",
        config=dict(workload=WORKLOAD.format(B=CFG["B"]), l2="inputs (1.3 GB) larger than L2", shard="batch x KV head, one workload per rank"),
        e2e=dict(value=world * fl / e2e_max / 1e9, unit="TFLOP/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
        gpu_launches=launches * args.steps,
        clocks=ck,
        roofline=dict(bound="tensor", achieved=fl / main_max / 1e9, peak=pk["bf16"], unit="TFLOP/s",
                      frac=fl / main_max / 1e9 / pk["bf16"],
                      # dram__bytes_read + write of one main-loop launch: 631.1 MB in an ncu capture at
                      # batch 1, scaled by the batch (the traffic is per request)
                      traffic=631.1e6 * CFG["B"],
                      note=f"main-loop kernel, of {pk['which']} sustained bf16 GEMM; burst peak {pk['bf16_burst']}; "
                           "traffic in bytes per launch, scaled from a batch-1 ncu capture"),
    )
    if rank == 0 and world == 1 and not args.no_e2e:
        val, sample = cpu_reference_tflops()
        line["cpu_baseline"] = dict(value=val, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port", sample=sample)
        if not args.no_extra:
            gqa = dict(CFG, HKV=8)
            ms_g, main_g, _, st_g, _ = time_backward(gqa, device, max(2, args.steps // 2), 3, 99, None)
            del st_g
            torch.cuda.empty_cache()
            line["extra"] = dict(gqa_32_8=dict(ms_per_step=ms_g, tflops=fl / ms_g / 1e9))
            for key, fn in (("varlen_config3", lambda: varlen_extra(device)),
                            ("train_fwd_bwd", lambda: train_extra(device)),
                            ("decode_config5", lambda: decode_extra(device, steps=6, B=256)),
                            ("decode_config4", lambda: decode_extra(device, B=128, dense=True))):
                try:
                    line["extra"][key] = fn()
                except Exception as e:  # the headline stands on its own
                    line["extra"][key] = dict(error=repr(e))
                torch.cuda.empty_cache()
    if world > 1 and not args.no_extra:
        # the decode path sharded over requests: config 5's shape, 32 requests per rank (8 ranks hold
        # its 256), every rank its own lengths; the step time is the slowest rank's
        try:
            d = decode_extra(device, seed=5 + 2 * rank)
            t = torch.tensor([d["us_per_step"], 0.0], device=device, dtype=torch.float64)
            u = torch.tensor([d["keys"], d["algorithmic_gbs"] * d["us_per_step"]], device=device, dtype=torch.float64)
        except Exception as e:
            d = dict(error=repr(e))
            t = torch.tensor([float("inf"), 1.0], device=device, dtype=torch.float64)
            u = torch.zeros(2, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(u, op=dist.ReduceOp.SUM)
        if t[1].item() == 0.0:
            us = t[0].item()
            line["extra"] = dict(decode_config5=dict(
                workload=d["workload"].replace("B32", f"B{32 * world} (32 per rank)"), kernel=d["kernel"], us_per_step=us,
                keys=int(u[0].item()), algorithmic_gbs=u[1].item() / us, hbm_frac_per_gpu=u[1].item() / us / world / pk["hbm"]))
        else:
            line["extra"] = dict(decode_config5=d if "error" in d else dict(error="a rank failed"))
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
