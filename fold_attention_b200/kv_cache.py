"""One attention layer's serving state: a causal prefill, then the decode over
a quantised paged cache. Same constructor, methods and tensor attributes as
the reference's `FoldKVCache` (src/fold_attention/kv_cache.py:65-963) for the
single-level serving path; every kernel runs in libfold_b200.

Every key carries its own scale, so a key appended later is quantised as
precisely as the prompt's and nothing is reserved for it. An 8-bit V takes
one power of two for the layer, fixed at prefill (`v_headroom`).
"""

from __future__ import annotations

import math

import torch

from .backward.launch import attention_forward
from .decode import tail as tail_fit
from .decode import write
from .decode.heuristics import (
    pick_split,
    refine_bands_for,
    refine_for,
    tail_rank_for,
    weight_terms_for,
)
from .decode.launch import mass_z, prepare_fold_decode
from .utils import Launch


class ReplayStep(Launch):
    """`prepare_replay_step`'s result: calling it runs the step again."""

BN = 64  # keys per decode tile: a fixed `chunk` is a multiple of it


class FoldKVCache:
    """A paged, quantised KV cache for `batch` requests of one layer, and the
    decode attention over it.

    `prefill` takes the prompts, packed, and returns their causal attention;
    `decode` appends one token per request and returns its attention over
    everything so far (`append` and `attend` do the two halves).

    `depth` is the truncation depth: a key whose weight is under `2^-depth`
    of its row's mass is dropped (its mass re-enters at V's mean), and None
    keeps every key. The reference is each row's log-sum-exp, estimated every
    step from the cache and the step's query alone. `v8` stores V as two e4m3
    planes rather than bf16 under one power-of-two scale: `v_scale` if given,
    otherwise set by the prefill from the batch's largest value.
    `refine_k`, `refine_v` and `weight_terms` trade accuracy for time and
    default to the reference's gates. `split` fixes the CTAs per row group and
    `chunk` the keys per split (a multiple of 64); with either, a request's
    output depends on the request alone.

    `kernel` (not a reference argument) picks the split-KV kernel: "mma" is
    the warp-level one, which takes every shape; "sm100" the tcgen05 one
    (head_dim 128, pages and chunks of a multiple of 128 keys), which
    streams K's first plane and V whole and is the faster the longer the
    contexts are; "auto" takes "sm100" where it applies, for
    the requests of 2048 keys or more (measured faster from 1024 keys up, on
    an 8-bit and on a 16-bit V, since requests of up to 8192 keys stream both
    planes of K there; a CTA's fixed cost is what very short requests would
    pay): the batch goes where most of its keys would. With `mix_kernels` set (and a `chunk`)
    the short requests of a batch go to "mma" and the long ones to "sm100" in
    the same step; on one B200 that measured slower up to 128 requests (the
    short requests' launch cannot fill the GPU by itself), so it is off.

    `tail` is the decode tail's rank on a bf16 V at a finite depth: dropped
    mass re-enters at each 64-key block's mean V (0) plus the part of a key's
    V its K predicts through a rank-16 map fitted on the prompt (16); None for
    V's mean alone, "auto" for the reference's policy (`tail_rank_for`: 16 for
    these groups; no tail where the pages do not hold whole 64-key blocks).
    The tail runs on the warp-level kernel, so a cache that has one does not
    take "sm100" (pass `tail=None` to put a truncating bf16 V there).
    `check_range` reads each
    step's denominators on the host and reruns the rows whose reference sat
    outside `[0.5, 2^60]` (`2^100` on a bf16 V) of their mass.
    """

    SM100_MIN_KEYS = 2048    # requests shorter than this stay on the warp-level kernel under kernel="auto"

    def __init__(
        self,
        batch,
        n_heads,
        n_kv_heads,
        head_dim,
        max_len,
        *,
        depth=None,
        v8=False,
        page_size=256,
        split=None,
        tail="auto",
        refine_k=None,
        refine_v=None,
        weight_terms=None,
        v_headroom=2.0,
        v_scale=None,
        check_range=False,
        chunk=None,
        device="cuda",
        kernel="auto",
    ):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not group over {n_kv_heads} KV heads")
        self.batch, self.n_heads, self.n_kv_heads, self.head_dim = batch, n_heads, n_kv_heads, head_dim
        self.group = n_heads // n_kv_heads
        self.n_groups = batch * n_kv_heads
        self.page_size = page_size
        self.max_len = max_len
        self.depth = depth
        self.v8 = bool(v8)
        self.v_headroom = float(v_headroom)
        self.split = split
        self.device = torch.device(device)
        # the split-KV kernel (not a reference argument): "mma", "sm100" or "auto"
        self.kernel = kernel
        self.mix_kernels = False
        if head_dim not in (64, 128):
            raise NotImplementedError(f"head_dim {head_dim}: the cache takes 64 or 128")
        if self.group > 8 and (self.group % 8 or self.group > 32):
            raise NotImplementedError(f"a row group of {self.group} rows: 1..8, 16, 24 or 32 are supported")
        # a group wider than 8 rows runs as groups of 8 on one KV head, on the warp-level kernel
        self._gsub = 1 if self.group <= 8 else self.group // 8
        if self._gsub > 1:
            if kernel == "sm100":
                raise NotImplementedError("row groups wider than 8 run on the warp-level kernel: kernel='mma' or 'auto'")
            self.kernel = "mma"
        if page_size < 16 or page_size % 16 or (page_size % 64 and 64 % page_size):
            raise ValueError(f"page_size={page_size}: a multiple of 64, or 16 or 32")

        dev, D, HKV, PS = self.device, head_dim, n_kv_heads, page_size
        pages = -(-max_len // PS)
        rows = batch * pages * HKV * PS
        self.page_table = torch.arange(batch * pages, device=dev, dtype=torch.int32).view(batch, pages)
        self.ka = torch.zeros((rows, D), device=dev, dtype=torch.int8)
        self.kb = torch.zeros_like(self.ka)
        if self.v8:
            self.va = torch.zeros((rows, D), device=dev, dtype=torch.float8_e4m3fn)
            self.vb = torch.zeros_like(self.va)
        else:
            self.va = torch.zeros((rows, D), device=dev, dtype=torch.bfloat16)
            self.vb = None
        self.ek = torch.zeros((rows,), device=dev, dtype=torch.bfloat16)
        if v_scale is not None and 2.0 ** round(math.log2(v_scale)) != v_scale:
            raise ValueError(f"v_scale={v_scale} is not a power of two")
        self._fixed_v_scale = v_scale
        self._v_scale = float(v_scale) if (self.v8 and v_scale is not None) else 1.0
        self.seq_lens = torch.zeros((batch,), device=dev, dtype=torch.int32)
        self.lens = [0] * batch
        self.order = torch.arange(self.n_groups * self._gsub, device=dev, dtype=torch.int32)
        self.vsum = torch.zeros((self.n_groups, D), device=dev, dtype=torch.float32)
        self.vmean = torch.zeros_like(self.vsum)
        self.qa = torch.zeros((self.n_groups, self.group, D), device=dev, dtype=torch.int8)
        self.qb = torch.zeros_like(self.qa)
        self.eq = torch.ones((self.n_groups, self.group), device=dev, dtype=torch.float32)
        self.z = torch.zeros((self.n_groups, self.group), device=dev, dtype=torch.float32)
        # each row's depth below its reference
        self.cut = torch.full_like(self.z, 1e4 if depth is None else float(depth))
        if tail == "auto":
            tail = tail_rank_for(D, self.group, self.v8) if depth is not None else -1
            if page_size % tail_fit.TAIL_BLOCK or kernel == "sm100" or self._gsub > 1:
                tail = -1
        self.tail_rank = -1 if tail is None else int(tail)
        self.tail = None
        if self.tail_rank >= 0:
            if depth is None:
                raise ValueError("the tail re-enters truncated mass, and depth=None truncates nothing")
            if self.v8:
                raise ValueError("the decode tail needs a bf16 V cache; pass tail=None with v8")
            if page_size % tail_fit.TAIL_BLOCK:
                raise ValueError(f"page_size={page_size}: the tail keeps one row per 64 keys, so a page must hold whole blocks")
            if kernel == "sm100":
                raise NotImplementedError("the tail runs on the warp-level kernel: kernel='mma' or 'auto'")
            if self._gsub > 1:
                raise NotImplementedError("the tail takes row groups of at most 8 rows")
            tail_fit.check_rank(self.tail_rank, D)
            R, nblk = self.tail_rank, rows // tail_fit.TAIL_BLOCK
            self.tail = tail_fit.TailState(
                rows=torch.zeros((nblk, D), device=dev, dtype=torch.bfloat16),
                vsum=torch.zeros((nblk, D), device=dev, dtype=torch.float32),
                ysum=torch.zeros((nblk, R), device=dev, dtype=torch.float32) if R else None,
                u=torch.zeros((self.n_groups, R, D), device=dev, dtype=torch.int8) if R else None,
                vr=torch.zeros((self.n_groups, D, R), device=dev, dtype=torch.float32) if R else None,
            )
            self.kernel = "mma"
        self._refine_k_fixed = refine_k
        self._refine_v_fixed = refine_v
        # after a step, look at every row's denominator and run the flagged rows again from a
        # reference moved to their log-sum-exp (one host sync per step; kv_cache.py:704-744)
        self.check_range = bool(check_range)
        # not a reference argument: read the decode's device status word after every step (one host
        # synchronisation) and raise FoldLibraryError if a kernel gave up a bounded wait. Steps
        # under `check_range` synchronise anyway and always check.
        self.check_status = False
        self._z_given = None
        if chunk is not None and (split is not None or chunk % BN):
            raise ValueError(f"chunk={chunk} is a multiple of {BN} and replaces split")
        self.chunk = chunk
        self.den = None
        self.counts = None
        self.weight_terms = weight_terms_for(depth) if weight_terms is None else int(weight_terms)
        self._launches = {}

    @property
    def v_scale(self) -> float:
        """V's scale. The prefill leaves it on the device, and the first read
        after it is where the host takes it."""
        if torch.is_tensor(self._v_scale):
            self._v_scale = float(self._v_scale)
        return self._v_scale

    def prefill(self, q, k, v, cu_seqlens, max_seqlen=None):
        """Causal attention over `batch` prompts packed along the first axis.

        `q` is `(total, H, D)`, `k` and `v` `(total, H_KV, D)`, `cu_seqlens`
        `(batch + 1,)` int32 on the device. Returns `(total, H, D)` in q's
        dtype. The prompts replace the cache's contents.
        """
        B = self.batch
        if cu_seqlens.shape != (B + 1,):
            raise ValueError(f"cu_seqlens is ({B + 1},) for a batch of {B}")
        lens = torch.diff(cu_seqlens).tolist()
        if min(lens) < 1 or max(lens) > self.max_len:
            raise ValueError(f"prompt lengths {min(lens)}..{max(lens)} are not in 1..{self.max_len}")
        if max_seqlen is None:
            max_seqlen = max(lens)
        out, _ = attention_forward(
            q, k, v, causal=True, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen,
            softmax_scale=1.0 / math.sqrt(self.head_dim),
        )
        self.write_prompt(k, v, cu_seqlens, lens)
        return out

    def write_prompt(self, k, v, cu_seqlens, lens=None):
        """Quantise packed prompts' K and V into the cache, which they replace,
        without computing their attention. `lens` are the host lengths
        `cu_seqlens` describes."""
        if lens is None:
            lens = torch.diff(cu_seqlens).tolist()
        if len(lens) != self.batch:
            raise ValueError(f"{len(lens)} prompts for a batch of {self.batch}")
        if min(lens) < 1 or max(lens) > self.max_len:
            raise ValueError(f"prompt lengths {min(lens)}..{max(lens)} are not in 1..{self.max_len}")
        self._v_scale = write.write_prompt(
            k, v, lens, self.page_table, self.page_size, self.ka, self.kb, self.va, self.vb,
            self.ek, self.vsum, self.vmean, v_headroom=self.v_headroom,
            v_scale=self._fixed_v_scale if self.v8 else None,
        )
        self.seq_lens.copy_(torch.tensor(lens, dtype=torch.int32), non_blocking=True)
        self.lens = list(lens)
        if self.tail is not None:
            self._fit_tail(v, lens)
        self._set_order()
        self._launches.clear()

    def _fit_tail(self, v, lens):
        """Each prompt's rank map and the block rows it fills, in the units and
        pool slots the append then keeps current. A request is fitted from its
        own keys alone (plane A and the scales as the prompt writer stored them,
        read back and un-swizzled), so its tail does not depend on its batch
        (reference: kv_cache.py:300-417, `_fit_tail`)."""
        t, PS, HKV, D, TB = self.tail, self.page_size, self.n_kv_heads, self.head_dim, tail_fit.TAIL_BLOCK
        dev, R = self.device, self.tail.rank
        heads = torch.arange(HKV, device=dev)[:, None]

        def keys_of(b, n):
            """Request b's pool rows (HKV, n), plane A in channel order and scales."""
            pos = torch.arange(n, device=dev)
            pg = self.page_table[b, pos // PS].long()
            prow = (pg[None, :] * HKV + heads) * PS + (pos % PS)[None, :]
            return prow, tail_fit.plane_rows(self.ka, prow, pos % PS, D), self.ek[prow]

        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        if R:
            # every row group's D x D problem in one batched solve and one batched eigendecomposition
            mom = [tail_fit.moments(*keys_of(b, n)[1:], v[starts[b]:starts[b] + n].transpose(0, 1)) for b, n in enumerate(lens)]
            u, vr = tail_fit.rank_map(torch.cat([m[0] for m in mom]), torch.cat([m[1] for m in mom]), R)
            t.u.copy_(u)
            t.vr.copy_(vr)
        for b, n in enumerate(lens):
            prow, kint, ek = keys_of(b, n)
            vsum, cnt = tail_fit.block_sums(v[starts[b]:starts[b] + n].transpose(0, 1).float())
            cnt = cnt[None, :, None].float()
            blk = prow[:, ::TB] // TB                                              # (HKV, blocks)
            rows = vsum / cnt
            if R:
                g = slice(b * HKV, (b + 1) * HKV)
                ysum, _ = tail_fit.block_sums(tail_fit.project(kint, ek, t.u[g]))
                rows = rows - (ysum / cnt) @ t.vr[g].transpose(1, 2)
                t.ysum[blk] = ysum
            t.vsum[blk] = vsum
            t.rows[blk] = rows.to(t.rows.dtype)

    def append(self, k, v):
        """Write one token per request, `(batch, H_KV, D)` each, at its length."""
        if max(self.lens) >= self.max_len:
            raise ValueError(f"a request is at max_len={self.max_len}")
        self._step(None, k, v)
        self.lens = [x + 1 for x in self.lens]

    def attend(self, q, split=None):
        """Attention of `q` `(batch, H, D)` over the cache as it stands."""
        self._step(q, None, None)
        return self._run(q, split)

    def decode(self, q, k, v, split=None):
        """One decode step: append `k`, `v` `(batch, H_KV, D)` and attend with
        `q` `(batch, H, D)`."""
        if max(self.lens) >= self.max_len:
            raise ValueError(f"a request is at max_len={self.max_len}")
        self._step(q, k, v)
        self.lens = [x + 1 for x in self.lens]
        return self._run(q, split)

    # ---- replay and tuning helpers (src/fold_attention/kv_cache.py:441-570) ----

    def prepare_replay_decode(self, split=None, out_dtype=torch.float32):
        """A repeatable decode-only launch over the last step's front state
        (Q planes, lengths, a copy of its reference), for timing: its outputs
        and partial buffers are its own, so replaying it leaves the layer's
        state untouched. `out_dtype` is the output it writes, so a benchmark
        times the launch it scores. Returns the launch (`(out, den, counts)`)."""
        split = self._resolve_split(split)
        refine = self._refine()
        truncate = self.depth is not None
        kernel = self.kernel
        if kernel == "auto" and 2 * sum(n for n in self.lens if n >= self.SM100_MIN_KEYS) < sum(self.lens):
            kernel = "mma"
        return prepare_fold_decode(
            self.qa, self.qb, self.eq, self.ka, self.kb, self.ek, self.va, self.z.clone(), self.cut,
            split=split, truncate=truncate, refine_k=refine[0], refine_v=refine[1], v8=self.v8, v2=self.vb,
            v_scale=self.v_scale, vmean=self.vmean.clone() if truncate and self.tail is None else None,
            tail=self.tail, page_table=self.page_table,
            page_size=self.page_size, seq_lens=self.seq_lens.clone(), n_kv_heads=self.n_kv_heads, reference="given",
            weight_terms=self.weight_terms, order=self.order.clone(), out_dtype=out_dtype,
            refine_bands=refine_bands_for(self.v8, head_dim=self.head_dim, group=self.group) if self._banded() else (),
            chunk_keys=self.chunk or 0, kernel=kernel,
        )

    def prepare_replay_step(self, q, k=None, v=None, split=None, at=None):
        """A repeatable full step on private buffers, for timing under CUDA
        graphs. The returned launch writes Q's planes and, with `k` and `v`,
        the token at `at` (the current lengths by default) WITHOUT advancing
        the lengths, estimates the reference and runs the decode. Its lengths,
        reference and running V sums are its own; only the token's cache slot
        and the Q planes are rewritten, with the same values every time."""
        if (k is None) != (v is None):
            raise ValueError("k and v are both given or both left out")
        qf = q.reshape(-1, self.head_dim)
        at = (self.seq_lens if at is None else at).clone()
        appends = k is not None
        if appends and int(at.max()) >= self.max_len:
            raise ValueError(f"a replay position is at max_len={self.max_len}")
        lens_out = torch.empty_like(at)
        vsum = self.vsum.clone() if appends else self.vsum
        vmean = self.vmean.clone() if appends else self.vmean
        vsum0, vmean0 = (vsum.clone(), vmean.clone()) if appends else (None, None)
        z = self.z.clone()
        seen = lens_out if appends else at          # the lengths the decode reads
        split = self._resolve_split(split)
        refine = self._refine(int(at.max()) + int(appends))
        truncate = self.depth is not None
        out_dtype = q.dtype if q.dtype in (torch.bfloat16, torch.float16) else torch.float32
        kernel = self.kernel
        if kernel == "auto" and 2 * sum(n for n in self.lens if n >= self.SM100_MIN_KEYS) < sum(self.lens):
            kernel = "mma"
        decode = prepare_fold_decode(
            self.qa, self.qb, self.eq, self.ka, self.kb, self.ek, self.va, z, self.cut,
            split=split, truncate=truncate, refine_k=refine[0], refine_v=refine[1], v8=self.v8, v2=self.vb,
            v_scale=self.v_scale, vmean=vmean if truncate and self.tail is None else None, tail=self.tail,
            page_table=self.page_table,
            page_size=self.page_size, seq_lens=seen, n_kv_heads=self.n_kv_heads, reference="given",
            weight_terms=self.weight_terms, order=self.order.clone(), out_dtype=out_dtype,
            refine_bands=refine_bands_for(self.v8, head_dim=self.head_dim, group=self.group) if self._banded() else (),
            chunk_keys=self.chunk or 0, kernel=kernel,
        )
        shape = (self.batch, self.n_heads, self.head_dim)
        t, saved = self.tail, None
        if appends and t is not None:
            # the token's blocks, whose sums and rows every replay rewrites: keep what they hold now
            PS, HKV = self.page_size, self.n_kv_heads
            pg = self.page_table[torch.arange(self.batch, device=at.device), (at // PS).long()].long()
            blk = ((pg[:, None] * HKV + torch.arange(HKV, device=at.device)[None, :]) * PS + (at % PS)[:, None].long()) // tail_fit.TAIL_BLOCK
            blk = blk.reshape(-1)
            saved = (blk, t.vsum[blk], t.rows[blk], t.ysum[blk] if t.rank else None)

        def replay():
            if appends:   # the running sums start from the same state every replay
                vsum.copy_(vsum0)
                vmean.copy_(vmean0)
            write.step(
                qf, k, v, self.qa.view(-1, self.head_dim), self.qb.view(-1, self.head_dim), self.eq.view(-1), self.ek,
                self.page_table, self.page_size, at, self.ka, self.kb, self.va, self.vb, self.v_scale, vsum, vmean, lens_out,
            )
            if saved is not None:
                write.tail_append(v, t, self.ka, self.ek, self.page_table, self.page_size, at, 0)
            mass_z(self.qa, self.qb, self.eq, self.ka, self.ek, self.page_table, self.page_size, seen, self.n_kv_heads, z)
            o, den, counts = decode.run()
            if saved is not None:   # the token's blocks go back to what they held: the tail is the cache's own
                t.vsum[saved[0]] = saved[1]
                t.rows[saved[0]] = saved[2]
                if t.rank:
                    t.ysum[saved[0]] = saved[3]
            return o.view(shape), den, counts

        launch = ReplayStep(replay, (qf, k, v, at, lens_out, vsum, vmean, vsum0, vmean0, z, decode))
        launch.status = decode.status
        launch.decode = decode
        return launch

    def tune_split(self, candidates=(4, 6, 8, 10, 12, 14, 16, 20, 24, 32), rounds=7, reps=10):
        """Time the decode at each split in `candidates` and at the default
        one, on the cache as it stands, and keep the fastest as `split`.
        Each candidate is replayed from a CUDA graph (the host's enqueue is
        not what is timed), in rotating order across `rounds` so a drifting
        clock cancels; the replays write only buffers of their own. Returns
        `{split: us}`."""
        if self.chunk is not None:
            raise ValueError("a fixed chunk sets the split: there is nothing to tune")
        tiles = -(-(sum(self.lens) // self.batch) // BN)
        auto = self._auto_split()
        cands = sorted({auto} | {int(c) for c in candidates if -(-tiles // int(c)) >= 4})
        graphs, runs = {}, {}
        for sp in cands:
            run = self.prepare_replay_decode(sp)
            runs[sp] = run      # a graph keeps device addresses, not the tensors that own them
            for _ in range(2):
                run()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    run()
            graphs[sp] = g
        torch.cuda.synchronize()
        times = {sp: [] for sp in cands}
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for r in range(rounds):
            order = cands[r % len(cands):] + cands[: r % len(cands)]
            for sp in order:
                graphs[sp].replay()
                ev[0].record()
                for _ in range(reps):
                    graphs[sp].replay()
                ev[1].record()
                ev[1].synchronize()
                times[sp].append(ev[0].elapsed_time(ev[1]) * 1e3 / reps)
        med = {sp: sorted(t)[len(t) // 2] for sp, t in times.items()}
        self.split = min(med, key=lambda sp: med[sp])
        self._launches.clear()
        return med

    # ---- internals -------------------------------------------------------

    def _set_order(self):
        """Which row group each grid slot takes; it changes no bit. Without a
        chunk a CTA walks a whole request, so the longest requests get the
        lowest slots: a long request placed late has nothing behind it to
        backfill its tail. Under a fixed chunk every CTA's work is bounded, and
        the short requests go first instead: their tiles hold the most refined
        keys and are the slowest, and should not be what the grid ends on."""
        sign = 1 if self.chunk else -1
        rank = sorted(range(self.batch), key=lambda b: (sign * self.lens[b], b))
        order = [(r * self.n_kv_heads + h) * self._gsub + s for r in rank for h in range(self.n_kv_heads) for s in range(self._gsub)]
        self.order.copy_(torch.tensor(order, dtype=torch.int32), non_blocking=True)

    def _auto_split(self):
        mean = sum(self.lens) / self.batch
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        sm100 = self.kernel == "sm100" or (
            self.kernel == "auto" and 2 * sum(n for n in self.lens if n >= self.SM100_MIN_KEYS) >= sum(self.lens))
        return pick_split(self.n_groups * self._gsub, max(1, int(mean)), max_len=max(self.lens), sms=sms,
                          resident=1.5 if sm100 else 3)

    def _resolve_split(self, split):
        if self.chunk is not None:
            # every request is cut at the same key offsets whatever its batch;
            # the batch's longest request only sets how many splits run
            return max(1, -(-max(self.lens) // self.chunk))
        if split is None:
            split = self.split
        if split is None:
            split = self._auto_split()
        return split

    def _banded(self):
        """Whether the kernel picks the dense gates from each request's length."""
        return self.depth is None and self._refine_k_fixed is None and self._refine_v_fixed is None

    def _refine(self, seq_len=None):
        if self._banded():
            seq_len = 1
        elif seq_len is None:
            seq_len = max(self.lens)
        rk, rv = refine_for(
            self.depth, self.v8, seq_len=seq_len, head_dim=self.head_dim, group=self.group,
            tail=self.tail_rank >= 0,
        )
        if self._refine_k_fixed is not None:
            rk = self._refine_k_fixed
        if self._refine_v_fixed is not None:
            rv = self._refine_v_fixed
        return rk, rv

    def refine_gates(self):
        """Each request's refine gates at its current length, `(refine_k,
        refine_v)` as `(batch,)` float32 depths below Z."""
        rk, rv = self._refine()
        n = torch.tensor(self.lens, dtype=torch.float32)
        if not self._banded():
            return torch.full_like(n, float(rk)), torch.full_like(n, float(rv))
        e0, e1, rk1, rk2, rv1, rv2 = refine_bands_for(self.v8, head_dim=self.head_dim, group=self.group)
        rk_t = torch.where(n > e1, rk2, torch.where(n > e0, rk1, float(rk)))
        rv_t = torch.where(n > e1, rv2, torch.where(n > e0, rv1, float(rv)))
        return rk_t, rv_t

    def _launch(self, split, out_dtype, given=False):
        """The step's decode launch; `given`: the one that reads `_z_given` instead of the mass reference."""
        refine = self._refine()
        kernel, short = self.kernel, 0
        if kernel == "auto":
            if self.chunk and self.mix_kernels:
                # the slot order is by length (_set_order): the short requests are its first slots
                short = self.n_kv_heads * sum(1 for n in self.lens if n < self.SM100_MIN_KEYS)
            elif 2 * sum(n for n in self.lens if n >= self.SM100_MIN_KEYS) < sum(self.lens):
                kernel = "mma"
        key = (split, out_dtype, refine, kernel, short, given)
        if given and self._z_given is None:
            self._z_given = torch.empty_like(self.z)
        if key not in self._launches:
            truncate = self.depth is not None
            self._launches[key] = prepare_fold_decode(
                self.qa, self.qb, self.eq, self.ka, self.kb, self.ek, self.va,
                self._z_given if given else self.z, self.cut,
                split=split, truncate=truncate, refine_k=refine[0], refine_v=refine[1],
                v8=self.v8, v2=self.vb, v_scale=self.v_scale,
                vmean=self.vmean if truncate and self.tail is None else None, tail=self.tail,
                page_table=self.page_table,
                page_size=self.page_size, seq_lens=self.seq_lens, n_kv_heads=self.n_kv_heads,
                reference="given", weight_terms=self.weight_terms, order=self.order,
                out_dtype=out_dtype,
                refine_bands=(
                    refine_bands_for(self.v8, head_dim=self.head_dim, group=self.group)
                    if self._banded() else ()
                ),
                chunk_keys=self.chunk or 0,
                kernel=kernel,
                short_slots=short,
            )
        return self._launches[key]

    def _step(self, q, k, v):
        """The step's front: Q's planes, the appended token, then each row's
        reference Z from the cache as it now stands."""
        qf = None if q is None else q.reshape(-1, self.head_dim)
        if k is not None and (k.shape != (self.batch, self.n_kv_heads, self.head_dim) or v.shape != k.shape):
            raise ValueError(f"k and v are ({self.batch}, {self.n_kv_heads}, {self.head_dim})")
        if qf is not None and qf.shape[0] != self.batch * self.n_heads:
            raise ValueError(f"q is ({self.batch}, {self.n_heads}, {self.head_dim})")
        write.step(
            qf, k, v, self.qa.view(-1, self.head_dim), self.qb.view(-1, self.head_dim),
            self.eq.view(-1), self.ek, self.page_table, self.page_size, self.seq_lens,
            self.ka, self.kb, self.va, self.vb, self.v_scale, self.vsum, self.vmean, self.seq_lens,
        )
        if k is not None and self.tail is not None:
            write.tail_append(v, self.tail, self.ka, self.ek, self.page_table, self.page_size, self.seq_lens, 1)
        if q is not None:
            mass_z(self.qa, self.qb, self.eq, self.ka, self.ek, self.page_table, self.page_size,
                   self.seq_lens, self.n_kv_heads, self.z)

    def _run(self, q, split):
        split = self._resolve_split(split)
        shape = (self.batch, self.n_heads, self.head_dim)
        out_dtype = q.dtype if q.dtype in (torch.bfloat16, torch.float16) else torch.float32
        # a fresh tensor per step: the caller may hold every step's output
        out = torch.empty((self.n_groups, self.group, self.head_dim), device=q.device, dtype=out_dtype)
        launch = self._launch(split, out_dtype)
        o, self.den, self.counts = launch.run(out=out)
        if self.check_range or self.check_status:
            launch.check()
        if self.check_range:
            bad = self._out_of_range(o, self.den)
            if bool(bad.any()):
                o, self.den, self.counts = self._rerun(bad, self.den, split, out_dtype, out)
        return o.view(shape).to(q.dtype)

    def _range_window(self):
        """`(lo, hi)` for a row's denominator `2^(LSE - Z)`: under `hi` no weight or sum overflows
        (the reference's 8-bit V path carries 2^64 in its weights, which lowers it); over `lo` Z is
        within a binade of the log-sum-exp, so a gate or cut at depth T below Z is at least T - 1
        below the row's mass (kv_cache.py:704-713)."""
        return 0.5, 2.0 ** (60 if self.v8 else 100)

    def _out_of_range(self, o, den):
        lo, hi = self._range_window()
        ok = (den >= lo) & (den <= hi)
        ok &= torch.isfinite(o.view(self.n_groups, self.group, self.head_dim)).all(-1)
        return ~ok

    def _rerun(self, bad, den, split, out_dtype, out):
        """The step's decode again with every flagged row's reference moved to its log-sum-exp
        (`Z + log2(den)`); an empty or infinite denominator moves it by 64 binades and tries again,
        four times at most (kv_cache.py:721-744)."""
        z = self.z.clone()
        launch = self._launch(split, out_dtype, given=True)
        tiny = torch.finfo(torch.float32).tiny
        for _ in range(4):
            shift = torch.where(
                torch.isfinite(den) & (den > 0), torch.log2(den.clamp_min(tiny)),
                torch.where(den == 0, torch.full_like(den, -64.0), torch.full_like(den, 64.0)))
            z = torch.where(bad, z + shift, z)
            self._z_given.copy_(z)
            o, den2, counts = launch.run(out=out)
            launch.check()
            bad2 = self._out_of_range(o, den2)
            if not bool(bad2.any()):
                return o, den2, counts
            bad, den = bad2, den2
        raise FloatingPointError("a row's reference left the exponent range after four moves")
