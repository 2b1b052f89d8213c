"""Host logic of the multi-GPU sharding, on CPU ranks (gloo, world size 2)."""

import math
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fold_attention_b200 import parallel
from oracle import cache_format as cf


def test_units_cover_the_batch_once_and_keep_groups_whole():
    for B, HKV, W in ((4, 32, 8), (4, 8, 8), (3, 5, 4), (1, 1, 2)):
        seen = set()
        for r in range(W):
            for b, (lo, hi) in parallel.backward_units(B, HKV, W, r).items():
                for h in range(lo, hi):
                    assert (b, h) not in seen
                    seen.add((b, h))
        assert len(seen) == B * HKV
    sizes = [len(parallel.split_even(10, 4, r)) for r in range(4)]
    assert sizes == [3, 3, 2, 2]


def test_balance_is_a_partition_and_is_balanced():
    rng = np.random.default_rng(0)
    lens = np.exp(rng.uniform(math.log(4096), math.log(131072), 256)).astype(int).tolist()
    parts = parallel.balance(lens, 8)
    assert sorted(i for p in parts for i in p) == list(range(256))
    loads = [sum(lens[i] for i in p) for p in parts]
    assert max(loads) / (sum(loads) / 8) < 1.03


def test_v_scale_rule_is_the_writers():
    for amax in (0.3, 1.0, 3.7, 20.0, 448.0, 1e-12):
        assert parallel.v_scale_from_amax(amax, 2.0) == float(cf.v_scale_rule(amax, 2.0))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(7)
    v = torch.randn(64, 8, 16, generator=g) * 3
    v[5, 1, 2] = 41.0
    mine = v[list(parallel.split_even(64, world, rank))]
    scale = parallel.shared_v_scale(mine, 2.0)
    rows = parallel.gather_rows(mine)
    ret[rank] = (scale, torch.equal(rows, v))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_agree_on_the_v_scale_and_gather_in_rank_order():
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    g = torch.Generator().manual_seed(7)
    v = torch.randn(64, 8, 16, generator=g) * 3
    v[5, 1, 2] = 41.0
    want = parallel.v_scale_from_amax(float(v.abs().amax()), 2.0)
    assert ret[0][0] == ret[1][0] == want
    assert ret[0][1] and ret[1][1]
