"""CPU, world_size 2 (gloo): the sequence-sharded <-> head-sharded reshuffle used around the PSA layer."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, H, S, D, ret):
    sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from psa_b200.parallel import HeadShard
    g = torch.Generator().manual_seed(7)
    full = torch.randn(3, S, H, D, generator=g)                  # q, k, v of the whole layer, [3, S, H, D]
    sl = S // world
    local = full[:, rank * sl:(rank + 1) * sl].contiguous()      # what a sequence-parallel model holds
    hs = HeadShard(world, rank, H, S, D)
    x = hs.to_head_sharded(local)                                # [3, H/world, S, D]
    h0, h1 = hs.head_range
    expect = full[:, :, h0:h1].permute(0, 2, 1, 3)
    ok1 = torch.equal(x, expect)
    o = x[0] * 2.0 + x[2]                                        # any per-head function of the head shard
    back = hs.to_seq_sharded(o)                                  # [H, S/world, D]
    expect_back = (full[0] * 2.0 + full[2])[rank * sl:(rank + 1) * sl].permute(1, 0, 2)
    ok2 = torch.equal(back, expect_back)
    ret[rank] = (ok1, ok2)
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_all_to_all_reshuffle_round_trip_world2():
    world, H, S, D = 2, 6, 40, 8
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, H, S, D, ret), nprocs=world, join=True)
    assert all(ret[r] == (True, True) for r in range(world)), dict(ret)


def test_head_shard_validation():
    sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
    from psa_b200.parallel import HeadShard
    with pytest.raises(ValueError):
        HeadShard(8, 0, 12, 32760, 128)          # 12 heads do not divide over 8 ranks
    with pytest.raises(ValueError):
        HeadShard(4, 0, 12, 32761, 128)          # tokens must divide too
    hs = HeadShard(8, 3, 40, 75600, 128)
    assert hs.head_range == (15, 20) and hs.tokens_per_rank == 9450
