"""CPU (gloo, world_size 2 to 8): the sequence-sharded <-> head-sharded reshuffles used around the PSA layer."""
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


def test_peer_exchange_address_contract_matches_the_reshuffle():
    """The per-row address formulas of the peer-memory exchange (push, pull, scattered output) applied to emulated rank
    buffers give exactly the head-sharded / sequence-sharded layouts of the all-to-all reshuffle."""
    sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
    from psa_b200.parallel import push_destination, pull_source
    world, H, S, D = 4, 8, 24, 2
    hp, sl = H // world, S // world
    g = torch.Generator().manual_seed(3)
    full = torch.randn(S, H, D, generator=g)
    seq_shards = [full[r * sl:(r + 1) * sl] for r in range(world)]                     # [S/P, H, D] per rank
    want_head_shards = [full[:, r * hp:(r + 1) * hp].permute(1, 0, 2) for r in range(world)]   # [H/P, S, D] per rank
    pushed = [torch.zeros(hp, S, D) for _ in range(world)]
    for r in range(world):
        for t in range(sl):
            for h in range(H):
                owner, hl, tok = push_destination(r, t, h, sl, hp)
                pushed[owner][hl, tok] = seq_shards[r][t, h]
    pulled = [torch.zeros(hp, S, D) for _ in range(world)]
    outs = [torch.zeros(sl, H, D) for _ in range(world)]
    for r in range(world):
        for hl in range(hp):
            for tok in range(S):
                owner, tl, h = pull_source(tok, hl, r * hp, sl)
                pulled[r][hl, tok] = seq_shards[owner][tl, h]
                outs[owner][tl, h] = want_head_shards[r][hl, tok] * 3.0              # "forward output" scattered home
    for r in range(world):
        assert torch.equal(pushed[r], want_head_shards[r]) and torch.equal(pulled[r], want_head_shards[r])
        assert torch.equal(outs[r], seq_shards[r] * 3.0)


def _grid_worker(rank, world, port, H, S, D, bm, ret):
    sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from psa_b200.parallel import GridShard
    g = torch.Generator().manual_seed(11)
    full = torch.randn(3, S, H, D, generator=g)
    sl = S // world
    local = full[:, rank * sl:(rank + 1) * sl].contiguous()
    gs = GridShard(world, rank, H, S, D, block_m=bm)
    q, k, v = gs.to_grid(local)
    h0, h1 = gs.head_range()
    r0, r1 = gs.query_range()
    ok_in = (torch.equal(q, full[0, r0:r1, h0:h1].permute(1, 0, 2)) and torch.equal(k, full[1, :, h0:h1].permute(1, 0, 2))
             and torch.equal(v, full[2, :, h0:h1].permute(1, 0, 2)))
    o = q * 2.0 + v[:, r0:r1]                                     # any row-wise function of the part
    back = gs.to_seq(o)
    expect = (full[0] * 2.0 + full[2])[rank * sl:(rank + 1) * sl].permute(1, 0, 2)
    ret[rank] = (ok_in, torch.equal(back, expect), r0 % bm == 0)
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world,H,S,bm", [(4, 6, 4 * 37, 16), (8, 12, 8 * 45, 32), (2, 4, 60, 16)])
def test_grid_shard_head_groups_times_query_parts(world, H, S, bm):
    """Head counts that do not divide the rank count: gcd(H, world) head groups x world/gcd query parts; the reshuffles
    from and to sequence shards are exact, and the parts are cut on query-block boundaries even when a rank's token
    shard straddles the cut."""
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 31000 + (os.getpid() + world) % 2000
    mp.spawn(_grid_worker, args=(world, port, H, S, 4, bm, ret), nprocs=world, join=True)
    assert all(ret[r] == (True, True, True) for r in range(world)), dict(ret)


def test_grid_shard_layout_for_12_heads_on_8_ranks():
    sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
    from psa_b200.parallel import GridShard
    parts = [GridShard(8, r, 12, 32760, 128) for r in range(8)]
    assert parts[0].groups == 4 and parts[0].parts == 2 and parts[0].heads_per_rank == 3
    assert [p.head_range() for p in parts] == [(0, 3), (0, 3), (3, 6), (3, 6), (6, 9), (6, 9), (9, 12), (9, 12)]
    assert parts[0].query_range() == (0, 16384) and parts[1].query_range() == (16384, 32760)
    # when the heads divide, it is the plain head sharding: one part covering every query block
    plain = GridShard(8, 5, 40, 75600, 128)
    assert plain.parts == 1 and plain.head_range() == (25, 30) and plain.query_range() == (0, 75600)
