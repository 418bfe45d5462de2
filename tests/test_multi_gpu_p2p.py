"""Peer-memory head exchange on two real GPUs: the pull kernel against the NCCL all-to-all it replaces, and the
scattering forward against the local forward followed by the return all-to-all.  Runs as two child processes; skipped
on boxes with fewer than two GPUs."""
import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "pyramid-sparse-attention_b200"))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, H: int, S: int, D: int, q):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        import psa_b200
        from psa_b200 import ops
        from psa_b200.parallel import HeadShard, PeerExchange
        import cases as C

        dtype = torch.bfloat16
        sl, hp = S // world, H // world
        full = [C.randn(900 + i, (H, S, D), dtype, smooth=8 if i < 2 else 0) for i in range(3)]      # q, k, v: [H, S, D]
        mine = torch.stack([x[:, rank * sl:(rank + 1) * sl].permute(1, 0, 2) for x in full]).contiguous().to(dev)   # [3, S/P, H, D]

        ex = PeerExchange(H, S, D, dtype, dev)
        ex.q.copy_(mine[0]); ex.k.copy_(mine[1]); ex.v.copy_(mine[2])
        torch.cuda.synchronize()
        dist.barrier()

        shard = HeadShard(world, rank, H, S, D)
        ref = shard.to_head_sharded(mine)                                  # NCCL: [3, H/P, S, D]
        got = ex.pull()
        assert torch.equal(got, ref), "pull differs from the all-to-all"
        want = torch.stack([x[rank * hp:(rank + 1) * hp] for x in full]).to(dev)
        assert torch.equal(got, want), "pull differs from the source data"
        part = ex.pull(first=1, count=hp - 1)
        assert torch.equal(part, ref[:, 1:])
        for parity in (0, 1):
            recv = ex.push(parity)
            dist.barrier()                              # enqueued after the push on every rank
            torch.cuda.synchronize()
            assert torch.equal(recv, ref), "push differs from the all-to-all"

        # scattering forward == local forward + return all-to-all
        bm, bn, tn = 128, 64, 32
        qq, kk, vv = got[0].unsqueeze(0), got[1].unsqueeze(0), got[2].unsqueeze(0)
        torch.manual_seed(7)
        iq = ops.draw_sample_indices(1, hp, bm, bm // 4, dev)
        ik = ops.draw_sample_indices(1, hp, bn, bn // 4, dev)
        po = ops.block_scores(qq, kk, iq, ik, bm, bn)
        mask = ops.assign_levels(po, C.DEFAULT_RATIOS, "topk_newtype", bn, tn)
        imgs = ops.pyramid_kv_images(kk, vv, bn)
        # sampled rows pushed ahead of the full rows give the same scores
        torch.manual_seed(7)
        iq_all = ops.draw_sample_indices(1, H, bm, bm // 4, dev)
        ik_all = ops.draw_sample_indices(1, H, bn, bn // 4, dev)
        ex.enable_sample_push(bm, bn)
        for parity in (0, 1):
            ex.push_samples(parity, iq_all, ik_all)
            dist.barrier()
            torch.cuda.synchronize()
            po_s = ex.scores_from_samples(parity)
            po_l = ops.block_scores(qq, kk, iq_all[:, rank * hp:(rank + 1) * hp].contiguous(),
                                    ik_all[:, rank * hp:(rank + 1) * hp].contiguous(), bm, bn)
            assert torch.equal(po_s, po_l), "scores from pushed samples differ"
        # the peer-reading variants of the score and image kernels see the same rows
        assert torch.equal(ex.block_scores(iq, ik, bm, bn), po), "scores from peer rows differ"
        peer_imgs = ex.pyramid_images(bn, max_blocks=24)
        assert torch.equal(peer_imgs.kimg, imgs.kimg) and torch.equal(peer_imgs.vimg, imgs.vimg), "images from peer rows differ"
        local = ops.psa_forward(qq, kk, vv, mask, bm, bn, tn, pyramid=imgs)
        back = shard.to_seq_sharded(local[0])                              # [H, S/P, D]
        ex.o.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        status = ex.forward_scatter(qq, imgs, mask, bm, bn, tn)
        torch.cuda.synchronize()
        dist.barrier()
        assert int(status.item()) == 0
        assert torch.equal(ex.o.permute(1, 0, 2), back), "scattered output differs from forward + all-to-all"
        dist.barrier()
        ex.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001 - the parent reports it
        import traceback
        q.put((rank, "".join(traceback.format_exception(type(e), e, e.__traceback__))[-3000:]))


@pytest.mark.parametrize("H,S,D", [(4, 1024, 128), (6, 900, 64)])
def test_pull_and_scatter_match_the_collective(H, S, D):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, H, S, D, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    for _ in procs:
        r, msg = q.get(timeout=240)
        results[r] = msg
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results


def _grid_worker(rank: int, world: int, port: int, H: int, S: int, D: int, q):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        import psa_b200
        from psa_b200 import ops
        from psa_b200.parallel import GridShard
        import cases as C

        dtype = torch.bfloat16
        sl = S // world
        full = [C.randn(700 + i, (H, S, D), dtype, smooth=8 if i < 2 else 0) for i in range(3)]      # q, k, v: [H, S, D]
        mine = torch.stack([x[:, rank * sl:(rank + 1) * sl].permute(1, 0, 2) for x in full]).contiguous().to(dev)   # [3, S/P, H, D]
        grid = GridShard(world, rank, H, S, D, 128)
        qp, kk, vv = grid.to_grid(mine)
        h0, h1 = grid.head_range()
        r0, r1 = grid.query_range()
        assert r0 % 128 == 0
        cfg = psa_b200.PSAConfig(mask_ratios=C.DEFAULT_RATIOS)
        torch.manual_seed(5)                                       # the same draw on every rank, sliced by head group
        iq = ops.draw_sample_indices(1, H, 128, 32, dev)
        ik = ops.draw_sample_indices(1, H, 64, 16, dev)
        mod = psa_b200.PSAAttention(cfg)
        part = mod(qp.unsqueeze(0), kk.unsqueeze(0), vv.unsqueeze(0), idx_q=iq[:, h0:h1].contiguous(), idx_k=ik[:, h0:h1].contiguous())
        back = grid.to_seq(part[0])                                # [H, S/P, D]: all heads of this rank's tokens
        # the same layer on one GPU, whole heads and all query blocks
        whole = mod(full[0].unsqueeze(0).to(dev), full[1].unsqueeze(0).to(dev), full[2].unsqueeze(0).to(dev), idx_q=iq, idx_k=ik)
        want = whole[0, :, rank * sl:(rank + 1) * sl]
        assert torch.equal(back, want), "2-D partition differs from the single-GPU layer"
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001 - the parent reports it
        import traceback
        q.put((rank, "".join(traceback.format_exception(type(e), e, e.__traceback__))[-3000:]))


@pytest.mark.parametrize("H,S,D", [(3, 2 * 1000, 128), (1, 2 * 700, 64)])
def test_head_group_times_query_range_split_is_bit_identical_to_one_gpu(H, S, D):
    """Head counts that do not divide the GPU count: gcd(H, 2) = 1 head group x 2 query-block ranges (the cut falls inside
    rank 1's token shard).  Each rank attends its query range against all keys; the reassembled output must equal the
    single-GPU layer bit for bit."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_grid_worker, args=(r, 2, port, H, S, D, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {}
    for _ in procs:
        r, msg = q.get(timeout=240)
        results[r] = msg
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results
