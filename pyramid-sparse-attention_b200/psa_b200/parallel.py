"""Head sharding of the PSA layer across the GPUs of one node.

Every stage of the layer is independent per (batch, head), so ranks own disjoint heads and no collective runs inside
the layer.  When the surrounding model keeps activations sequence-sharded ([S/P, H, D] per rank), one all-to-all turns
them into head shards ([H/P, S, D]) before the layer and one turns the output back (Ulysses-style).  The collective is
NCCL's (torch.distributed.all_to_all_single) on GPUs and gloo's in the CPU tests; kernels only ever read local memory.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class HeadShard:
    def __init__(self, world: int, rank: int, heads: int, seq: int, head_dim: int):
        if heads % world:
            raise ValueError(f"{heads} heads do not divide over {world} ranks")
        if seq % world:
            raise ValueError(f"{seq} tokens do not divide over {world} ranks")
        self.world, self.rank, self.heads, self.seq, self.head_dim = world, rank, heads, seq, head_dim
        self.heads_per_rank = heads // world
        self.tokens_per_rank = seq // world
        self.head_range = (rank * self.heads_per_rank, (rank + 1) * self.heads_per_rank)

    def to_head_sharded(self, x: torch.Tensor) -> torch.Tensor:
        """[n, S/P, H, D] (n stacked tensors, e.g. q/k/v) on every rank -> [n, H/P, S, D]."""
        n, sl, H, D = x.shape
        hp, P = self.heads_per_rank, self.world
        if P == 1:
            return x.permute(0, 2, 1, 3).contiguous()
        send = x.view(n, sl, P, hp, D).permute(2, 0, 3, 1, 4).contiguous()           # [P_dst, n, hp, S/P, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return recv.permute(1, 2, 0, 3, 4).reshape(n, hp, P * sl, D)                  # [n, hp, S, D]

    def to_seq_sharded(self, o: torch.Tensor) -> torch.Tensor:
        """[H/P, S, D] -> [H, S/P, D] (head-major rows of this rank's tokens)."""
        hp, S, D = o.shape
        P = self.world
        sl = S // P
        if P == 1:
            return o
        send = o.view(hp, P, sl, D).permute(1, 0, 2, 3).contiguous()                  # [P_dst, hp, S/P, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return recv.view(P * hp, sl, D)

    # ------------------------------------------------------------------ chunked variants (for overlap)
    def chunks(self, n_chunks: int):
        """Split this rank's heads into n_chunks equal groups; returns [(first_local_head, heads_in_chunk), ...]."""
        n_chunks = max(1, min(n_chunks, self.heads_per_rank))
        while self.heads_per_rank % n_chunks:
            n_chunks -= 1
        hc = self.heads_per_rank // n_chunks
        return [(c * hc, hc) for c in range(n_chunks)]

    def to_head_sharded_chunk(self, x: torch.Tensor, first: int, count: int) -> torch.Tensor:
        """Like to_head_sharded, but only local heads [first, first+count) of every rank: [n, S/P, H, D] -> [n, count, S, D]."""
        n, sl, H, D = x.shape
        hp, P = self.heads_per_rank, self.world
        send = x.view(n, sl, P, hp, D)[:, :, :, first:first + count].permute(2, 0, 3, 1, 4).contiguous()   # [P, n, count, S/P, D]
        if P == 1:
            return send[0].reshape(n, count, sl, D)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        return recv.permute(1, 2, 0, 3, 4).reshape(n, count, P * sl, D)

    def to_seq_sharded_chunk(self, o: torch.Tensor, first: int, out: torch.Tensor) -> None:
        """[count, S, D] of local heads [first, first+count) -> rows of out [H, S/P, D] (every rank's same local heads)."""
        count, S, D = o.shape
        P, hp = self.world, self.heads_per_rank
        sl = S // P
        if P == 1:
            out[first:first + count] = o
            return
        send = o.view(count, P, sl, D).permute(1, 0, 2, 3).contiguous()                 # [P_dst, count, S/P, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        out.view(P, hp, sl, D)[:, first:first + count] = recv
