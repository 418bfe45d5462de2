"""Head sharding of the PSA layer across the GPUs of one node.

Every stage of the layer is independent per (batch, head), so ranks own disjoint heads and no collective runs inside
the layer.  When the surrounding model keeps activations sequence-sharded ([S/P, H, D] per rank), one all-to-all turns
them into head shards ([H/P, S, D]) before the layer and one turns the output back (Ulysses-style).

Two implementations of that exchange:
  * HeadShard: the collective (torch.distributed.all_to_all_single: NCCL on GPUs, gloo in the CPU tests).
  * PeerExchange: no collective.  Every rank maps its peers' q/k/v/o buffers (CUDA IPC), pulls the rows of its heads
    with a copy kernel that reads peer memory directly, and the attention forward stores its output rows straight into
    the owning peer's buffer.  The host orders the steps with barriers; no kernel waits on another GPU.
"""
from __future__ import annotations

import ctypes as C

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


class GridShard:
    """2-D partition for head counts that do not divide over the ranks (e.g. 12 heads on 8 GPUs = 4 head groups x 2
    query ranges).  With G = gcd(heads, world) head groups of heads/G heads each and world/G query parts per group, rank
    r works on head group r // parts and query part r % parts.  Query blocks are independent rows of the layer
    (src/psa_triton/kernels/psa_kernel.py:173,198), so a part is just the attention call on a slice of q: it needs q
    of its own block range only, but k and v (hence the pooled pyramid and the k samples) of ALL tokens, which are
    rebuilt on every rank of the group.  Parts are cut on block_m boundaries, so every query block - and with it every
    score row, mask row and output row - is the one a single GPU computes.

    to_grid / to_seq are the reshuffles from and to sequence-sharded activations ([S/P, H, D] per rank), one
    all_to_all_single each with uneven splits (NCCL on GPUs, gloo in the CPU tests)."""

    def __init__(self, world: int, rank: int, heads: int, seq: int, head_dim: int, block_m: int = 128):
        import math
        if seq % world:
            raise ValueError(f"{seq} tokens do not divide over {world} ranks")
        self.world, self.rank, self.heads, self.seq, self.head_dim, self.block_m = world, rank, heads, seq, head_dim, block_m
        self.groups = math.gcd(heads, world)
        self.parts = world // self.groups
        self.heads_per_rank = heads // self.groups
        self.tokens_per_rank = seq // world
        mq = -(-seq // block_m)
        if self.parts > mq:
            raise ValueError(f"{self.parts} query parts need at least as many query blocks (have {mq})")
        per = -(-mq // self.parts)
        self._cuts = [min(seq, p * per * block_m) for p in range(self.parts)] + [seq]     # token boundaries of the parts

    def coords(self, rank: int):
        """(head group, query part) of a rank."""
        return rank // self.parts, rank % self.parts

    def head_range(self, rank: int = None):
        g, _ = self.coords(self.rank if rank is None else rank)
        return g * self.heads_per_rank, (g + 1) * self.heads_per_rank

    def query_range(self, rank: int = None):
        """Token range [r0, r1) of the rank's query part; r0 is a multiple of block_m."""
        _, part = self.coords(self.rank if rank is None else rank)
        return self._cuts[part], self._cuts[part + 1]

    def _overlap(self, token_owner: int, part_rank: int):
        """Tokens of rank `token_owner`'s sequence shard that lie in rank `part_rank`'s query part, as a global range."""
        t0, t1 = token_owner * self.tokens_per_rank, (token_owner + 1) * self.tokens_per_rank
        r0, r1 = self.query_range(part_rank)
        lo, hi = max(t0, r0), min(t1, r1)
        return (lo, hi) if lo < hi else (lo, lo)

    def to_grid(self, x: torch.Tensor):
        """[3, S/P, H, D] (this rank's tokens of q, k, v) -> (q_part [hp, r1-r0, D], k [hp, S, D], v [hp, S, D])."""
        n, sl, H, D = x.shape
        assert n == 3 and sl == self.tokens_per_rank and H == self.heads
        hp, P = self.heads_per_rank, self.world
        t0 = self.rank * sl
        send, send_sizes = [], []
        for d in range(P):
            h0, h1 = self.head_range(d)
            lo, hi = self._overlap(self.rank, d)
            pieces = [x[1, :, h0:h1].permute(1, 0, 2).reshape(-1), x[2, :, h0:h1].permute(1, 0, 2).reshape(-1),
                      x[0, lo - t0:hi - t0, h0:h1].permute(1, 0, 2).reshape(-1)]
            send.append(torch.cat(pieces))
            send_sizes.append(int(send[-1].numel()))
        recv_sizes = []
        for src in range(P):
            lo, hi = self._overlap(src, self.rank)
            recv_sizes.append((2 * sl + (hi - lo)) * hp * D)
        send_buf = torch.cat(send)
        recv_buf = torch.empty(sum(recv_sizes), dtype=x.dtype, device=x.device)
        if P == 1:
            recv_buf.copy_(send_buf)
        else:
            dist.all_to_all_single(recv_buf, send_buf, output_split_sizes=recv_sizes, input_split_sizes=send_sizes)
        r0, r1 = self.query_range()
        k = torch.empty((hp, self.seq, D), dtype=x.dtype, device=x.device)
        v = torch.empty_like(k)
        q = torch.empty((hp, r1 - r0, D), dtype=x.dtype, device=x.device)
        off = 0
        for src in range(P):
            lo, hi = self._overlap(src, self.rank)
            kv = sl * hp * D
            k[:, src * sl:(src + 1) * sl] = recv_buf[off:off + kv].view(hp, sl, D)
            v[:, src * sl:(src + 1) * sl] = recv_buf[off + kv:off + 2 * kv].view(hp, sl, D)
            if hi > lo:
                q[:, lo - r0:hi - r0] = recv_buf[off + 2 * kv:off + recv_sizes[src]].view(hp, hi - lo, D)
            off += recv_sizes[src]
        return q, k, v

    def to_seq(self, o_part: torch.Tensor) -> torch.Tensor:
        """[hp, r1-r0, D] (output rows of this rank's query part and heads) -> [H, S/P, D] (all heads of this rank's
        tokens)."""
        hp, rows, D = o_part.shape
        r0, r1 = self.query_range()
        assert hp == self.heads_per_rank and rows == r1 - r0
        P, sl = self.world, self.tokens_per_rank
        send, send_sizes = [], []
        for d in range(P):                                   # d owns tokens [d*sl, (d+1)*sl)
            lo, hi = self._overlap(d, self.rank)
            send.append(o_part[:, lo - r0:hi - r0].reshape(-1))
            send_sizes.append(int(send[-1].numel()))
        recv_sizes = []
        for src in range(P):
            lo, hi = self._overlap(self.rank, src)
            recv_sizes.append((hi - lo) * hp * D)
        send_buf = torch.cat(send)
        recv_buf = torch.empty(sum(recv_sizes), dtype=o_part.dtype, device=o_part.device)
        if P == 1:
            recv_buf.copy_(send_buf)
        else:
            dist.all_to_all_single(recv_buf, send_buf, output_split_sizes=recv_sizes, input_split_sizes=send_sizes)
        out = torch.empty((self.heads, sl, D), dtype=o_part.dtype, device=o_part.device)
        t0 = self.rank * sl
        off = 0
        for src in range(P):
            lo, hi = self._overlap(self.rank, src)
            if hi > lo:
                h0, h1 = self.head_range(src)
                out[h0:h1, lo - t0:hi - t0] = recv_buf[off:off + recv_sizes[src]].view(hp, hi - lo, D)
            off += recv_sizes[src]
        return out


# Address contract of the peer exchange (what psa_push_heads / psa_pull_heads / psa_fwd_images_scatter compute per row).
def push_destination(rank: int, t_local: int, head: int, tokens_per_rank: int, heads_per_rank: int):
    """Row (t_local, head) of rank `rank`'s [S/P, H, D] buffer goes to -> (owner rank, local head, global token)."""
    return head // heads_per_rank, head % heads_per_rank, rank * tokens_per_rank + t_local


def pull_source(token: int, local_head: int, head0: int, tokens_per_rank: int):
    """Row (local_head, token) of a head owner's [H/P, S, D] buffer comes from -> (owner rank, local token, global head);
    the scattering forward stores output row (local_head, token) to the same place of the owner's o buffer."""
    return token // tokens_per_rank, token % tokens_per_rank, head0 + local_head


class _DeviceBuffer:
    """A raw device allocation exposed to torch through the CUDA array interface."""

    def __init__(self, ptr: int, shape, dtype: torch.dtype):
        typestr = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4"}[dtype]
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


def _as_tensor(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    t = torch.as_tensor(_DeviceBuffer(ptr, shape, dtype), device=device)
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


class PeerExchange:
    """Exchange buffers of one attention layer, mapped into every rank of the node.

    Each rank owns q, k, v and o buffers of shape [S/P, H, D] (its tokens, all heads), allocated by the library so that
    an IPC handle exists for them.  After construction:
      * `q`, `k`, `v`, `o` are torch views of this rank's own buffers (the surrounding model writes q/k/v, reads o);
      * `pull()` returns this rank's heads of all tokens, [3, H/P, S, D], read from the peers' buffers;
      * `push(parity)` is the same exchange driven by the senders (posted stores into the peers' receive buffers);
      * `forward_scatter(...)` runs the tile-image forward and stores every output row into the owner's `o`.
    The caller places a barrier between "all ranks wrote q/k/v" and pull(), and between forward_scatter() and reading o.
    """

    def __init__(self, heads: int, seq: int, head_dim: int, dtype: torch.dtype, device, group=None, push_buffers: bool = True):
        from ._lib import lib, check
        self.lib, self.check = lib, check
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerExchange covers the GPUs of one node (at most 8 ranks)")
        if heads % self.world or seq % self.world:
            raise ValueError(f"{heads} heads / {seq} tokens do not divide over {self.world} ranks")
        self.heads, self.seq, self.head_dim, self.dtype, self.device = heads, seq, head_dim, dtype, torch.device(device)
        self.heads_per_rank, self.tokens_per_rank = heads // self.world, seq // self.world
        self.head0 = self.rank * self.heads_per_rank
        esz = torch.empty(0, dtype=dtype).element_size()
        self.elem_bytes = esz
        nbytes = self.tokens_per_rank * heads * head_dim * esz
        # q/k/v/o: this rank's tokens, all heads.  r0/r1: two head-sharded receive buffers [3, H/P, S, D] for push()
        # (alternating between steps, so a fast rank never overwrites what a slow one still reads).
        sizes = {"q": nbytes, "k": nbytes, "v": nbytes, "o": nbytes}
        if push_buffers:
            sizes["r0"] = sizes["r1"] = 3 * self.heads_per_rank * seq * head_dim * esz
        names = tuple(sizes)
        self._own, self._opened = {}, []
        handles = {}
        with torch.cuda.device(self.device):
            for name in names:
                ptr, h = C.c_void_p(), (C.c_ubyte * 64)()
                check(lib.psa_peer_alloc(sizes[name], C.byref(ptr), h), "psa_peer_alloc")
                self._own[name] = ptr.value
                handles[name] = bytes(h)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=group)
        self._peer = {name: [0] * self.world for name in names}
        with torch.cuda.device(self.device):
            for r, hs in enumerate(gathered):
                for name in names:
                    if r == self.rank:
                        self._peer[name][r] = self._own[name]
                    else:
                        ptr = C.c_void_p()
                        buf = (C.c_ubyte * 64).from_buffer_copy(hs[name])
                        check(lib.psa_peer_open(buf, C.byref(ptr)), "psa_peer_open")
                        self._peer[name][r] = ptr.value
                        self._opened.append(ptr.value)
        shape = (self.tokens_per_rank, heads, head_dim)
        self.q, self.k, self.v, self.o = (_as_tensor(self._own[n], shape, dtype, self.device) for n in ("q", "k", "v", "o"))
        self._ptr_arrays = {n: (C.c_void_p * self.world)(*self._peer[n]) for n in ("q", "k", "v", "o")}
        self._recv, self._push_arrays = [], []
        if push_buffers:
            one = self.heads_per_rank * seq * head_dim * esz
            for par in ("r0", "r1"):
                self._recv.append(_as_tensor(self._own[par], (3, self.heads_per_rank, seq, head_dim), dtype, self.device))
                self._push_arrays.append([(C.c_void_p * self.world)(*[p + i * one for p in self._peer[par]]) for i in range(3)])

    def push(self, parity: int, names=("q", "k", "v"), max_blocks: int = 0) -> torch.Tensor:
        """Send this rank's rows of q/k/v to the ranks that own the heads (receive buffer `parity` of every peer) and return
        this rank's receive buffer [3, H/P, S, D].  It holds all ranks' rows once a barrier that every rank enqueues after
        its push has completed."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            for i, name in enumerate(("q", "k", "v")):
                if name not in names:
                    continue
                rc = self.lib.psa_push_heads(self._own[name], self._push_arrays[parity][i], self.world, self.tokens_per_rank,
                                             self.heads, self.head_dim, self.elem_bytes, self.rank, int(max_blocks), stream)
                self.check(rc, "psa_push_heads")
        return self._recv[parity]

    def pull(self, first: int = 0, count: int = None, out: torch.Tensor = None, max_blocks: int = 0,
             names=("q", "k", "v")) -> torch.Tensor:
        """This rank's local heads [first, first+count) of all tokens: [3, count, S, D] (rows q, k, v), read from the
        peers.  `names` restricts the copy to some of the three (the other rows of `out` are left alone), so that e.g.
        v can follow on a second stream while the scores are computed from q and k.  max_blocks > 0 caps the copy
        kernel's grid (use a few dozen when it runs under compute kernels)."""
        count = self.heads_per_rank - first if count is None else count
        if out is None:
            out = torch.empty((3, count, self.seq, self.head_dim), dtype=self.dtype, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            for i, name in enumerate(("q", "k", "v")):
                if name not in names:
                    continue
                rc = self.lib.psa_pull_heads(self._ptr_arrays[name], self.world, out[i].data_ptr(), self.tokens_per_rank, self.heads,
                                             self.head0 + first, count, self.head_dim, self.elem_bytes, int(max_blocks),
                                             self.rank, stream)
                self.check(rc, "psa_pull_heads")
        return out

    # ------------------------------------------------------------------ sampled rows first
    def enable_sample_push(self, block_m: int, block_n: int):
        """Allocate and map the compacted sample matrices (two sets, alternating between steps) that push_samples() fills
        on the head owners.  Collective: every rank calls it once, with the same block sizes."""
        nq, nkv, nk = C.c_int64(), C.c_int64(), C.c_int64()
        self.check(self.lib.psa_sample_rows(self.seq, self.seq, block_m, block_n, C.byref(nq), C.byref(nkv), C.byref(nk)),
                   "psa_sample_rows")
        self._samp = dict(block_m=block_m, block_n=block_n, nq=nq.value, nk_valid=nkv.value, nk=nk.value)
        hp, D, esz = self.heads_per_rank, self.head_dim, self.elem_bytes
        q_bytes, k_bytes = hp * nq.value * D * esz, hp * nk.value * D * esz
        q_bytes = (q_bytes + 255) // 256 * 256
        handles, own = {}, {}
        with torch.cuda.device(self.device):
            for name in ("s0", "s1"):
                ptr, h = C.c_void_p(), (C.c_ubyte * 64)()
                self.check(self.lib.psa_peer_alloc(q_bytes + k_bytes, C.byref(ptr), h), "psa_peer_alloc")
                own[name], handles[name] = ptr.value, bytes(h)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=self.group)
        self._samp_ptrs, self._samp_views = [], []
        with torch.cuda.device(self.device):
            for name in ("s0", "s1"):
                peers = []
                for r, hs in enumerate(gathered):
                    if r == self.rank:
                        peers.append(own[name])
                    else:
                        ptr = C.c_void_p()
                        buf = (C.c_ubyte * 64).from_buffer_copy(hs[name])
                        self.check(self.lib.psa_peer_open(buf, C.byref(ptr)), "psa_peer_open")
                        peers.append(ptr.value)
                        self._opened.append(ptr.value)
                self._own[name] = own[name]
                self._samp_ptrs.append(((C.c_void_p * self.world)(*peers), (C.c_void_p * self.world)(*[p + q_bytes for p in peers])))
                self._samp_views.append((own[name], own[name] + q_bytes))

    def push_samples(self, parity: int, idx_q_all: torch.Tensor, idx_k_all: torch.Tensor):
        """Send the sampled rows of this rank's tokens (offsets of ALL heads: [1, H, block/4]) to the head owners' sample
        matrices number `parity`.  Complete on every rank after a barrier enqueued behind it."""
        sp = self._samp
        iq = idx_q_all.to(torch.int32).contiguous()
        ik = idx_k_all.to(torch.int32).contiguous()
        assert iq.shape == (1, self.heads, sp["block_m"] // 4) and ik.shape == (1, self.heads, sp["block_n"] // 4)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            rc = self.lib.psa_push_samples(self._own["q"], iq.data_ptr(), self._samp_ptrs[parity][0], self.world, self.tokens_per_rank,
                                           self.heads, self.head_dim, self.elem_bytes, sp["block_m"], sp["block_m"] // 4, sp["nq"],
                                           sp["nq"], self.rank, stream)
            self.check(rc, "psa_push_samples")
            rc = self.lib.psa_push_samples(self._own["k"], ik.data_ptr(), self._samp_ptrs[parity][1], self.world, self.tokens_per_rank,
                                           self.heads, self.head_dim, self.elem_bytes, sp["block_n"], sp["block_n"] // 4,
                                           sp["nk_valid"], sp["nk"], self.rank, stream)
            self.check(rc, "psa_push_samples")
        self._keep = (iq, ik)      # the kernels read the offsets asynchronously

    def scores_from_samples(self, parity: int) -> torch.Tensor:
        """Block scores [1, H/P, Mq, Nk] of this rank's heads from the sample matrices number `parity`."""
        from .ops import _dt
        sp, hp = self._samp, self.heads_per_rank
        Mq, Nk = -(-self.seq // sp["block_m"]), -(-self.seq // sp["block_n"])
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            po = torch.empty((1, hp, Mq, Nk), dtype=self.dtype, device=self.device)
            nbytes = self.lib.psa_block_scores_scratch_bytes(hp, self.seq, self.seq, sp["block_m"], sp["block_n"], _dt(po))
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            qs, ks = self._samp_views[parity]
            rc = self.lib.psa_block_scores_samples(qs, ks, po.data_ptr(), scratch.data_ptr(), nbytes, hp, self.seq, self.seq,
                                                   self.head_dim, sp["block_m"], sp["block_n"], _dt(po), stream)
        self.check(rc, "psa_block_scores_samples")
        return po

    def block_scores(self, idx_q: torch.Tensor, idx_k: torch.Tensor, block_m: int, block_n: int) -> torch.Tensor:
        """Block scores [1, H/P, Mq, Nk] of this rank's heads; the sampled q/k rows are read from the peers' buffers."""
        from .ops import _dt
        hp = self.heads_per_rank
        assert idx_q.shape == (1, hp, block_m // 4) and idx_k.shape == (1, hp, block_n // 4)
        iq, ik = idx_q.to(torch.int32).contiguous(), idx_k.to(torch.int32).contiguous()
        Mq, Nk = -(-self.seq // block_m), -(-self.seq // block_n)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            po = torch.empty((1, hp, Mq, Nk), dtype=self.dtype, device=self.device)
            nbytes = self.lib.psa_block_scores_scratch_bytes(hp, self.seq, self.seq, block_m, block_n, _dt(po))
            if nbytes == 0:
                raise ValueError(f"unsupported block sizes m={block_m} n={block_n}")
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            rc = self.lib.psa_block_scores_peers(self._ptr_arrays["q"], self._ptr_arrays["k"], self.world, self.tokens_per_rank,
                                                 self.heads, self.head0, iq.data_ptr(), ik.data_ptr(), po.data_ptr(),
                                                 scratch.data_ptr(), nbytes, hp, self.head_dim, block_m, block_n, _dt(po), stream)
        self.check(rc, "psa_block_scores_peers")
        return po

    def pyramid_images(self, block_n: int, max_blocks: int = 0):
        """Tile images of this rank's heads of K and V, every element read once from the peer that owns the token."""
        from .ops import KVImages, _dt
        hp = self.heads_per_rank
        nbytes = self.lib.psa_kv_image_bytes(hp, self.seq, self.head_dim, block_n)
        if nbytes == 0:
            raise ValueError(f"tile images need head_dim 64/128 and block_n 64/128 (got {self.head_dim}, {block_n})")
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            kimg = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            vimg = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            rc = self.lib.psa_pyramid_kv_images_peers(self._ptr_arrays["k"], self._ptr_arrays["v"], self.world, self.tokens_per_rank,
                                                      self.heads, self.head0, kimg.data_ptr(), vimg.data_ptr(), hp, self.head_dim,
                                                      block_n, _dt(self.k), int(max_blocks), stream)
        self.check(rc, "psa_pyramid_kv_images_peers")
        return KVImages(kimg, vimg, block_n)

    def forward_scatter(self, q: torch.Tensor, images, mask: torch.Tensor, block_m: int, block_n: int, tile_n: int,
                        first: int = 0, sm_scale: float = None, compat_quirk: bool = True) -> torch.Tensor:
        """Tile-image forward on local heads [first, first+q.shape[-3]); output rows land in the owners' `o` buffers.
        Returns the device status word of the launch."""
        from .ops import _dt, status_word
        hc, S, D = q.shape[-3], q.shape[-2], q.shape[-1]
        sm_scale = D ** -0.5 if sm_scale is None else sm_scale
        status = status_word(q.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            rc = self.lib.psa_fwd_images_scatter(q.data_ptr(), images.kimg.data_ptr(), images.vimg.data_ptr(), mask.data_ptr(),
                                                 self._ptr_arrays["o"], self.world, self.tokens_per_rank, self.heads,
                                                 self.head0 + first, hc, S, S, D, block_m, block_n, tile_n, mask.shape[-1],
                                                 float(sm_scale), int(compat_quirk), _dt(q), status.data_ptr(), stream)
        self.check(rc, "psa_fwd_images_scatter")
        return status

    def close(self):
        """Unmap the peers' buffers and free the own ones (all ranks must be past their last use: barrier first)."""
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.lib.psa_peer_close(p)
            self._opened = []
            self.q = self.k = self.v = self.o = None
            self._recv = []
            for p in self._own.values():
                self.lib.psa_peer_free(p)
            self._own = {}
