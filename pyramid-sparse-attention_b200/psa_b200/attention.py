"""Plug-and-play PSA module: same names, fields, validation and call contract as
src/psa_triton/attention.py (PSAConfig :36-104, PSAAttention :226-310, psa_attention :314-367).
The work is done by the sm_100a kernels; nothing here falls back to PyTorch math."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .kernels import legacy_sparse_attention_factory, sparse_attention_factory


@dataclass
class PSAConfig:
    """Configuration for PSA attention; defaults give ~85% sparsity."""
    block_m: int = 128
    block_n: int = 64
    tile_n: int = 32
    mask_ratios: Dict[int, Tuple[float, float]] = field(default_factory=lambda: {
        1: (0.0, 0.1), 2: (0.1, 0.15), 4: (0.15, 0.15), 8: (0.15, 0.35), 0: (0.35, 1.0)})
    mask_mode: str = 'topk'
    use_sim_mask: bool = False
    sim_2x_threshold: float = 0.0
    sim_4x_threshold: float = 0.0
    sim_8x_threshold: float = -1.0
    rearrange_method: str = None
    attn_impl: str = "new_mask_type"

    def __post_init__(self):
        if self.attn_impl == "new_mask_type" and self.use_sim_mask:
            raise ValueError(
                "Incompatible configuration: 'new_mask_type' does not support 'use_sim_mask=True'.\n"
                "Please choose one of the following options:\n"
                "  1. Set 'use_sim_mask=False' to disable similarity mask\n"
                "  2. Use 'attn_impl=\"old_mask_type\"' with block_size config (m=128, n=128, tile_n=32)")
        if self.attn_impl == "old_mask_type":
            if self.block_m != 128 or self.block_n != 128:
                raise ValueError(
                    f"attn_impl='old_mask_type' only supports block_m=128 and block_n=128.\n"
                    f"Got block_m={self.block_m}, block_n={self.block_n}.\n"
                    f"Use attn_impl='new_mask_type' for flexible block sizes (128/64/32).")
        if self.attn_impl == "new_mask_type":
            if self.block_n not in [128, 64, 32]:
                raise ValueError(
                    f"attn_impl='new_mask_type' only supports block_n in [128, 64, 32].\n"
                    f"Got block_n={self.block_n}.")


def compute_block_mask(q, k, config, text_length: int = 0, idx_q=None, idx_k=None, perm=None, rope=None):
    """Scores -> level mask (-> similarity cap), the no-grad half of PSAAttention.forward
    (src/psa_triton/attention.py:178-223, 276-299).  Returns (mask, scores, sim_mask).
    The sample offsets are drawn from torch's generator of q's device, Q first and K second, exactly as
    the reference does; tests may pass them in instead.  perm (int32 [S]): the mask of q[..., perm, :],
    k[..., perm, :] with the rows read in place.  rope (ops.RotaryTables; no similarity cap): q and k are given
    unrotated and the sampled rows are rotated as they are gathered."""
    B, H = q.shape[0], q.shape[1]
    sim = None
    if config.use_sim_mask:
        sim = ops.k_similarity(k, config.block_n, float(config.sim_2x_threshold), float(config.sim_4x_threshold),
                               float(config.sim_8x_threshold), perm=perm)
    if idx_q is None:
        idx_q = ops.draw_sample_indices(B, H, config.block_m, config.block_m // 4, q.device)
    if idx_k is None:
        idx_k = ops.draw_sample_indices(B, H, config.block_n, config.block_n // 4, q.device)
    assert rope is None or not config.use_sim_mask, "the similarity cap would see unrotated keys"
    po = ops.block_scores(q, k, idx_q, idx_k, config.block_m, config.block_n, perm_q=perm, perm_k=perm, rope=rope)
    if config.attn_impl == "old_mask_type":
        mode = config.mask_mode
    else:
        mode = f"{config.mask_mode}_newtype"
    mask = ops.assign_levels(po, config.mask_ratios, mode, config.block_n, config.tile_n, text_length=text_length)
    if config.use_sim_mask and sim is not None:
        mask = torch.min(sim.unsqueeze(-2).to(mask.dtype), mask)
    return mask, po, sim


def token_major_view(x: torch.Tensor):
    """If x ([B, H, S, D]) is the transpose(1, 2) view of a contiguous [B, S, H, D] tensor - what the diffusers
    processors pass (modify_diffusers.py:302-304, :357-359) - return that tensor, else None."""
    if x.dim() != 4 or x.shape[1] == 1 or x.shape[2] == 1:
        return None
    t = x.transpose(1, 2)
    return t if t.is_contiguous() else None


def psa_attention_token_major(q, k, v, config, perm=None, text_length: int = 0, idx_q=None, idx_k=None, rope=None):
    """The PSA layer on token-major tensors: q, k, v [B, S, H, D] contiguous (16-bit, separator-format mask, no
    similarity cap), perm an optional int32 [S] row table (attention token t = stored token perm[t]).  Returns
    (out [B, S, H, D], mask).  No transposed or reordered copy of k, v or the output is made; the result equals
    PSAAttention on q.transpose(1, 2)[:, :, perm] ... put back, bit for bit (same sample offsets).
    rope (ops.RotaryTables): q and k are given UNROTATED and every kernel that reads one of their rows rotates it on
    the way - the result equals rotating q and k first (as the processors of modify_diffusers.py do) bit for bit,
    without the two rotated copies."""
    B, S, H, D = q.shape
    if config.use_sim_mask or config.attn_impl != "new_mask_type":
        raise ValueError("the token-major route covers new_mask_type without the similarity cap")
    if not ops.images_supported(q, config.block_m, config.block_n, config.tile_n):
        raise ValueError("the token-major route needs f16/bf16, block_m 128, tile_n 32, block_n 64/128, head_dim 64/128")
    if idx_q is None:
        idx_q = ops.draw_sample_indices(B, H, config.block_m, config.block_m // 4, q.device)
    if idx_k is None:
        idx_k = ops.draw_sample_indices(B, H, config.block_n, config.block_n // 4, q.device)
    with torch.no_grad():
        po = torch.cat([ops.block_scores_tm(q[b], k[b], idx_q[b], idx_k[b], config.block_m, config.block_n, perm=perm,
                                            rope=rope) for b in range(B)], dim=0)
        mask = ops.assign_levels(po, config.mask_ratios, f"{config.mask_mode}_newtype", config.block_n, config.tile_n,
                                 text_length=text_length)
    out = torch.empty_like(q)
    for b in range(B):
        images = ops.pyramid_kv_images_tm(k[b], v[b], config.block_n, perm=perm, rope=rope)
        q_heads = ops.gather_heads(q[b], perm, rope=rope)
        ops.psa_forward_tm(q_heads, images, mask[b], out[b], config.block_m, config.block_n, config.tile_n, out_perm=perm)
    return out, mask


class PSAAttention(nn.Module):
    """Drop-in attention: ``out = PSAAttention(config)(q, k, v)`` with q, k, v of shape [B, H, L, D]."""

    def __init__(self, config: PSAConfig = None):
        super().__init__()
        self.config = config if config is not None else PSAConfig()
        if self.config.attn_impl == "old_mask_type":
            self.sparse_attention_fn = legacy_sparse_attention_factory(self.config.block_m, self.config.tile_n,
                                                                       self.config.block_n)
        else:
            self.sparse_attention_fn = sparse_attention_factory(self.config.block_m, self.config.tile_n,
                                                                self.config.block_n)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, idx_q=None, idx_k=None) -> torch.Tensor:
        config = self.config
        with torch.no_grad():
            mask, _, _ = compute_block_mask(q, k, config, text_length=0, idx_q=idx_q, idx_k=idx_k)
        return self.sparse_attention_fn(q.contiguous(), k.contiguous(), v.contiguous(), mask, None)

    @staticmethod
    def check_status(device=None) -> None:
        """Ask, once per run, whether any attention kernel gave up on a bounded device-side wait (its output would be
        incomplete); raises PSAKernelError if so.  The calls themselves never synchronise with the host."""
        ops.check_status(device)


def psa_attention(q, k, v, *, config: PSAConfig = None, mask_ratios=None, mask_mode: str = None, block_m: int = None,
                  block_n: int = None) -> torch.Tensor:
    """Functional form (src/psa_triton/attention.py:314-367); a block_n override also sets tile_n=min(32, block_n)."""
    if config is None:
        config = PSAConfig()
    if mask_ratios is not None:
        config.mask_ratios = mask_ratios
    if mask_mode is not None:
        config.mask_mode = mask_mode
    if block_m is not None:
        config.block_m = block_m
    if block_n is not None:
        config.block_n = block_n
        config.tile_n = min(32, block_n)
    return PSAAttention(config)(q, k, v)


def psa_attention_host(q, k, v, config: PSAConfig = None, out=None, device=None, heads_per_chunk: int = 0,
                       idx_q=None, idx_k=None):
    """The PSA layer for tensors that live in pinned HOST memory: q, k, v [B, H, L, D] -> out [B, H, L, D] (pinned host).

    Heads are independent in every stage, so the layer runs chunk by chunk over the heads with the copies on two side
    streams: while chunk c is computed, chunk c+1 is on its way to the device and the output of chunk c-1 on its way
    back, and the call costs about the longer of (transfer, compute) instead of their sum.  The sample offsets are drawn
    once for all heads (same generator consumption as PSAAttention), so the result equals PSAAttention on device copies
    bit for bit.  The returned tensor is complete once the current stream has been synchronised."""
    config = config if config is not None else PSAConfig()
    for t in (q, k, v):
        if t.device.type != "cpu" or not t.is_pinned() or not t.is_contiguous():
            raise ValueError("psa_attention_host takes contiguous tensors in pinned host memory")
    B, H, L, D = q.shape
    dev = torch.device(device if device is not None else "cuda")
    module = PSAAttention(config)
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    if heads_per_chunk > 0:
        hc = heads_per_chunk
    else:
        # about fourteen chunks (the first one's copy and the last one's compute and copy back are not overlapped with
        # anything), but no chunk below ~32 MB of input: smaller copies and kernels cost more than they hide
        per_head = 3 * B * L * D * q.element_size()
        hc = min(H, max(-(-H // 14), -(-(32 << 20) // per_head)))
    chunks = [(h0, min(H, h0 + hc)) for h0 in range(0, H, hc)]
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        if idx_q is None:
            idx_q = ops.draw_sample_indices(B, H, config.block_m, config.block_m // 4, dev)
        if idx_k is None:
            idx_k = ops.draw_sample_indices(B, H, config.block_n, config.block_n // 4, dev)
        # two sets of staging buffers, allocated on the current stream before any side stream touches them
        stage = [[torch.empty((B, hc, L, D), dtype=q.dtype, device=dev) for _ in range(3)] for _ in range(2)]
        outs = [torch.empty((B, hc, L, D), dtype=q.dtype, device=dev) for _ in range(2)]
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)
        s_out.wait_event(start)
        computed = [None, None]      # per buffer set: compute of the chunk that last used the inputs has finished
        drained = [None, None]       # per buffer set: the output copy of the chunk that last used it has finished
        for c, (h0, h1) in enumerate(chunks):
            b, n = c & 1, h1 - h0
            with torch.cuda.stream(s_in):
                if computed[b] is not None:
                    s_in.wait_event(computed[b])
                # q and k first: the scores and the level mask need nothing else, v is only read by the attention kernel
                for dst, src in zip(stage[b][:2], (q, k)):
                    dst[:, :n].copy_(src[:, h0:h1], non_blocking=True)
                arrived_qk = torch.cuda.Event()
                arrived_qk.record(s_in)
                stage[b][2][:, :n].copy_(v[:, h0:h1], non_blocking=True)
                arrived_v = torch.cuda.Event()
                arrived_v.record(s_in)
            main.wait_event(arrived_qk)
            dq, dk = (t[:, :n] for t in stage[b][:2])
            if n != hc:
                dq, dk = dq.contiguous(), dk.contiguous()
            with torch.no_grad():
                mask, _, _ = compute_block_mask(dq, dk, config, idx_q=idx_q[:, h0:h1].contiguous(),
                                                idx_k=idx_k[:, h0:h1].contiguous())
            main.wait_event(arrived_v)
            if drained[b] is not None:
                main.wait_event(drained[b])
            dv = stage[b][2][:, :n]
            if n != hc:
                dv = dv.contiguous()
            o = module.sparse_attention_fn(dq, dk, dv, mask, None)
            outs[b][:, :n].copy_(o)
            computed[b] = torch.cuda.Event()
            computed[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[b])
                out[:, h0:h1].copy_(outs[b][:, :n], non_blocking=True)
                drained[b] = torch.cuda.Event()
                drained[b].record(s_out)
        for e in drained:
            if e is not None:
                main.wait_event(e)
    return out
