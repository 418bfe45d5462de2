"""Host side of the causal (vision-language) call site, mirroring
qwen2.5-vl-example/src/attention/PSA_casual/PyramidAdaptiveBlockSparseAttn.py: same config fields, function names,
argument meaning and errors.  Estimate (antidiagonal scores) -> level mask -> similarity cap -> legacy causal attention.

Differences: the sparsity log is an in-memory list (`records`), and the estimate needs f16/bf16 tensors (the CUDA
kernels have no fp32 variant)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .kernels import legacy_sparse_attention_factory


@dataclass
class AttentionConfig:
    """Same fields and defaults as the reference's AttentionConfig (:22-57)."""
    text_length: int = 512
    query_block: int = 128
    warmup_steps: int = 0
    mask_ratios: Dict[int, Tuple[float, float]] = field(default_factory=lambda: {
        1: (0.0, 0.05), 2: (0.05, 0.15), 4: (0.15, 0.25), 8: (0.25, 0.5), 0: (0.5, 1.0)})
    mask_mode: str = "topk"
    importance_method: str = "xattn"
    xattn_stride: int = 16
    xattn_chunk_size: int = 4096
    causal_main: bool = True
    sim_2x_threshold: float = 0.75
    sim_4x_threshold: float = 0.7
    sim_8x_threshold: float = 0.7

    def __post_init__(self) -> None:
        self.importance_method = self.importance_method.lower()
        if self.importance_method not in {"xattn"}:
            raise ValueError("importance_method must be 'xattn'")
        self.mask_mode = self.mask_mode.lower()
        if self.mask_mode not in {"topk", "energybound"}:
            raise ValueError("mask_mode must be 'topk' or 'energybound'")


def x_block_imp_estimate(query, key, *, block_size: int, stride: int, chunk_size: int, causal: bool) -> torch.Tensor:
    """(:60-81)"""
    return ops.antidiag_block_scores(query, key, block_size, stride, chunk_size, causal)


def transfer_attn_to_mask(attn, mask_ratios, text_length: int, mode: str, *, block_size: int, causal: bool) -> torch.Tensor:
    """(:85-168)"""
    return ops.assign_levels_causal(attn, mask_ratios, text_length, mode, block_size, causal)


def calc_density(mask: torch.Tensor, causal: bool):
    """Mean of 1/level over the entries a row may attend to (:171-196).  Returns device tensors (overall, per head):
    no host synchronisation."""
    dens = torch.where(mask > 0, 1.0 / mask.clamp(min=1).float(), torch.zeros((), device=mask.device))
    n = mask.size(-1)
    if causal:
        dens = dens * torch.tril(torch.ones(n, n, device=mask.device))
        count = n * (n + 1) / 2
    else:
        count = n * n
    per_head = dens.sum(dim=(0, 2, 3)) / max(1.0, count * mask.size(0))
    return dens.sum() / max(1.0, count * mask.size(0) * mask.size(1)), per_head


def adaptive_block_sparse_attn(q, k, v, config: AttentionConfig, sparse_attention_fn):
    """(:199-247) Returns (out, sparsity, per-head density) - the last two as device tensors."""
    block = config.query_block
    with torch.no_grad():
        est = x_block_imp_estimate(q, k, block_size=block, stride=config.xattn_stride, chunk_size=config.xattn_chunk_size,
                                   causal=config.causal_main)
        mask = transfer_attn_to_mask(est, config.mask_ratios, config.text_length, config.mask_mode, block_size=block,
                                     causal=config.causal_main)
        sim = ops.k_similarity(k, block, float(config.sim_2x_threshold), float(config.sim_4x_threshold),
                               float(config.sim_8x_threshold))
        mask = torch.min(sim.unsqueeze(-2).to(mask.dtype), mask)
    out = sparse_attention_fn(q.contiguous(), k.contiguous(), v.contiguous(), mask.contiguous(), None)
    avg, per_head = calc_density(mask, config.causal_main)
    return out, 1 - avg, per_head


class PyramidAdaptiveBlockSparseAttnTrain(nn.Module):
    """(:250-333) One instance per layer; dense attention during the warm-up calls."""

    def __init__(self, config: Optional[AttentionConfig] = None, *, layer_idx: int = -1, log_dir: Optional[str] = None,
                 log_prefix: str = "psa_sparsity", session_name: Optional[str] = None, **extra: object) -> None:
        super().__init__()
        self.config = config or AttentionConfig()
        self.layer_idx = layer_idx
        self.sparse_attention_fn = legacy_sparse_attention_factory(128, 32, 128, causal=self.config.causal_main)
        self.sparsity_acc = 0.0
        self.sparsity_counter = 0
        self.records = [] if (log_dir is not None or "save_dir" in extra) else None

    def forward(self, q, k, v, frame_num=None, height=None, width=None, *, layer_idx: Optional[int] = None):
        if layer_idx is not None:
            self.layer_idx = layer_idx
        self.sparsity_counter += 1
        if self.sparsity_counter <= self.config.warmup_steps:
            return torch.nn.functional.scaled_dot_product_attention(q, k, v)
        out, sparsity, per_head = adaptive_block_sparse_attn(q, k, v, self.config, self.sparse_attention_fn)
        self.sparsity_acc = self.sparsity_acc + sparsity
        if self.records is not None:
            self.records.append(dict(layer_idx=self.layer_idx, sparsity=sparsity, per_head_density=per_head,
                                     sequence_length=q.size(2), batch_size=q.size(0), num_heads=q.size(1)))
        return out
