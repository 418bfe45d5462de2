"""Full-featured PSA module used by the video-model attention processors: same constructor, fields, call contract and
warm-up rule as PyramidSparseAttention / AttentionConfig (src/psa_triton/pyramid_sparse_attention.py:28-83, 252-413).

Differences, all outside the arithmetic: only the 'Gilbert' rearrangement is built (the k-means / STA / hybrid
rearrangers are out of scope and raise NotImplementedError), and the sparsity log is an in-memory list (the reference's
PSALogger writes JSONL files) fed from a device-side density kernel so that logging never forces a host sync per call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .attention import compute_block_mask, psa_attention_token_major, token_major_view
from .kernels import legacy_sparse_attention_factory, sparse_attention_factory
from .rearrange import GilbertRearranger


@dataclass
class AttentionConfig:
    width: int = 45
    height: int = 30
    depth: int = 13
    text_length: int = 226
    use_rearrange: bool = True
    block_m: int = 32
    block_n: int = 32
    tile_n: int = 32
    use_sim_mask: bool = True
    mask_ratios: Dict[int, Tuple[float, float]] = None
    mask_mode: str = 'topk'
    warmup_steps: int = 12
    tile_size: Optional[Tuple[int, int, int]] = None
    rearrange_method: str = None
    attn_impl: str = "new_mask_type"
    verbose: bool = False
    enable_logging: bool = True
    log_dir: str = "./psa_logs/"
    sim_2x_threshold: float = 0
    sim_4x_threshold: float = 0
    sim_8x_threshold: float = -1

    def __post_init__(self):
        if self.mask_ratios is None:
            self.mask_ratios = {1: (0.0, 0.05), 2: (0.05, 0.15), 4: (0.15, 0.25), 8: (0.25, 0.5), 0: (0.5, 1.0)}
        if self.attn_impl == "new_mask_type" and self.use_sim_mask:
            raise ValueError(
                "Incompatible configuration: 'new_mask_type' does not support 'use_sim_mask=True'.\n"
                "Please choose one of the following options:\n"
                "  1. Set 'use_sim_mask: false' to disable similarity mask\n"
                "  2. Use 'attn_impl: old_mask_type' with block_size config (m=128, n=128, tile_n=32)")


class SparsityLog:
    """Stand-in for PSALogger: one record per forward; densities stay on the device until somebody reads them."""

    def __init__(self):
        self.records: List[dict] = []

    def log_sparsity(self, **kw):
        self.records.append(kw)

    def close(self):
        pass

    def write_jsonl(self, path: str) -> int:
        """One line per forward with the keys of PSALogger's sparsity.jsonl (src/psa_triton/utils/psa_logger.py:265-283,
        minus the timestamp and the similarity statistics).  The per-(batch, head) densities were computed on the device
        by psa_density during the run; they are brought to the host here in ONE copy, so logging costs no
        synchronisation per layer call.  Returns the number of lines written."""
        import json
        import os
        dens = [r["density"].float().mean(dim=0).reshape(-1) for r in self.records if r.get("density") is not None]
        host = torch.stack(dens).cpu().tolist() if dens else []
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        it = iter(host)
        with open(path, "w") as f:
            for step, r in enumerate(self.records):
                per_head = next(it) if r.get("density") is not None else []
                density = sum(per_head) / len(per_head) if per_head else 1.0
                f.write(json.dumps({
                    "global_step": step, "layer_idx": r.get("layer_idx"), "sparsity": round(1.0 - density, 6),
                    "density": round(density, 6), "per_head_density": [round(d, 6) for d in per_head],
                    "sequence_length": r.get("sequence_length"), "batch_size": r.get("batch_size"),
                    "num_heads": r.get("num_heads"), "is_warmup": bool(r.get("is_warmup", False))}) + "\n")
        return len(self.records)

    def summary(self) -> dict:
        dens = [float(r["density"].mean().item()) for r in self.records if r.get("density") is not None]
        return {"calls": len(self.records), "sparse_calls": len(dens),
                "mean_sparsity": 1.0 - sum(dens) / len(dens) if dens else 0.0}


def adaptive_block_sparse_attn(q, k, v, config: AttentionConfig, sparse_attention_fn, compute_stats: bool = False):
    """Scores -> mask (-> similarity cap) -> sparse attention (pyramid_sparse_attention.py:188-249).
    Returns (out, density [B,H] device tensor or None, sim_mask)."""
    if config.attn_impl not in ("old_mask_type", "new_mask_type"):
        raise ValueError(f"Unknown attn_impl: {config.attn_impl}")
    with torch.no_grad():
        mask, _, sim = compute_block_mask(q, k, config, text_length=config.text_length)
    out = sparse_attention_fn(q.contiguous(), k.contiguous(), v.contiguous(), mask, None)
    dens = ops.density(mask, config.attn_impl == "new_mask_type") if compute_stats else None
    return out, dens, sim


class PyramidSparseAttention(nn.Module):
    def __init__(self, config: AttentionConfig = None, inference_num=50, layer_num=42, model_type="wan"):
        super().__init__()
        self.config = config if config is not None else AttentionConfig()
        config = self.config
        self.model_type = model_type.lower()
        self.gilbert_rearranger = None
        if config.use_rearrange:
            if config.rearrange_method == 'Gilbert':
                self.gilbert_rearranger = GilbertRearranger(config.width, config.height, config.depth, config.text_length)
            elif config.rearrange_method in ('SemanticAware', 'STA', 'Hybrid'):
                raise NotImplementedError(f"rearrange_method={config.rearrange_method!r} is outside this library's scope "
                                          "(no shipped preset selects it); use 'Gilbert' or use_rearrange=False")
            else:
                raise ValueError(f"Unknown rearrange_method: {config.rearrange_method}")
        self.sparsity_counter = 0
        self.use_rearrange = config.use_rearrange
        self.inference_num = inference_num
        self.layer_num = layer_num
        if config.attn_impl == "old_mask_type":
            self.sparse_attention_fn = legacy_sparse_attention_factory(config.block_m, config.tile_n, config.block_n)
        elif config.attn_impl == "new_mask_type":
            self.sparse_attention_fn = sparse_attention_factory(config.block_m, config.tile_n, config.block_n)
        else:
            raise ValueError(f"Unknown attn_impl: {config.attn_impl}")
        self.logger = SparsityLog() if config.enable_logging else None

    def get_current_time(self):
        """Denoising step index: one call per layer for cogvideo / 4-step Wan, two (CFG) passes per step otherwise
        (pyramid_sparse_attention.py:317-322)."""
        if self.model_type == "cogvideo" or self.model_type == "wan2.1_1.3b_4steps":
            return (self.sparsity_counter // self.layer_num) % self.inference_num
        return (self.sparsity_counter // (2 * self.layer_num)) % self.inference_num

    def _rows_in_place(self, q, k) -> bool:
        """Whether the Gilbert order can be folded into the kernels (k, v, the output and the sampled q rows are never
        copied): 16-bit tensors on the tcgen05 kernels, separator-format mask without the similarity cap."""
        c = self.config
        return (self.use_rearrange and c.attn_impl == "new_mask_type" and not c.use_sim_mask and q.is_cuda
                and q.shape[2] == k.shape[2] == self.gilbert_rearranger.total_elements + self.gilbert_rearranger.text_length
                and ops.images_supported(k, c.block_m, c.block_n, c.tile_n)
                and -(-k.shape[2] // c.block_n) + 5 <= 1472)

    def _rows_in_place_old_format(self, q, k) -> bool:
        """The same for the old mask format (with or without the similarity cap; block 128): inference only, the
        differentiable route keeps the copies."""
        c = self.config
        return (self.use_rearrange and c.attn_impl == "old_mask_type" and q.is_cuda
                and not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or self._v_requires_grad))
                and q.dtype in (torch.float16, torch.bfloat16) and c.block_m == 128 and c.block_n == 128 and c.tile_n == 32
                and q.shape[-1] in (64, 128) and -(-q.shape[2] // 128) + 5 <= 1472
                and q.shape[2] == k.shape[2] == self.gilbert_rearranger.total_elements + self.gilbert_rearranger.text_length)

    _v_requires_grad = False      # set per call by forward()

    def _forward_old_format_in_place(self, q, k, v, compute_stats):
        c = self.config
        perm = self.gilbert_rearranger.source_rows(q.device)
        mask, _, _ = compute_block_mask(q, k, c, text_length=c.text_length, perm=perm)
        out = ops.legacy_forward_reordered(q, k, v, mask, perm)
        dens = ops.density(mask, False) if compute_stats else None
        return out, dens

    def _forward_rows_in_place(self, q, k, v, compute_stats, rope=None):
        c = self.config
        perm = self.gilbert_rearranger.source_rows(q.device)
        with torch.no_grad():
            mask, _, _ = compute_block_mask(q, k, c, text_length=c.text_length, perm=perm, rope=rope)
        images = ops.pyramid_kv_images(k.contiguous(), v.contiguous(), c.block_n, perm=perm, rope=rope)
        q_r = ops.gather_rows(q.contiguous(), perm, rope=rope)
        out = ops.psa_forward(q_r, k, v, mask, c.block_m, c.block_n, c.tile_n, None, pyramid=images, out_perm=perm)
        dens = ops.density(mask, True) if compute_stats else None
        return out.view(q.shape), dens

    fuses_rotary = True       # forward() takes rotary=..., so a processor may hand over unrotated q and k

    def forward(self, q, k, v, layer_idx, rotary=None):
        """q, k, v [B, H, S, D].  rotary (ops.RotaryTables, optional): q and k arrive unrotated; on the token-major route
        the kernels rotate the rows as they read them, on every other route they are rotated here first."""
        is_warmup = self.get_current_time() < self.config.warmup_steps
        if rotary is not None:
            # the in-place routes (token-major views or head-major tensors) rotate inside their loads
            if is_warmup or not self._rows_in_place(q, k):
                q, k = ops.rotate_rows(q, rotary), ops.rotate_rows(k, rotary)
                rotary = None
        compute_stats = self.config.verbose or self.logger is not None
        dens = None
        self._v_requires_grad = v.requires_grad
        if not is_warmup and self._rows_in_place_old_format(q, k):
            out, dens = self._forward_old_format_in_place(q, k, v, compute_stats)
            self.sparsity_counter += 1
            if self.logger is not None:
                self.logger.log_sparsity(layer_idx=layer_idx, density=dens, sequence_length=q.shape[2],
                                         batch_size=q.shape[0], num_heads=q.shape[1], is_warmup=False)
            return out
        if not is_warmup and self._rows_in_place(q, k):
            tm = [token_major_view(x) for x in (q, k, v)]
            if all(t is not None for t in tm):
                # the processors hand over transposed views of [B, S, H, D] tensors: read those where they lie and return
                # the same kind of view, so that the caller's transpose(1, 2).flatten(2, 3) costs nothing
                out_tm, mask = psa_attention_token_major(*tm, self.config, perm=self.gilbert_rearranger.source_rows(q.device),
                                                         text_length=self.config.text_length, rope=rotary)
                out = out_tm.transpose(1, 2)
                dens = ops.density(mask, True) if compute_stats else None
            else:
                out, dens = self._forward_rows_in_place(q, k, v, compute_stats, rope=rotary)
            self.sparsity_counter += 1
            if self.logger is not None:
                self.logger.log_sparsity(layer_idx=layer_idx, density=dens, sequence_length=q.shape[2],
                                         batch_size=q.shape[0], num_heads=q.shape[1], is_warmup=False)
            return out
        if self.use_rearrange:
            q_r, k_r, v_r = self.gilbert_rearranger.rearrange(q, k, v)
        else:
            q_r, k_r, v_r = q, k, v
        if is_warmup:
            # dense warm-up steps, exactly what the reference runs (:353-357)
            out_r = torch.nn.functional.scaled_dot_product_attention(q_r, k_r, v_r)
        else:
            out_r, dens, _ = adaptive_block_sparse_attn(q_r, k_r, v_r, self.config, self.sparse_attention_fn, compute_stats)
        self.sparsity_counter += 1
        if self.logger is not None:
            self.logger.log_sparsity(layer_idx=layer_idx, density=dens, sequence_length=q.shape[2], batch_size=q.shape[0],
                                     num_heads=q.shape[1], is_warmup=is_warmup)
        return self.gilbert_rearranger.reversed_rearrange(out_r) if self.use_rearrange else out_r

    def close_logger(self, jsonl_path: str = None):
        """Reference name (pyramid_sparse_attention.py:408-413).  With logging enabled the per-call records go to
        ``<config.log_dir>/sparsity.jsonl`` (the file PSALogger keeps, src/psa_triton/utils/psa_logger.py:265-283) or to
        jsonl_path, in one host copy for the whole run.  Also the point where a run learns whether an attention kernel
        gave up on a bounded device-side wait (ops.check_status)."""
        if self.logger is not None:
            if self.logger.records:
                import os
                self.logger.write_jsonl(jsonl_path if jsonl_path is not None
                                        else os.path.join(self.config.log_dir, "sparsity.jsonl"))
            self.logger.close()
        ops.check_status()
