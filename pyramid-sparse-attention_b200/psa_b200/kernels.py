"""Kernel-level callables with the reference's factory signatures.

``sparse_attention_factory(BLOCK_M, BLOCK_N(=tile_n), POOLING_BLOCK_N(=block_n))`` mirrors
src/psa_triton/kernels/psa_kernel.py:441-457; ``legacy_sparse_attention_factory(128, 32, 128, causal)``
mirrors src/psa_triton/kernels/psa_kernel_legacy.py:1323-1370 and is differentiable.
"""
from __future__ import annotations

import torch

from . import ops


def sparse_attention_factory(BLOCK_M=128, BLOCK_N=128, POOLING_BLOCK_N=128, compat_quirk=True, impl=ops.IMPL_AUTO):
    """Forward-only multi-level sparse attention on the separator-format mask."""
    def _sparse_attention_fn(q, k, v, block_sparse_dense, sm_scale=None):
        sm_scale = sm_scale if sm_scale is not None else q.shape[-1] ** -0.5
        return ops.psa_forward(q, k, v, block_sparse_dense, BLOCK_M, POOLING_BLOCK_N, BLOCK_N, sm_scale,
                               compat_quirk=compat_quirk, impl=impl)
    return _sparse_attention_fn


class _LegacySparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, block_sparse_dense, sm_scale, causal):
        need_backward = q.requires_grad or k.requires_grad or v.requires_grad
        qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
        # the reference takes int32 or int64 masks with any strides (psa_kernel_legacy.py:1254); forward and backward
        # both read the one normalised copy
        mask = ops._mask32(block_sparse_dense)
        o, lse, pooled = ops.legacy_forward(qc, kc, vc, mask, causal, sm_scale, need_lse=need_backward)
        if need_backward:
            ctx.save_for_backward(qc, kc, vc, mask, o, lse)
            ctx.pooled = pooled            # the pooled K/V the forward built (not part of the graph)
            ctx.sm_scale = sm_scale
            ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, mask, o, lse = ctx.saved_tensors
        dq, dk, dv = ops.legacy_backward(q, k, v, mask, o, lse, do.contiguous(), ctx.causal, ctx.sm_scale, ctx.pooled)
        return dq, dk, dv, None, None, None


def legacy_sparse_attention_factory(BLOCK_M=128, BLOCK_N=32, POOLING_BLOCK_N=128, causal=False):
    """Legacy (old-format mask) attention; same fixed block sizes and ValueErrors as the reference."""
    if BLOCK_M != 128:
        raise ValueError(f"BLOCK_M must be 128, got {BLOCK_M}. "
                         "Current version only supports BLOCK_M=128, BLOCK_N=32, POOLING_BLOCK_N=128.")
    if BLOCK_N != 32:
        raise ValueError(f"BLOCK_N must be 32, got {BLOCK_N}. "
                         "Current version only supports BLOCK_M=128, BLOCK_N=32, POOLING_BLOCK_N=128.")
    if POOLING_BLOCK_N != 128:
        raise ValueError(f"POOLING_BLOCK_N must be 128, got {POOLING_BLOCK_N}. "
                         "Current version only supports BLOCK_M=128, BLOCK_N=32, POOLING_BLOCK_N=128.")

    def _fn(q, k, v, block_sparse_dense, sm_scale=None):
        sm_scale = sm_scale if sm_scale is not None else q.shape[-1] ** -0.5
        return _LegacySparseAttention.apply(q, k, v, block_sparse_dense, sm_scale, causal)
    return _fn
