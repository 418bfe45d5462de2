"""psa_b200: B200 (sm_100a) kernels behind the Pyramid-Sparse-Attention plug-and-play API."""
from . import ops
from .attention import PSAAttention, PSAConfig, compute_block_mask, psa_attention
from .kernels import legacy_sparse_attention_factory, sparse_attention_factory

__all__ = ["ops", "PSAAttention", "PSAConfig", "psa_attention", "compute_block_mask",
           "sparse_attention_factory", "legacy_sparse_attention_factory"]
