"""psa_b200: B200 (sm_100a) kernels behind the Pyramid-Sparse-Attention plug-and-play API."""
from . import ops
from .attention import PSAAttention, PSAConfig, compute_block_mask, psa_attention, psa_attention_host
from .kernels import legacy_sparse_attention_factory, sparse_attention_factory

__all__ = ["ops", "PSAAttention", "PSAConfig", "psa_attention", "psa_attention_host", "compute_block_mask",
           "sparse_attention_factory", "legacy_sparse_attention_factory"]
