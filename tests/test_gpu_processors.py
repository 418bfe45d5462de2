"""GPU: a [B, S, H*D] hidden state through attention processor -> PyramidSparseAttention -> output projection, compared
with the same pipeline whose attention is the CPU oracle (same projections, same rotary tables, same sample offsets)."""
import pytest
import torch

import cases as C
from oracle import psa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))


class _Tap(torch.nn.Module):
    """Records what the processor hands to the sparse module, then calls it."""

    def __init__(self, inner):
        super().__init__()
        self.inner, self.seen = inner, None

    def forward(self, q, k, v, layer_idx):
        self.seen = (q.detach().clone(), k.detach().clone(), v.detach().clone())
        return self.inner(q, k, v, layer_idx)


def _attn(hidden, heads, per_head_norm):
    torch.manual_seed(3)
    a = torch.nn.Module()
    a.heads = heads
    a.to_q, a.to_k, a.to_v = (torch.nn.Linear(hidden, hidden) for _ in range(3))
    dim = hidden // heads if per_head_norm else hidden
    a.norm_q, a.norm_k = torch.nn.RMSNorm(dim, eps=1e-6), torch.nn.RMSNorm(dim, eps=1e-6)
    a.to_out = torch.nn.ModuleList([torch.nn.Linear(hidden, hidden), torch.nn.Identity()])
    a.add_k_proj = None
    a.is_cross_attention = False
    a.fused_projections = False
    return a.to(DEV).to(torch.bfloat16)


def _module(grid, text, rearrange):
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    w, h, d = grid
    cfg = AttentionConfig(width=w, height=h, depth=d, text_length=text, use_rearrange=rearrange,
                          rearrange_method="Gilbert" if rearrange else None, block_m=128, block_n=64, tile_n=32,
                          use_sim_mask=False, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk", warmup_steps=0,
                          enable_logging=False)
    return PyramidSparseAttention(cfg, inference_num=4, layer_num=1, model_type="wan" if text == 0 else "cogvideo")


def _oracle_attention(q, k, v, module, heads):
    """The sparse module's arithmetic on the CPU: Gilbert order (text to the end), scores, mask, forward, order undone.
    Consumes the CUDA generator exactly as the module does (Q offsets, then K offsets)."""
    from psa_b200 import ops
    iq = ops.draw_sample_indices(1, heads, 128, 32, DEV).cpu()
    ik = ops.draw_sample_indices(1, heads, 64, 16, DEV).cpu()
    q, k, v = q.cpu(), k.cpu(), v.cpu()
    r = module.gilbert_rearranger
    if r is not None:
        q, k, v = r.rearrange(q, k, v)
    o, mask, _ = O.psa_attention(q, k, v, block_m=128, block_n=64, tile_n=32, mask_ratios=C.DEFAULT_RATIOS,
                                 mask_mode="topk", idx_q=iq, idx_k=ik)
    return (r.reversed_rearrange(o) if r is not None else o), mask


@pytest.mark.parametrize("rearrange", [False, True])
def test_wan_processor_pipeline_vs_oracle(rearrange):
    from psa_b200.presets import SparseWanAttnProcessor
    B, H, D, grid = 1, 2, 64, (16, 16, 8)
    S = grid[0] * grid[1] * grid[2]
    attn = _attn(H * D, H, per_head_norm=False)
    module = _module(grid, 0, rearrange)
    attn.inner_attention = _Tap(module)
    x = C.randn(70, (B, S, H * D), torch.bfloat16, smooth=8).to(DEV)
    ang = torch.rand(1, S, 1, D // 2, generator=torch.Generator().manual_seed(9)) * 6.28
    rot = (torch.cos(ang).repeat_interleave(2, -1).to(DEV), torch.sin(ang).repeat_interleave(2, -1).to(DEV))
    torch.manual_seed(123)
    with torch.no_grad():
        out = SparseWanAttnProcessor(0)(attn, x, rotary_emb=rot)
    q, k, v = attn.inner_attention.seen
    # the operands are rotated: undoing the rotation on q gives the normalised projection back
    assert not torch.allclose(q.transpose(1, 2).flatten(2, 3).float(), attn.norm_q(attn.to_q(x)).float(), atol=1e-2)
    torch.manual_seed(123)
    o_ref, _ = _oracle_attention(q, k, v, module, H)
    with torch.no_grad():
        expect = attn.to_out[0](o_ref.to(DEV).transpose(1, 2).flatten(2, 3))
    assert cosine(out, expect) >= 0.999
    assert float((out.float() - expect.float()).abs().max()) <= 3e-2 * max(1.0, float(expect.float().abs().max()))
    module.close_logger()          # also asks the device status word: no bounded wait expired


def test_cogvideox_processor_pipeline_vs_oracle():
    from psa_b200.presets import SparseCogVideoXAttnProcessor
    B, H, D, grid, text = 1, 2, 64, (15, 12, 5), 226
    n_video = grid[0] * grid[1] * grid[2]
    attn = _attn(H * D, H, per_head_norm=True)
    module = _module(grid, text, True)
    attn.inner_attention = _Tap(module)
    video = C.randn(71, (B, n_video, H * D), torch.bfloat16, smooth=8).to(DEV)
    words = C.randn(72, (B, text, H * D), torch.bfloat16).to(DEV)
    ang = torch.rand(n_video, D // 2, generator=torch.Generator().manual_seed(10)) * 6.28
    rot = (torch.cos(ang).repeat_interleave(2, -1).to(DEV), torch.sin(ang).repeat_interleave(2, -1).to(DEV))
    torch.manual_seed(321)
    with torch.no_grad():
        out_video, out_text = SparseCogVideoXAttnProcessor(0)(attn, video, words, image_rotary_emb=rot)
    q, k, v = attn.inner_attention.seen
    assert q.shape == (B, H, text + n_video, D)
    torch.manual_seed(321)
    o_ref, _ = _oracle_attention(q, k, v, module, H)
    with torch.no_grad():
        expect = attn.to_out[0](o_ref.to(DEV).transpose(1, 2).reshape(B, -1, H * D))
    got = torch.cat([out_text, out_video], dim=1)
    assert cosine(got, expect) >= 0.999
    assert float((got.float() - expect.float()).abs().max()) <= 3e-2 * max(1.0, float(expect.float().abs().max()))
