"""Seeded synthetic video-shaped attention inputs.

Real DiT activations need model weights that are not available offline; these stand in for them.  For every
tensor X in {Q, K, V} and head h a low-frequency random field over the T x H x W token grid is drawn as a sum of 8
sinusoids with random integer wave-vectors in {0..3}^3 \\ {0}, N(0,1) amplitudes and U[0, 2pi) phases per channel,
normalised per (head, channel) to zero mean / unit variance over the grid, tokens in raster order (t, y, x), plus
0.3 * N(0,1) i.i.d. noise.  Optional text tokens ~ N(0,1) are prepended.  The random parameters come from a CPU
generator (identical on every rank and device); the fields are evaluated on the target device.
"""
from __future__ import annotations

import math

import torch

WAN_1_3B = dict(name="wan2.1-1.3b-attn-layer", heads=12, head_dim=128, grid=(21, 30, 52), text=0)
WAN_14B = dict(name="wan2.1-14b-attn-layer", heads=40, head_dim=128, grid=(21, 45, 80), text=0)
COGVIDEOX_5B = dict(name="cogvideox-5b-attn-layer", heads=48, head_dim=64, grid=(13, 30, 45), text=226)
TINY = dict(name="tiny-attn-layer", heads=2, head_dim=64, grid=(4, 32, 32), text=0)
# causal forward + backward of the legacy kernels: batch 2 x 16 heads, 32768 tokens laid out as 8 frames of 64x64
CAUSAL_TRAIN = dict(name="causal-legacy-fwd-bwd", heads=16, head_dim=128, grid=(8, 64, 64), text=0, batch=2)

# the Wan2.1-1.3B layer through the plug-and-play module with the pipeline's DEFAULT preset (old mask format, block 128,
# cumulative-mass thresholds, similarity cap, Gilbert order)
WAN_1_3B_PRESET = dict(name="wan2.1-1.3b-default-preset", heads=12, head_dim=128, grid=(21, 30, 52), text=0,
                       model="Wan2.1_1.3b", video_shape=(832, 480, 81))

# the causal (vision-language prefill) call site: 28 query heads x 128 channels as in Qwen2.5-VL-7B, 32768 tokens
CAUSAL_PREFILL = dict(name="qwen2.5-vl-causal-layer", heads=28, head_dim=128, grid=(8, 64, 64), text=0)
WORKLOADS = {w["name"]: w for w in (WAN_1_3B, WAN_14B, COGVIDEOX_5B, TINY, CAUSAL_TRAIN, WAN_1_3B_PRESET, CAUSAL_PREFILL)}


def structured_field(seed: int, heads: int, head_dim: int, grid, text: int = 0, dtype=torch.bfloat16, device="cpu",
                     head_range=None, token_range=None, noise: float = 0.3) -> torch.Tensor:
    """[1, heads_in_range, tokens_in_range, head_dim].  head_range / token_range select a shard without changing
    the values (every shard of the same seed is a slice of the same global tensor)."""
    T, Hh, W = grid
    n_video = T * Hh * W
    S = text + n_video
    h0, h1 = head_range if head_range is not None else (0, heads)
    s0, s1 = token_range if token_range is not None else (0, S)
    g = torch.Generator().manual_seed(seed)
    freqs = torch.zeros(heads, 8, 3)
    for h in range(heads):
        for i in range(8):
            f = torch.zeros(3)
            while float(f.abs().sum()) == 0:
                f = torch.randint(0, 4, (3,), generator=g).float()
            freqs[h, i] = f
    amp = torch.randn(heads, 8, head_dim, generator=g)
    phase = torch.rand(heads, 8, head_dim, generator=g) * (2 * math.pi)
    out = torch.empty(1, h1 - h0, s1 - s0, head_dim, dtype=dtype, device=device)
    pos = torch.arange(n_video, device=device)
    tt = (pos // (Hh * W)).float() / T
    yy = ((pos // W) % Hh).float() / Hh
    xx = (pos % W).float() / W
    coords = torch.stack([tt, yy, xx], dim=1)                                   # [n_video, 3]
    for h in range(h0, h1):
        theta = 2 * math.pi * coords @ freqs[h].t().to(device)                   # [n_video, 8]
        ca = (amp[h] * torch.cos(phase[h])).to(device)
        sa = (amp[h] * torch.sin(phase[h])).to(device)
        field = torch.cos(theta) @ ca - torch.sin(theta) @ sa                    # [n_video, D]
        field = (field - field.mean(0, keepdim=True)) / field.std(0, keepdim=True).clamp_min(1e-6)
        gn = torch.Generator(device=device).manual_seed(seed * 1000003 + h)
        full = torch.empty(S, head_dim, device=device)
        if text:
            full[:text] = torch.randn(text, head_dim, generator=gn, device=device)
        full[text:] = field + noise * torch.randn(n_video, head_dim, generator=gn, device=device)
        out[0, h - h0] = full[s0:s1].to(dtype)
    return out


def make_qkv(workload: dict, seed: int, dtype=torch.bfloat16, device="cpu", head_range=None, token_range=None):
    kw = dict(heads=workload["heads"], head_dim=workload["head_dim"], grid=workload["grid"], text=workload["text"],
              dtype=dtype, device=device, head_range=head_range, token_range=token_range)
    return tuple(structured_field(seed + i, **kw) for i in range(3))


def seq_len(workload: dict) -> int:
    T, Hh, W = workload["grid"]
    return workload["text"] + T * Hh * W
