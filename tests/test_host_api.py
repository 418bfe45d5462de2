"""CPU: host-side logic that needs no GPU - Gilbert order, presets, installer wiring, interval arithmetic."""
import numpy as np
import pytest
import torch

import cases as C
from oracle import psa_oracle as O


@pytest.mark.parametrize("shape", C.GILBERT_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gilbert_order_matches_reference_curve(golden, shape):
    from psa_b200.rearrange import gilbert_order
    w, h, d = shape
    order = gilbert_order(w, h, d)
    assert sorted(order.tolist()) == list(range(w * h * d))
    assert C.order_checksum(order) == int(golden[f"gilbert_sum_{w}x{h}x{d}"][0])
    key = f"gilbert_{w}x{h}x{d}"
    if key in golden.files:
        assert np.array_equal(order, golden[key])


def test_gilbert_rearranger_round_trip_with_text():
    from psa_b200.rearrange import GilbertRearranger
    r = GilbertRearranger(6, 4, 3, text_length=5)
    x = torch.arange(2 * (5 + 72) * 3, dtype=torch.float32).view(1, 2, 77, 3)
    q, k, v = r.rearrange(x, x + 1, x + 2)
    assert torch.equal(q[..., -5:, :], x[..., :5, :])                 # text moved to the end
    assert torch.equal(r.reversed_rearrange(q), x)
    assert torch.equal(r.reversed_rearrange(v), x + 2)
    # the row table the kernels read: gathering through it is rearrange_single, scattering through it is the inverse
    rows = r.source_rows("cpu").long()
    assert torch.equal(x.index_select(-2, rows), q)
    back = torch.empty_like(q)
    back[..., rows, :] = q
    assert torch.equal(back, x)
    r0 = GilbertRearranger(6, 4, 3, text_length=0)
    y = x[..., :72, :]
    assert torch.equal(r0.reversed_rearrange(r0.rearrange_single(y)), y)


def test_preset_loader_values_and_errors():
    from psa_b200.presets import WanAttentionConfigLoader
    L = WanAttentionConfigLoader()
    assert set(L.list_presets("Wan2.1_1.3b")) == {"baseline", "psa_balanced", "psa_topk"}
    info = L.get_attention_config("Wan2.1_1.3b", "psa_topk", [832, 480, 81])
    p = info["params"]
    assert (p["width"], p["height"], p["depth"]) == (52, 30, 21)
    assert (p["block_m"], p["block_n"], p["tile_n"]) == (128, 32, 32)
    assert p["mask_ratios"] == C.RATIOS_90 and p["mask_mode"] == "topk" and p["warmup_steps"] == 15
    d = L.get_attention_config("Wan2.1_1.3b", None, [832, 480, 81])["params"]       # default preset
    assert d["attn_impl"] == "old_mask_type" and d["use_sim_mask"] and d["sim_2x_threshold"] == 0.7
    c = L.get_attention_config("CogVideo_5b", "psa_balanced", [720, 480, 49])["params"]
    assert c["text_length"] == 226 and not c["use_rearrange"] and (c["width"], c["height"], c["depth"]) == (45, 30, 13)
    assert L.get_attention_config("Wan2.1_14b", "baseline", [1280, 720, 81])["type"] == "dense"
    for bad in (lambda: L.get_attention_config("Wan2.1_1.3b_4steps", None, [1, 1, 1]),
                lambda: L.get_attention_config("Wan2.1_14b", "nope", [1, 1, 1]),
                lambda: L.get_attention_config("Wan2.1_14b", None, [1, 1])):
        with pytest.raises(ValueError):
            bad()


class _Attn:
    def __init__(self):
        self.processor = None
        self.inner_attention = None

    def set_processor(self, p):
        self.processor = p


class _Block:
    def __init__(self):
        self.attn1 = _Attn()


class _Transformer:
    def __init__(self, n):
        self.blocks = [_Block() for _ in range(n)]


class _Pipe:
    def __init__(self, n, two=False):
        self.transformer = _Transformer(n)
        self.transformer_2 = _Transformer(n) if two else None


def test_installer_shares_one_module_and_dense_preset_is_a_no_op():
    from psa_b200.presets import set_adaptive_sparse_attention, reset_wan_attention_to_dense
    pipe = _Pipe(4, two=True)
    info = set_adaptive_sparse_attention(pipe, "Wan2.2_A14B", inference_num=40, video_shape=[832, 480, 81])
    mod = pipe.transformer.blocks[0].attn1.inner_attention
    assert info["type"] == "psa" and mod is not None and mod.layer_num == 4 and mod.inference_num == 40
    mods = {id(b.attn1.inner_attention) for t in (pipe.transformer, pipe.transformer_2) for b in t.blocks}
    assert mods == {id(mod)}
    assert [b.attn1.processor.layer_idx for b in pipe.transformer.blocks] == [0, 1, 2, 3]
    assert mod.config.block_n == 32 and mod.config.mask_mode == "thresholdbound" and mod.gilbert_rearranger is not None
    reset_wan_attention_to_dense(pipe)
    assert all(b.attn1.inner_attention is None for b in pipe.transformer.blocks)
    pipe2 = _Pipe(2)
    assert set_adaptive_sparse_attention(pipe2, "Wan2.1_14b", video_shape=[832, 480, 81], attention_preset="baseline")["type"] == "dense"
    assert pipe2.transformer.blocks[0].attn1.processor is None
    with pytest.raises(ValueError):
        set_adaptive_sparse_attention(pipe2, "NotAModel", video_shape=[1, 1, 1])


def test_warmup_schedule_follows_the_reference_counter_rule():
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    cfg = AttentionConfig(use_rearrange=False, use_sim_mask=False, warmup_steps=2, enable_logging=False)
    wan = PyramidSparseAttention(cfg, inference_num=5, layer_num=3, model_type="wan")
    cog = PyramidSparseAttention(cfg, inference_num=5, layer_num=3, model_type="cogvideo")
    times_wan, times_cog = [], []
    for _ in range(40):
        times_wan.append(wan.get_current_time()); wan.sparsity_counter += 1
        times_cog.append(cog.get_current_time()); cog.sparsity_counter += 1
    assert times_wan[:13] == [0] * 6 + [1] * 6 + [2]          # two CFG passes per step: 2 * layer_num calls per step
    assert times_cog[:7] == [0] * 3 + [1] * 3 + [2]
    assert times_cog[15] == 0                                 # wraps after inference_num steps
    with pytest.raises(ValueError):
        AttentionConfig()                                      # default new_mask_type + use_sim_mask=True is rejected
    with pytest.raises(NotImplementedError):
        PyramidSparseAttention(AttentionConfig(use_sim_mask=False, rearrange_method="STA"))


def test_topk_intervals_host_arithmetic_equals_oracle():
    from psa_b200.ops import topk_intervals
    for nk in (1, 9, 37, 64, 139, 278, 512, 1182, 2363):
        for bn in (32, 64, 128):
            for ratios in (C.DEFAULT_RATIOS, C.RATIOS_90, C.RATIOS_DENSE, C.RATIOS_THR):
                for newtype in (True, False):
                    mine = [(l, s, e) for l, s, e in topk_intervals(nk, ratios, bn, 32, newtype) if newtype or s < e]
                    assert mine == O.topk_intervals(nk, ratios, bn, 32, newtype)


def test_sparsity_log_writes_jsonl(tmp_path):
    """The per-call records (densities as tensors, None for warm-up calls) become one JSON line each."""
    import json
    from psa_b200.pyramid_sparse_attention import SparsityLog
    log = SparsityLog()
    log.log_sparsity(layer_idx=0, density=None, sequence_length=640, batch_size=1, num_heads=2, is_warmup=True)
    log.log_sparsity(layer_idx=1, density=torch.tensor([[0.25, 0.75]]), sequence_length=640, batch_size=1, num_heads=2,
                     is_warmup=False)
    path = tmp_path / "logs" / "sparsity.jsonl"
    assert log.write_jsonl(str(path)) == 2
    lines = [json.loads(x) for x in path.read_text().splitlines()]
    assert lines[0]["is_warmup"] and lines[0]["per_head_density"] == [] and lines[0]["density"] == 1.0
    assert lines[1]["per_head_density"] == [0.25, 0.75] and lines[1]["density"] == 0.5 and lines[1]["sparsity"] == 0.5
    assert lines[1]["global_step"] == 1 and lines[1]["layer_idx"] == 1


# ---------------------------------------------------------------------------------------------------------------------
# The diffusers attention processors on stand-in attention modules (linear layers, norms, a recording inner_attention).
class _Recorder:
    def __init__(self):
        self.calls = []

    def __call__(self, q, k, v, layer_idx):
        self.calls.append((q.clone(), k.clone(), v.clone(), layer_idx))
        return q + 0.5 * v          # any function of the operands: the processors must pass it on untouched


class _RMS(torch.nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.linspace(0.5, 1.5, dim))

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * self.weight


def _stub_attn(hidden, heads, *, per_head_norm=False, fused=False, image=False, seed=0):
    torch.manual_seed(seed)
    a = torch.nn.Module()
    a.heads = heads
    a.to_q, a.to_k, a.to_v = (torch.nn.Linear(hidden, hidden) for _ in range(3))
    a.norm_q = _RMS(hidden // heads if per_head_norm else hidden)
    a.norm_k = _RMS(hidden // heads if per_head_norm else hidden)
    a.to_out = torch.nn.ModuleList([torch.nn.Linear(hidden, hidden), torch.nn.Identity()])
    a.add_k_proj = a.add_v_proj = None
    a.is_cross_attention = False
    a.cross_attention_dim_head = None
    a.fused_projections = fused
    if fused:
        a.to_qkv = torch.nn.Linear(hidden, 3 * hidden)
        with torch.no_grad():
            a.to_qkv.weight.copy_(torch.cat([a.to_q.weight, a.to_k.weight, a.to_v.weight]))
            a.to_qkv.bias.copy_(torch.cat([a.to_q.bias, a.to_k.bias, a.to_v.bias]))
    if image:
        a.add_k_proj, a.add_v_proj = torch.nn.Linear(hidden, hidden), torch.nn.Linear(hidden, hidden)
        a.norm_added_k = _RMS(hidden)
    a.inner_attention = _Recorder()
    return a


def _rotate_pairs(x, cos_half, sin_half):
    """(x0 + i x1) * (cos + i sin) on neighbouring channel pairs, written with complex numbers."""
    z = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2).contiguous())
    return torch.view_as_real(z * torch.complex(cos_half.float(), sin_half.float())).flatten(-2)


@pytest.mark.parametrize("fused", [False, True])
def test_wan_processor_rotates_q_and_k_and_passes_head_major_views(fused):
    from psa_b200.presets import SparseWanAttnProcessor
    B, S, H, D = 2, 24, 3, 8
    attn = _stub_attn(H * D, H, fused=fused)
    x = torch.randn(B, S, H * D)
    ang = torch.rand(1, S, 1, D // 2) * 6.28
    # diffusers hands over full-width tables whose neighbouring entries repeat; the processor reads cos at the even
    # and sin at the odd positions
    freqs_cos = torch.cos(ang).repeat_interleave(2, dim=-1)
    freqs_sin = torch.sin(ang).repeat_interleave(2, dim=-1)
    freqs_cos[..., 1::2] += 7.0          # entries the processor must NOT read
    freqs_sin[..., 0::2] -= 7.0
    out = SparseWanAttnProcessor(5)(attn, x, rotary_emb=(freqs_cos, freqs_sin))
    (q, k, v, idx), = attn.inner_attention.calls
    assert idx == 5 and q.shape == (B, H, S, D)
    q_lin = attn.norm_q(attn.to_q(x)).view(B, S, H, D)
    k_lin = attn.norm_k(attn.to_k(x)).view(B, S, H, D)
    assert torch.allclose(q.transpose(1, 2), _rotate_pairs(q_lin, torch.cos(ang), torch.sin(ang)), atol=1e-5)
    assert torch.allclose(k.transpose(1, 2), _rotate_pairs(k_lin, torch.cos(ang), torch.sin(ang)), atol=1e-5)
    assert not torch.allclose(q.transpose(1, 2), q_lin, atol=1e-3)          # un-rotated operands would be a silent bug
    assert torch.allclose(v.transpose(1, 2), attn.to_v(x).view(B, S, H, D), atol=1e-6)
    expect = attn.to_out[0]((q + 0.5 * v).transpose(1, 2).flatten(2, 3))
    assert torch.allclose(out, expect, atol=1e-5)
    # the module's token-major fast path recognises what the processor hands over
    from psa_b200.attention import token_major_view
    q_in = attn.norm_q(attn.to_q(x)).unflatten(2, (H, -1)).transpose(1, 2)
    assert token_major_view(q_in) is not None


def test_wan_processor_image_conditioning_branch_adds_dense_attention_over_image_keys():
    from psa_b200.presets import SparseWanAttnProcessor
    B, S, H, D = 1, 16, 2, 8
    attn = _stub_attn(H * D, H, image=True)
    seen = {}

    def inner(q, k, v, layer_idx):          # cross-attention lengths differ, so this stand-in returns q alone
        seen["k"] = k.shape
        return q
    attn.inner_attention = inner
    x = torch.randn(B, S, H * D)
    ctx = torch.randn(B, 512 + 7, H * D)                  # 7 image tokens in front of the 512 text tokens
    out = SparseWanAttnProcessor(0)(attn, x, encoder_hidden_states=ctx)
    assert seen["k"] == (B, H, 512, D)                    # keys/values of the sparse call come from the text context
    k_img = attn.norm_added_k(attn.add_k_proj(ctx[:, :7])).view(B, 7, H, D).transpose(1, 2)
    v_img = attn.add_v_proj(ctx[:, :7]).view(B, 7, H, D).transpose(1, 2)
    q_lin = attn.norm_q(attn.to_q(x)).view(B, S, H, D).transpose(1, 2)
    p = torch.softmax(q_lin @ k_img.transpose(-1, -2) / D ** 0.5, dim=-1)
    img = (p @ v_img).transpose(1, 2).flatten(2, 3)
    assert torch.allclose(out, attn.to_out[0](q_lin.transpose(1, 2).flatten(2, 3) + img), atol=1e-5)


def test_cogvideox_processor_norms_per_head_and_rotates_video_tokens_only():
    from psa_b200.presets import SparseCogVideoXAttnProcessor
    B, S, T, H, D = 2, 20, 6, 2, 8
    attn = _stub_attn(H * D, H, per_head_norm=True)
    video, text = torch.randn(B, S, H * D), torch.randn(B, T, H * D)
    ang = torch.rand(S, D // 2) * 6.28
    cos, sin = torch.cos(ang).repeat_interleave(2, dim=-1), torch.sin(ang).repeat_interleave(2, dim=-1)
    out_video, out_text = SparseCogVideoXAttnProcessor(3)(attn, video, text, image_rotary_emb=(cos, sin))
    (q, k, v, idx), = attn.inner_attention.calls
    assert idx == 3 and q.shape == (B, H, T + S, D)
    x = torch.cat([text, video], dim=1)
    q_lin = attn.norm_q(attn.to_q(x).view(B, T + S, H, D).transpose(1, 2))      # the norm sees D channels: per head
    k_lin = attn.norm_k(attn.to_k(x).view(B, T + S, H, D).transpose(1, 2))
    assert torch.allclose(q[:, :, :T], q_lin[:, :, :T], atol=1e-6)              # text tokens are not rotated
    assert torch.allclose(k[:, :, :T], k_lin[:, :, :T], atol=1e-6)
    assert torch.allclose(q[:, :, T:], _rotate_pairs(q_lin[:, :, T:], torch.cos(ang), torch.sin(ang)), atol=1e-5)
    assert torch.allclose(k[:, :, T:], _rotate_pairs(k_lin[:, :, T:], torch.cos(ang), torch.sin(ang)), atol=1e-5)
    full = attn.to_out[0]((q + 0.5 * v).transpose(1, 2).reshape(B, T + S, H * D))
    assert torch.allclose(out_video, full[:, T:], atol=1e-5) and torch.allclose(out_text, full[:, :T], atol=1e-5)


def test_installers_use_the_reference_names_and_keep_the_original_processor():
    from psa_b200 import presets
    for name in ("SparseWanAttnProcessor", "SparseCogVideoXAttnProcessor", "set_block_sparse_attn_wan",
                 "set_block_sparse_attn_cogvideox", "set_adaptive_sparse_attention", "reset_wan_attention_to_dense"):
        assert hasattr(presets, name)
    pipe = _Pipe(3)
    for b in pipe.transformer.blocks:
        b.attn1.processor = "stock"
    info = presets.set_adaptive_sparse_attention(pipe, "Wan2.1_1.3b", video_shape=[832, 480, 81], attention_preset="psa_topk")
    assert info["name"] == "psa_topk"
    a0 = pipe.transformer.blocks[0].attn1
    assert isinstance(a0.processor, presets.SparseWanAttnProcessor) and a0.origin_processor == "stock"
    presets.reset_wan_attention_to_dense(pipe)
    assert a0.processor == "stock" and a0.inner_attention is None

    class _Cog:
        def __init__(self, n):
            self.transformer_blocks = [_Block() for _ in range(n)]
    cog = _Cog(2)
    info = presets.set_adaptive_sparse_attention(cog, "CogVideo_5b", video_shape=[720, 480, 49], attention_preset="psa_balanced")
    mod = cog.transformer_blocks[1].attn1.inner_attention
    assert isinstance(cog.transformer_blocks[1].attn1.processor, presets.SparseCogVideoXAttnProcessor)
    assert mod.model_type == "cogvideo" and mod.layer_num == 2 and mod.config.text_length == 226


def test_rotary_tables_of_the_fused_loads_reproduce_both_processor_formulas():
    """ops.rotate_rows (the element-wise statement of what the rotating loads compute) against the two rotary
    formulations of the processors, bit for bit on bf16: Wan (interleaved pairs, cosine at even / sine at odd table
    entries) and CogVideoX (real tables, video tokens only)."""
    from psa_b200 import ops
    from psa_b200.presets import _rotary_tables, rope_interleaved_pairs, rope_real_pairs
    B, H, S, D, n_text = 2, 3, 50, 16, 7
    g = torch.Generator().manual_seed(4)
    x = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    ang = torch.rand(1, S, 1, D, generator=g) * 6.28
    cos, sin = torch.cos(ang), torch.sin(ang)                  # entries differ between the two channels of a pair
    wan = rope_interleaved_pairs(x.transpose(1, 2), cos, sin).transpose(1, 2)
    assert torch.equal(ops.rotate_rows(x, _rotary_tables("wan", cos, sin, 0)), wan)
    ang2 = torch.rand(S - n_text, D // 2, generator=g).repeat_interleave(2, -1) * 6.28
    c2, s2 = torch.cos(ang2), torch.sin(ang2)
    cog = torch.cat([x[:, :, :n_text], rope_real_pairs(x[:, :, n_text:], (c2, s2))], dim=2)
    assert torch.equal(ops.rotate_rows(x, _rotary_tables("real", c2, s2, n_text)), cog)
    assert _rotary_tables("wan", cos.expand(2, S, 1, D), sin.expand(2, S, 1, D), 0) is None   # per-sample tables: not fused
