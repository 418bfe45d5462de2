"""GPU: rotary embedding applied inside the loads of the token-major route.  The kernels that read q or k rows rotate
them on the way; everything must equal, bit for bit, the same calls on copies rotated beforehand with the framework's
element-wise operations (what the processors of modify_diffusers.py:260-281 and :363-369 produce)."""
import pytest
import torch

import cases as C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tables(S, first, D, seed):
    ang = torch.rand(S - first, D, generator=torch.Generator().manual_seed(seed)) * 6.28
    return torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D,first,reorder", [(128, 0, False), (128, 0, True), (64, 226, True), (128, 40, False)])
def test_rotating_loads_equal_rotated_copies(dtype, D, first, reorder):
    from psa_b200 import ops
    S, H = 1000 + first, 3
    q, k, v = (C.randn(80 + i, (S, H, D), dtype, smooth=4).to(DEV) for i in range(3))
    a, b = _tables(S, first, D, 7)
    rope = ops.RotaryTables(a, b, first)
    perm = torch.randperm(S, generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV) if reorder else None

    def rotated(x):       # [S, H, D] -> rotated copy, same layout
        return ops.rotate_rows(x.transpose(0, 1)[None], rope)[0].transpose(0, 1).contiguous()

    q_r, k_r = rotated(q), rotated(k)
    assert not torch.equal(q_r[first:], q[first:]) and torch.equal(q_r[:first], q[:first])
    assert torch.equal(ops.gather_heads(q, perm, rope=rope), ops.gather_heads(q_r, perm))
    fused, plain = ops.pyramid_kv_images_tm(k, v, 64, perm=perm, rope=rope), ops.pyramid_kv_images_tm(k_r, v, 64, perm=perm)
    assert torch.equal(fused.kimg, plain.kimg) and torch.equal(fused.vimg, plain.vimg)
    iq, ik = C.sample_idx(41, 1, H, 128, 32)[0].to(DEV), C.sample_idx(42, 1, H, 64, 16)[0].to(DEV)
    assert torch.equal(ops.block_scores_tm(q, k, iq, ik, 128, 64, perm=perm, rope=rope),
                       ops.block_scores_tm(q_r, k_r, iq, ik, 128, 64, perm=perm))


def test_layer_with_fused_rotation_equals_layer_on_rotated_inputs():
    import psa_b200
    from psa_b200 import ops
    from psa_b200.attention import psa_attention_token_major
    B, S, H, D, first = 1, 2048 + 64, 2, 128, 64
    q, k, v = (C.randn(90 + i, (B, S, H, D), torch.bfloat16, smooth=8).to(DEV) for i in range(3))
    a, b = _tables(S, first, D, 11)
    rope = ops.RotaryTables(a, b, first)
    cfg = psa_b200.PSAConfig(block_m=128, block_n=64, tile_n=32, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk")
    perm = torch.randperm(S, generator=torch.Generator().manual_seed(6)).to(torch.int32).to(DEV)
    iq, ik = C.sample_idx(41, B, H, 128, 32).to(DEV), C.sample_idx(42, B, H, 64, 16).to(DEV)
    q_r = ops.rotate_rows(q.transpose(1, 2), rope).transpose(1, 2).contiguous()
    k_r = ops.rotate_rows(k.transpose(1, 2), rope).transpose(1, 2).contiguous()
    out_f, mask_f = psa_attention_token_major(q, k, v, cfg, perm=perm, idx_q=iq, idx_k=ik, rope=rope)
    out_p, mask_p = psa_attention_token_major(q_r, k_r, v, cfg, perm=perm, idx_q=iq, idx_k=ik)
    ops.check_status()
    assert torch.equal(mask_f, mask_p)
    assert torch.equal(out_f, out_p)


def test_wan_processor_hands_unrotated_rows_to_a_module_that_rotates_in_its_kernels(monkeypatch):
    """Processor -> module with the Gilbert order folded in: with the module's `fuses_rotary` visible the processor
    passes q, k unrotated plus the tables; hidden behind a plain wrapper it rotates them itself.  Same bits."""
    from psa_b200 import ops
    from psa_b200.presets import SparseWanAttnProcessor
    from test_gpu_processors import _Tap, _attn, _module
    B, H, D, grid = 1, 2, 64, (16, 16, 8)
    S = grid[0] * grid[1] * grid[2]
    attn = _attn(H * D, H, per_head_norm=False)
    module = _module(grid, 0, True)
    x = C.randn(70, (B, S, H * D), torch.bfloat16, smooth=8).to(DEV)
    ang = torch.rand(1, S, 1, D // 2, generator=torch.Generator().manual_seed(9)) * 6.28
    rot = (torch.cos(ang).repeat_interleave(2, -1).to(DEV), torch.sin(ang).repeat_interleave(2, -1).to(DEV))
    fused_calls = []
    real = ops.gather_heads
    monkeypatch.setattr(ops, "gather_heads", lambda t, perm=None, rope=None: (fused_calls.append(rope is not None), real(t, perm, rope=rope))[1])
    proc = SparseWanAttnProcessor(0)
    outs = []
    for inner in (module, _Tap(module)):
        attn.inner_attention = inner
        torch.manual_seed(123)
        with torch.no_grad():
            outs.append(proc(attn, x, rotary_emb=rot))
    ops.check_status()
    assert fused_calls == [True, False], fused_calls
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("first,reorder", [(0, False), (226, True)])
def test_head_major_rotating_loads_equal_rotated_copies(first, reorder):
    """The same three loads for head-major tensors [B, H, S, D] (what the CogVideoX processor holds after its per-head
    norms): rows read through an optional order table and rotated on the way."""
    from psa_b200 import ops
    B, H, D = 1, 3, 64
    S = 1000 + first
    q, k, v = (C.randn(60 + i, (B, H, S, D), torch.bfloat16, smooth=4).to(DEV) for i in range(3))
    a, b = _tables(S, first, D, 17)
    rope = ops.RotaryTables(a, b, first)
    perm = torch.randperm(S, generator=torch.Generator().manual_seed(5)).to(torch.int32).to(DEV) if reorder else None
    q_r, k_r = ops.rotate_rows(q, rope), ops.rotate_rows(k, rope)
    want_q = ops.gather_rows(q_r, perm) if reorder else q_r
    assert torch.equal(ops.gather_rows(q, perm, rope=rope), want_q)
    fused, plain = ops.pyramid_kv_images(k, v, 64, perm=perm, rope=rope), ops.pyramid_kv_images(k_r, v, 64, perm=perm)
    assert torch.equal(fused.kimg, plain.kimg) and torch.equal(fused.vimg, plain.vimg)
    iq, ik = C.sample_idx(41, B, H, 128, 32).to(DEV), C.sample_idx(42, B, H, 64, 16).to(DEV)
    assert torch.equal(ops.block_scores(q, k, iq, ik, 128, 64, perm_q=perm, perm_k=perm, rope=rope),
                       ops.block_scores(q_r, k_r, iq, ik, 128, 64, perm_q=perm, perm_k=perm))


def test_cogvideox_processor_hands_unrotated_head_major_rows_to_the_module(monkeypatch):
    """CogVideoX: text tokens first, per-head norms (head-major q, k), rotary tables for the video tokens only.  With the
    module's `fuses_rotary` visible the processor passes q, k unrotated; behind a plain wrapper it rotates them itself."""
    from psa_b200 import ops
    from psa_b200.presets import SparseCogVideoXAttnProcessor
    from test_gpu_processors import _Tap, _attn, _module
    B, H, D, grid, n_text = 1, 2, 64, (16, 16, 8), 226
    S = grid[0] * grid[1] * grid[2]
    attn = _attn(H * D, H, per_head_norm=True)
    module = _module(grid, n_text, True)
    hidden = C.randn(71, (B, S, H * D), torch.bfloat16, smooth=8).to(DEV)
    text = C.randn(72, (B, n_text, H * D), torch.bfloat16).to(DEV)
    ang = (torch.rand(S, D // 2, generator=torch.Generator().manual_seed(9)) * 6.28).repeat_interleave(2, -1)
    rot = (torch.cos(ang).to(DEV), torch.sin(ang).to(DEV))
    fused_calls = []
    real = ops.gather_rows
    monkeypatch.setattr(ops, "gather_rows", lambda t, perm, rope=None: (fused_calls.append(rope is not None), real(t, perm, rope=rope))[1])
    proc = SparseCogVideoXAttnProcessor(0)
    outs = []
    for inner in (module, _Tap(module)):
        attn.inner_attention = inner
        torch.manual_seed(123)
        with torch.no_grad():
            outs.append(proc(attn, hidden, text, image_rotary_emb=rot))
    ops.check_status()
    assert fused_calls == [True, False], fused_calls
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
