"""GPU: the token reordering folded into the kernels (row tables read in place) against reordering with copies.

Every comparison is bit for bit: the kernels do the same arithmetic on the same values, only the addresses differ.  The
copy-based path they are compared with is itself checked against the CPU oracle in test_gpu_parity.py; the module test
here also compares with the oracle composed with the reordering."""
import pytest
import torch

import cases as C
from oracle import psa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def P():
    import psa_b200
    assert torch.cuda.is_available()
    return psa_b200


def _perm(seed, n):
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(n, generator=g).to(torch.int32)


@pytest.mark.parametrize("dt,D,S", [(torch.bfloat16, 128, 1000), (torch.float16, 64, 333), (torch.float32, 64, 130),
                                    (torch.bfloat16, 64, 1)])
def test_gather_rows(P, dt, D, S):
    x = C.randn(5, (2, 3, S, D), dt).to(DEV)
    perm = _perm(1, S).to(DEV)
    assert torch.equal(P.ops.gather_rows(x, perm), x.index_select(2, perm.long()))


def test_gather_rows_rejects_bad_tables(P):
    x = C.randn(5, (1, 1, 64, 64), torch.bfloat16).to(DEV)
    with pytest.raises(ValueError):
        P.ops.gather_rows(x, _perm(1, 63).to(DEV))
    with pytest.raises(ValueError):
        P.ops.gather_rows(x, _perm(1, 64).long().to(DEV))


@pytest.mark.parametrize("dt,D,S,bn", [(torch.bfloat16, 128, 1000, 64), (torch.float16, 64, 777, 128), (torch.bfloat16, 64, 64, 64)])
def test_tile_images_through_row_table(P, dt, D, S, bn):
    k = C.randn(11, (1, 3, S, D), dt).to(DEV)
    v = C.randn(12, (1, 3, S, D), dt).to(DEV)
    perm = _perm(2, S).to(DEV)
    a = P.ops.pyramid_kv_images(k, v, bn, perm=perm)
    b = P.ops.pyramid_kv_images(k.index_select(2, perm.long()), v.index_select(2, perm.long()), bn)
    assert torch.equal(a.kimg, b.kimg) and torch.equal(a.vimg, b.vimg)


@pytest.mark.parametrize("dt,D,S,bn", [(torch.bfloat16, 128, 1000, 64), (torch.float16, 64, 777, 128)])
def test_block_scores_through_row_table(P, dt, D, S, bn):
    H = 3
    q, k, _ = C.qkv(100, 1, H, S, D, dt)
    q, k = q.to(DEV), k.to(DEV)
    iq, ik = C.sample_idx(7, 1, H, 128, 32).to(DEV), C.sample_idx(8, 1, H, bn, bn // 4).to(DEV)
    perm = _perm(3, S).to(DEV)
    a = P.ops.block_scores(q, k, iq, ik, 128, bn, perm_q=perm, perm_k=perm)
    b = P.ops.block_scores(q.index_select(2, perm.long()), k.index_select(2, perm.long()), iq, ik, 128, bn,
                           impl=P.ops.IMPL_TENSOR)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dt,D,S,bn", [(torch.bfloat16, 128, 1000, 64), (torch.float16, 64, 777, 128)])
def test_forward_stores_rows_through_table(P, dt, D, S, bn):
    from psa_b200.attention import PSAConfig, compute_block_mask
    H = 2
    q, k, v = (x.to(DEV) for x in C.qkv(200, 1, H, S, D, dt))
    cfg = PSAConfig(block_m=128, block_n=bn, tile_n=32, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk")
    torch.manual_seed(5)
    mask, _, _ = compute_block_mask(q, k, cfg)
    perm = _perm(4, S).to(DEV)
    plain = P.ops.psa_forward(q, k, v, mask, 128, bn, 32)
    moved = P.ops.psa_forward(q, k, v, mask, 128, bn, 32, out_perm=perm)
    assert int(moved._psa_status.item()) == 0
    assert torch.equal(moved.index_select(2, perm.long()), plain)


@pytest.mark.parametrize("text", [0, 37])
def test_module_reorders_in_place(P, text):
    """PyramidSparseAttention with the Gilbert order on 16-bit inputs takes the in-place route; its output equals the
    route with four reordering copies bit for bit (same sample offsets), and the oracle composed the same way."""
    from psa_b200.attention import compute_block_mask
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    W, Hh, T, H, D = 12, 8, 9, 2, 128                      # 864 video tokens (+ text)
    cfg = AttentionConfig(width=W, height=Hh, depth=T, text_length=text, use_rearrange=True, rearrange_method="Gilbert",
                          block_m=128, block_n=64, tile_n=32, use_sim_mask=False, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk",
                          warmup_steps=0, attn_impl="new_mask_type")
    mod = PyramidSparseAttention(cfg, inference_num=10, layer_num=1, model_type="cogvideo")
    S = W * Hh * T + text
    q, k, v = C.qkv(991, 1, H, S, D, torch.bfloat16)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    assert mod._rows_in_place(qd, kd)
    torch.manual_seed(321)
    fused = mod(qd, kd, vd, 0)
    # the same layer with explicit copies
    torch.manual_seed(321)
    qr, kr, vr = mod.gilbert_rearranger.rearrange(qd, kd, vd)
    mask, _, _ = compute_block_mask(qr, kr, cfg, text_length=text)
    o = P.ops.psa_forward(qr.contiguous(), kr.contiguous(), vr.contiguous(), mask, 128, 64, 32)
    copied = mod.gilbert_rearranger.reversed_rearrange(o)
    assert torch.equal(fused, copied)
    # the oracle's forward on the reordered 16-bit inputs and the same level mask, reordered back
    qc, kc, vc = mod.gilbert_rearranger.rearrange(q, k, v)
    oo = O.psa_forward_newmask(qc, kc, vc, mask.cpu(), 128, 64, 32).float()
    ref = mod.gilbert_rearranger.reversed_rearrange(oo)
    assert float((fused.float().cpu() - ref).abs().max()) <= 2e-2
    a, b = fused.float().cpu().double().flatten(), ref.double().flatten()
    assert float((a @ b) / (a.norm() * b.norm())) >= 0.999
    assert mod.logger.records[0]["density"].shape == (1, H)


def test_similarity_cap_through_a_row_table(P):
    """psa_ksim_perm: the cap of k[..., perm, :] read in place equals the cap of the reordered copy (thresholds at 0, where
    the mean cosines of these keys fall on both sides)."""
    S, H, D = 1000, 3, 64
    k = C.randn(17, (1, H, S, D), torch.bfloat16, smooth=4).to(DEV)
    perm = _perm(9, S).to(DEV)
    for bn in (128, 64, 32):
        a = P.ops.k_similarity(k, bn, 0.0, 0.0, 0.0, perm=perm)
        b = P.ops.k_similarity(k[:, :, perm.long()].contiguous(), bn, 0.0, 0.0, 0.0)
        assert torch.equal(a, b)
        assert len(torch.unique(b)) > 1


@pytest.mark.parametrize("text,sim", [(0, True), (37, True), (226, False)])
def test_module_reorders_in_place_old_format(P, text, sim):
    """The presets with the old mask format (block 128, thresholdbound, similarity cap - the default preset of the Wan
    2.1 1.3B pipeline) also skip the four reordering copies: the similarity cap, the scores and the tile images read k
    through the row table, only q is gathered, the legacy forward stores its rows back through the table.  Bit-identical
    to the copy route; and the oracle's legacy forward on the reordered inputs agrees."""
    from psa_b200.attention import compute_block_mask
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    W, Hh, T, H, D = 12, 8, 9, 2, 128
    cfg = AttentionConfig(width=W, height=Hh, depth=T, text_length=text, use_rearrange=True, rearrange_method="Gilbert",
                          block_m=128, block_n=128, tile_n=32, use_sim_mask=sim, mask_ratios=C.RATIOS_THR, mask_mode="thresholdbound",
                          warmup_steps=0, attn_impl="old_mask_type", sim_2x_threshold=0.7, sim_4x_threshold=0.65,
                          sim_8x_threshold=0.6)
    mod = PyramidSparseAttention(cfg, inference_num=10, layer_num=1, model_type="wan")
    S = W * Hh * T + text
    q, k, v = C.qkv(993, 1, H, S, D, torch.bfloat16, smooth=16)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    assert mod._rows_in_place_old_format(qd, kd)
    torch.manual_seed(77)
    fused = mod(qd, kd, vd, 0)
    assert int(fused._psa_status.item()) == 0
    # the same layer with explicit copies
    torch.manual_seed(77)
    qr, kr, vr = mod.gilbert_rearranger.rearrange(qd, kd, vd)
    mask, _, simm = compute_block_mask(qr.contiguous(), kr.contiguous(), cfg, text_length=text)
    o, _, _ = P.ops.legacy_forward(qr.contiguous(), kr.contiguous(), vr.contiguous(), mask, False)
    copied = mod.gilbert_rearranger.reversed_rearrange(o)
    assert torch.equal(fused, copied)
    assert (simm is not None) == sim
    qc, kc, vc = mod.gilbert_rearranger.rearrange(q, k, v)
    oo, _ = O.legacy_forward(qc, kc, vc, mask.cpu(), False)
    ref = mod.gilbert_rearranger.reversed_rearrange(oo.float())
    assert float((fused.float().cpu() - ref).abs().max()) <= 2e-2
    a, b = fused.float().cpu().double().flatten(), ref.double().flatten()
    assert float((a @ b) / (a.norm() * b.norm())) >= 0.999


# ------------------------------------------------------------------ token-major tensors ----------------
@pytest.mark.parametrize("with_perm", [False, True])
def test_gather_heads(P, with_perm):
    S, H, D = 517, 3, 64
    x = C.randn(6, (S, H, D), torch.bfloat16).to(DEV)
    perm = _perm(8, S).to(DEV) if with_perm else None
    ref = x.transpose(0, 1)
    if with_perm:
        ref = ref.index_select(1, perm.long())
    assert torch.equal(P.ops.gather_heads(x, perm)[0], ref)


@pytest.mark.parametrize("with_perm", [False, True])
@pytest.mark.parametrize("dt,D,S,bn,B", [(torch.bfloat16, 128, 1000, 64, 2), (torch.float16, 64, 777, 128, 1)])
def test_token_major_layer_equals_head_major(P, dt, D, S, bn, B, with_perm):
    from psa_b200.attention import PSAConfig, compute_block_mask, psa_attention_token_major
    H = 3
    qs, ks, vs = zip(*(C.qkv(300 + b, 1, H, S, D, dt) for b in range(B)))
    q, k, v = (torch.cat(x, 0).to(DEV) for x in (qs, ks, vs))            # [B, H, S, D]
    q_tm, k_tm, v_tm = (x.transpose(1, 2).contiguous() for x in (q, k, v))   # [B, S, H, D]
    cfg = PSAConfig(block_m=128, block_n=bn, tile_n=32, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk")
    iq = torch.cat([C.sample_idx(7 + b, 1, H, 128, 32) for b in range(B)], 0).to(DEV)
    ik = torch.cat([C.sample_idx(17 + b, 1, H, bn, bn // 4) for b in range(B)], 0).to(DEV)
    perm = _perm(9, S).to(DEV) if with_perm else None
    out_tm, mask_tm = psa_attention_token_major(q_tm, k_tm, v_tm, cfg, perm=perm, idx_q=iq, idx_k=ik)
    # head-major, with copies
    if with_perm:
        qr, kr, vr = (x.index_select(2, perm.long()) for x in (q, k, v))
    else:
        qr, kr, vr = q, k, v
    mask, _, _ = compute_block_mask(qr, kr, cfg, idx_q=iq, idx_k=ik)
    assert torch.equal(mask_tm, mask)
    o = P.ops.psa_forward(qr, kr, vr, mask, 128, bn, 32)
    if with_perm:
        back = torch.empty_like(o)
        back[:, :, perm.long()] = o
        o = back
    assert torch.equal(out_tm, o.transpose(1, 2))


def test_module_reads_transposed_views_in_place(P):
    """Handed q.transpose(1, 2) views of [B, S, H, D] tensors (what the diffusers processors pass), the module returns a
    view of a token-major output: the same values as for contiguous head-major inputs, no transposed copy on either side."""
    from psa_b200.pyramid_sparse_attention import AttentionConfig, PyramidSparseAttention
    W, Hh, T, H, D, text = 12, 8, 9, 2, 128, 20
    cfg = AttentionConfig(width=W, height=Hh, depth=T, text_length=text, use_rearrange=True, rearrange_method="Gilbert",
                          block_m=128, block_n=64, tile_n=32, use_sim_mask=False, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk",
                          warmup_steps=0, attn_impl="new_mask_type")
    mod = PyramidSparseAttention(cfg, inference_num=10, layer_num=1, model_type="cogvideo")
    q, k, v = (x.to(DEV) for x in C.qkv(992, 1, H, W * Hh * T + text, D, torch.bfloat16))
    torch.manual_seed(55)
    a = mod(q, k, v, 0)                                                     # head-major, contiguous
    q_tm, k_tm, v_tm = (x.transpose(1, 2).contiguous() for x in (q, k, v))
    torch.manual_seed(55)
    b = mod(q_tm.transpose(1, 2), k_tm.transpose(1, 2), v_tm.transpose(1, 2), 0)
    assert b.shape == a.shape and b.transpose(1, 2).is_contiguous()
    assert torch.equal(a, b)


# ------------------------------------------------------------------ host buffers, pipelined by head chunks ----------
@pytest.mark.parametrize("H,hc", [(5, 2), (4, 0), (3, 8)])
def test_host_buffer_layer_equals_device_layer(P, H, hc):
    """psa_attention_host (pinned host tensors in and out, head chunks with overlapped copies) gives the bits of
    PSAAttention on device copies: ragged last chunk, default chunking, one chunk."""
    S, D = 900, 128
    q, k, v = (x.pin_memory() for x in C.qkv(410, 1, H, S, D, torch.bfloat16))
    cfg = P.PSAConfig(block_m=128, block_n=64, tile_n=32, mask_ratios=C.DEFAULT_RATIOS, mask_mode="topk")
    torch.manual_seed(31)
    out = P.psa_attention_host(q, k, v, cfg, device=DEV, heads_per_chunk=hc)
    torch.cuda.synchronize()
    torch.manual_seed(31)
    ref = P.PSAAttention(cfg)(q.to(DEV), k.to(DEV), v.to(DEV))
    assert out.is_pinned() and torch.equal(out, ref.cpu())
    # a second call into the same output buffer, explicit offsets
    iq, ik = C.sample_idx(7, 1, H, 128, 32).to(DEV), C.sample_idx(8, 1, H, 64, 16).to(DEV)
    out2 = P.psa_attention_host(q, k, v, cfg, out=out, device=DEV, heads_per_chunk=hc, idx_q=iq, idx_k=ik)
    torch.cuda.synchronize()
    assert out2 is out
    assert torch.equal(out2, P.PSAAttention(cfg)(q.to(DEV), k.to(DEV), v.to(DEV), idx_q=iq, idx_k=ik).cpu())


def test_host_buffer_layer_rejects_pageable_memory(P):
    q, k, v = C.qkv(410, 1, 2, 256, 64, torch.bfloat16)
    with pytest.raises(ValueError):
        P.psa_attention_host(q, k, v, device=DEV)
