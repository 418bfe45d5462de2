"""GPU: the causal (vision-language) call site - antidiagonal estimate, level mask, full layer - through the C ABI
against the reference's fixtures and the CPU oracle."""
import os

import numpy as np
import pytest
import torch

import cases as C
from oracle import psa_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def P():
    import psa_b200
    assert torch.cuda.is_available()
    return psa_b200


@pytest.fixture(scope="module")
def golden_causal():
    return np.load(os.path.join(ROOT, "tests", "golden", "causal_reference_outputs.npz"))


# ------------------------------------------------------------------ level mask: bit exact --------------------
@pytest.mark.parametrize("case", C.CAUSAL_MASK_CASES, ids=lambda c: c[0])
def test_causal_level_mask_golden(P, golden_causal, case):
    name, n, H, dt, mode, causal, text = case
    attn = C.causal_scores(900 + n, H, n, C.DT[dt], causal)
    ratios = C.RATIOS_CAUSAL if mode == "topk" else C.RATIOS_ENERGY
    mask = P.ops.assign_levels_causal(attn.to(DEV), ratios, text, mode, 128, causal).cpu()
    assert torch.equal(mask, torch.from_numpy(golden_causal[name]).to(torch.int32))


@pytest.mark.parametrize("dt", ["bf16", "fp32"])
@pytest.mark.parametrize("mode", ["topk", "energybound"])
def test_causal_level_mask_long_rows_vs_oracle(P, dt, mode):
    n = 300                                                   # 38k tokens at block 128; general + register sort paths
    attn = C.causal_scores(77, 1, n, C.DT[dt], True)
    ratios = C.RATIOS_CAUSAL if mode == "topk" else C.RATIOS_ENERGY
    mask = P.ops.assign_levels_causal(attn.to(DEV), ratios, 512, mode, 128, True).cpu()
    assert torch.equal(mask, O.causal_level_mask(attn, ratios, 512, mode, 128, True))


def test_causal_level_mask_errors(P):
    attn = C.causal_scores(1, 1, 8, torch.bfloat16, True).to(DEV)
    with pytest.raises(ValueError):
        P.ops.assign_levels_causal(attn, {}, 0, "topk", 128, True)
    with pytest.raises(ValueError):
        P.ops.assign_levels_causal(attn, C.RATIOS_CAUSAL, 0, "thresholdbound", 128, True)


# ------------------------------------------------------------------ antidiagonal estimate --------------------
@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("case", C.ANTIDIAG_CASES, ids=lambda c: c[0])
def test_antidiagonal_estimate_vs_oracle(P, golden_causal, case, dt):
    """Against the oracle on the same 16-bit inputs (logits differ only by fp32 accumulation order; the output is rounded
    to the 16-bit type once: tolerance 2^-8 relative to a block's mass), and against the reference's fp32 fixture with
    the looser bound that the 16-bit inputs themselves cause."""
    name, L, D, H, block, stride, chunk, causal = case
    q, k, _ = C.qkv(500, 1, H, L, D, C.DT[dt])
    got = P.ops.antidiag_block_scores(q.to(DEV), k.to(DEV), block, stride, chunk, causal).float().cpu().double()
    ref = O.antidiag_block_scores(q, k, block, stride, causal, chunk)
    rb = block // stride
    assert got.shape == ref.shape
    assert float((got - ref).abs().max()) <= rb * 2.0 ** -8
    fix = torch.from_numpy(golden_causal[name]).double()
    assert float((got - fix).abs().max()) <= 0.05 * rb
    # every valid group row carries a probability mass of one
    n_valid = -(-L // stride)
    rows = torch.tensor([min(rb, n_valid - b * rb) for b in range(ref.shape[-1])], dtype=torch.float64)
    assert float((got.sum(-1) - rows).abs().max()) <= 0.05 * rb


TC_CASES = [  # L (a multiple of the stride), D, H, block, stride, chunk, causal
    (1024, 128, 2, 128, 16, 1024, True),       # one chunk, n = 64 groups: a single partial tile
    (1008, 64, 2, 128, 16, 1024, True),        # 63 valid groups of 64: the last group row is padding
    (4096 + 512, 128, 1, 128, 8, 4096, True),  # two chunks, 576 valid of 1024 groups, 5 row tiles, K = 1024
    (2304, 64, 3, 128, 16, 1024, False),       # not causal: every column tile of the padded length
    (3072, 128, 1, 64, 16, 1024, True),        # 4 groups per block
]


@pytest.mark.parametrize("dt", ["bf16", "fp16"])
@pytest.mark.parametrize("case", TC_CASES, ids=lambda c: f"L{c[0]}_d{c[1]}_s{c[4]}_{'c' if c[6] else 'n'}")
def test_antidiagonal_estimate_tcgen05_vs_oracle_and_warp_mma(P, case, dt):
    """The tcgen05 GEMM (TMA boxes over a 4-D view of q and k) against the oracle on the same 16-bit inputs, and against
    the warp-level mma.sync kernel: both accumulate the same products in fp32, so the rounded masses may differ by one
    unit in the last place of the 16-bit result at most."""
    L, D, H, block, stride, chunk, causal = case
    q, k, _ = C.qkv(510, 1, H, L, D, C.DT[dt])
    qd, kd = q.to(DEV), k.to(DEV)
    tc = P.ops.antidiag_block_scores(qd, kd, block, stride, chunk, causal, impl=P.ops.IMPL_TENSOR)
    assert int(tc._psa_status.item()) == 0
    mma = P.ops.antidiag_block_scores(qd, kd, block, stride, chunk, causal, impl=P.ops.IMPL_WARP_MMA)
    auto = P.ops.antidiag_block_scores(qd, kd, block, stride, chunk, causal)
    assert torch.equal(auto, tc)                                   # a length that divides picks the tcgen05 kernel
    ref = O.antidiag_block_scores(q, k, block, stride, causal, chunk)
    rb = block // stride
    got = tc.float().cpu().double()
    assert got.shape == ref.shape
    assert float((got - ref).abs().max()) <= rb * 2.0 ** -8
    ulp = 2.0 ** -8 if dt == "bf16" else 2.0 ** -11
    assert float((got - mma.float().cpu().double()).abs().max()) <= rb * ulp
    assert torch.equal(P.ops.antidiag_block_scores(qd, kd, block, stride, chunk, causal, impl=P.ops.IMPL_TENSOR), tc)   # repeatable


def test_antidiagonal_estimate_tcgen05_needs_whole_groups(P):
    q, k, _ = C.qkv(500, 1, 1, 1000, 64, torch.bfloat16)
    with pytest.raises(ValueError):
        P.ops.antidiag_block_scores(q.to(DEV), k.to(DEV), 128, 16, 1024, True, impl=P.ops.IMPL_TENSOR)


def test_antidiagonal_estimate_rejects_fp32(P):
    q, k, _ = C.qkv(500, 1, 1, 256, 64, torch.float32)
    with pytest.raises(ValueError):
        P.ops.antidiag_block_scores(q.to(DEV), k.to(DEV), 128, 16, 1024, True)


# ------------------------------------------------------------------ the layer ---------------------------------
def test_causal_layer_vs_oracle(P):
    """PyramidAdaptiveBlockSparseAttnTrain: estimate -> mask -> similarity cap -> legacy causal attention.  The mask is
    rebuilt by the oracle from the device's estimate (bit exact), the output is compared with the oracle's legacy
    forward on that mask (north-star bar: max-abs <= 2e-2, cosine >= 0.999)."""
    from psa_b200.causal import AttentionConfig, PyramidAdaptiveBlockSparseAttnTrain, x_block_imp_estimate
    H, L, D = 2, 1100, 128
    q, k, v = C.qkv(640, 1, H, L, D, torch.bfloat16)
    cfg = AttentionConfig(text_length=200, xattn_chunk_size=1024)
    mod = PyramidAdaptiveBlockSparseAttnTrain(cfg, layer_idx=3, log_dir="unused")
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = mod(qd, kd, vd).float().cpu()
    est = x_block_imp_estimate(qd, kd, block_size=128, stride=16, chunk_size=1024, causal=True).cpu()
    mask = O.causal_level_mask(est, cfg.mask_ratios, 200, "topk", 128, True)
    sim = O.k_similarity(k, 128, 0.75, 0.7, 0.7)
    mask = torch.min(sim.unsqueeze(-2).to(mask.dtype), mask)
    ref = O.legacy_forward(q, k, v, mask, causal=True)[0].float()
    a, b = out.double().flatten(), ref.double().flatten()
    assert float((a @ b) / (a.norm() * b.norm())) >= 0.999 and float((out - ref).abs().max()) <= 2e-2
    rec = mod.records[0]
    assert rec["layer_idx"] == 3 and rec["per_head_density"].shape == (H,)
    assert 0.0 < float(rec["sparsity"]) < 1.0
