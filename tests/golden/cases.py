"""Case definitions shared by the fixture generator (make_golden.py) and the tests.

Inputs are regenerated from numpy's PCG64 generator (bit-stable across machines and library
versions), so the committed fixtures only hold the reference's OUTPUTS.
"""
from __future__ import annotations

import numpy as np
import torch

DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}

DEFAULT_RATIOS = {1: (0.0, 0.1), 2: (0.1, 0.15), 4: (0.15, 0.15), 8: (0.15, 0.35), 0: (0.35, 1.0)}
RATIOS_90 = {1: (0.0, 0.05), 2: (0.05, 0.1), 4: (0.1, 0.15), 8: (0.15, 0.25), 0: (0.25, 1.0)}
RATIOS_THR = {1: (0.0, 0.5), 2: (0.5, 0.6), 4: (0.6, 0.7), 8: (0.7, 0.8), 0: (0.8, 1.0)}
RATIOS_THR2 = {1: (0.0, 0.4), 2: (0.4, 0.5), 4: (0.5, 0.6), 8: (0.6, 0.8), 0: (0.8, 1.0)}
RATIOS_DENSE = {1: (0.0, 0.3), 2: (0.3, 0.5), 4: (0.5, 0.7), 8: (0.7, 1.0), 0: (1.0, 1.0)}


def sub(x):
    """Row subsample kept in the fixtures for [B,H,S,D] float outputs (every 4th token row)."""
    return x[..., ::4, :]


def randn(seed: int, shape, dtype=torch.float32, smooth: int = 0) -> torch.Tensor:
    """Seeded N(0,1) tensor; smooth>0 adds a moving average along dim -2 so that neighbouring
    tokens correlate (gives non-trivial block scores / similarities)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape).astype(np.float32)
    if smooth:
        c = np.cumsum(x, axis=-2)
        c[..., smooth:, :] = c[..., smooth:, :] - c[..., :-smooth, :]
        x = 0.6 * x + c / np.sqrt(smooth)
    return torch.from_numpy(x).to(dtype)


def qkv(seed: int, B, H, S, D, dtype=torch.float32, smooth: int = 8):
    return (randn(seed, (B, H, S, D), dtype, smooth), randn(seed + 1, (B, H, S, D), dtype, smooth),
            randn(seed + 2, (B, H, S, D), dtype))


def sample_idx(seed: int, B, H, block, keep) -> torch.Tensor:
    """Deterministic stand-in for topk(rand) used where the test supplies the indices."""
    rng = np.random.default_rng(seed)
    out = np.stack([rng.permutation(block)[:keep] for _ in range(B * H)]).reshape(B, H, keep)
    return torch.from_numpy(out.astype(np.int64))


def scores_like(seed: int, B, H, Mq, Nk, dtype, ties: bool = True) -> torch.Tensor:
    """A positive score tensor shaped like the block-score output.  ties=True: row-normalised, with a
    few exact ties per row (several cells at the row maximum is the normal case for the estimator; in
    bf16 ties are everywhere).  ties=False: every row holds Nk DISTINCT values of the dtype (random
    distinct bit patterns in [2^-12, 1)), not normalised - the sort order is then unambiguous."""
    rng = np.random.default_rng(seed)
    if not ties:
        mant_bits = {torch.float32: 23, torch.float16: 10, torch.bfloat16: 7}[dtype]
        span = 12 << mant_bits                        # 12 binades worth of consecutive bit patterns
        rows = [rng.choice(span, size=Nk, replace=False) for _ in range(B * H * Mq)]
        steps = np.stack(rows).reshape(B, H, Mq, Nk).astype(np.int64)
        mant = (steps & ((1 << mant_bits) - 1)).astype(np.float64) / (1 << mant_bits)
        val = (1.0 + mant) * np.exp2((steps >> mant_bits).astype(np.float64) - 12.0)
        return torch.from_numpy(val).to(dtype)
    x = np.exp2(-np.abs(rng.standard_normal((B, H, Mq, Nk))) * 6).astype(np.float32)
    if ties:
        for _ in range(3):
            j = rng.integers(0, Nk, size=(B, H, Mq, 1))
            np.put_along_axis(x, j, 1.0, axis=-1)
    t = torch.from_numpy(x).to(dtype)
    s = torch.sum(t, dim=-1, keepdim=True)
    return t / s


# (name, S, D, H, bm, bn, dtype)
SCORE_CASES = [
    ("s512_d64_bn64_fp32", 512, 64, 2, 128, 64, "fp32"),
    ("s1000_d64_bn32_fp32", 1000, 64, 1, 128, 32, "fp32"),
    ("s700_d128_bn128_fp32", 700, 128, 1, 128, 128, "fp32"),
    ("s640_d64_bn64_fp16", 640, 64, 1, 128, 64, "fp16"),
]

# (name, Mq, Nk, bn, tn, mode, ratios-name, dtype, text_length, ties)
ASSIGN_CASES = []
for _dt in ("fp32", "bf16", "fp16"):
    for _mode in ("topk", "topk_newtype", "thresholdbound", "thresholdbound_newtype"):
        for (_nk, _bn, _rn) in ((64, 64, "DEFAULT_RATIOS"), (139, 32, "RATIOS_90"), (37, 128, "RATIOS_THR"),
                                (278, 64, "RATIOS_THR2"), (50, 32, "RATIOS_DENSE"), (9, 64, "DEFAULT_RATIOS")):
            for _ties in (False, True):
                ASSIGN_CASES.append((f"{_mode}_{_dt}_nk{_nk}_bn{_bn}_{_rn}_{'ties' if _ties else 'distinct'}", 3, _nk,
                                     _bn, 32, _mode, _rn, _dt,
                                     226 if (_nk == 37 and not _mode.endswith("newtype")) else 0, _ties))

# (name, S, D, H, bm, bn, tn, mode, ratios-name)
FWD_CASES = [
    ("fwd_s512_d64_bn64_topk", 512, 64, 2, 128, 64, 32, "topk", "DEFAULT_RATIOS"),
    ("fwd_s1000_d64_bn32_topk", 1000, 64, 1, 128, 32, 32, "topk", "RATIOS_90"),
    ("fwd_s700_d128_bn128_thr", 700, 128, 1, 128, 128, 32, "thresholdbound", "RATIOS_THR"),
    ("fwd_s900_d64_bn64_thr", 900, 64, 1, 128, 64, 32, "thresholdbound", "RATIOS_THR2"),
    ("fwd_s777_d64_bn32_thr", 777, 64, 1, 128, 32, 32, "thresholdbound", "RATIOS_THR"),
]

# (name, S, D, H, B, causal, diag-level-1?)
LEGACY_CASES = [
    ("legacy_s512_d64_nc", 512, 64, 2, 1, False, False),
    ("legacy_s600_d64_nc", 600, 64, 1, 1, False, False),
    ("legacy_s512_d64_causal_diag1", 512, 64, 1, 2, True, True),
    ("legacy_s640_d128_causal_mixed", 640, 128, 1, 1, True, False),
]

KSIM_CASES = [("ksim_s1024_bn128", 1024, 64, 2, 128), ("ksim_s1500_bn128", 1500, 128, 1, 128),
              ("ksim_s1024_bn32", 1024, 64, 1, 32)]

E2E_CASES = [
    # (name, S, D, H, cfg kwargs, torch seed)
    ("e2e_default_s1024", 1024, 64, 2, dict(), 2000),
    ("e2e_bn32_s900", 900, 64, 1, dict(block_n=32, mask_ratios="RATIOS_90"), 2001),
    ("e2e_thr_bn128_s768", 768, 128, 1, dict(block_n=128, mask_mode="thresholdbound", mask_ratios="RATIOS_THR2"), 2002),
    ("e2e_old_s768", 768, 64, 1, dict(block_n=128, attn_impl="old_mask_type", mask_ratios="RATIOS_THR",
                                      mask_mode="thresholdbound"), 2003),
]


def legacy_mask(seed, B, H, S, causal, diag1):
    """Random old-format mask [B,H,M128,N128] in {0,1,2,4,8}; column 0 always level 1 so that no causal
    row is empty; diag1 forces level 1 on the diagonal."""
    n = -(-S // 128)
    rng = np.random.default_rng(seed)
    m = rng.choice(np.array([0, 1, 2, 4, 8], dtype=np.int32), size=(B, H, n, n), p=[0.2, 0.3, 0.2, 0.15, 0.15])
    m[..., 0] = 1
    if diag1:
        for i in range(n):
            m[..., i, i] = 1
    if causal:
        m = m * np.tril(np.ones((n, n), dtype=np.int32))
    return torch.from_numpy(m.astype(np.int32))


GILBERT_SHAPES = [(4, 4, 4), (7, 5, 3), (1, 9, 2), (3, 17, 6), (10, 1, 1), (45, 30, 13), (52, 30, 21), (80, 45, 21)]


def order_checksum(order) -> int:
    """Position-weighted checksum of a visiting order (detects any transposition)."""
    o = np.asarray(order, dtype=np.int64)
    return int(((np.arange(o.size, dtype=np.int64) % 1000003) * (o % 999983)).sum() % (1 << 61))


# ---- causal (vision-language) call site: antidiagonal estimate and its level mask -------------------------------------
RATIOS_CAUSAL = {1: (0.0, 0.05), 2: (0.05, 0.15), 4: (0.15, 0.25), 8: (0.25, 0.5), 0: (0.5, 1.0)}
RATIOS_ENERGY = {1: (0.0, 0.6), 2: (0.6, 0.75), 4: (0.75, 0.85), 8: (0.85, 0.95), 0: (0.95, 1.0)}
# name, L, D, H, block, stride, chunk, causal
ANTIDIAG_CASES = [
    ("ad_1000_d64", 1000, 64, 2, 128, 16, 4096, True),
    ("ad_700_d128_s8", 700, 128, 2, 128, 8, 1024, True),
    ("ad_1500_two_chunks", 1500, 64, 1, 128, 16, 1024, True),
    ("ad_900_noncausal", 900, 64, 2, 128, 16, 1024, False),
    ("ad_1024_exact", 1024, 128, 1, 128, 16, 1024, True),
]
# name, n, H, dtype, mode, causal, text_length
CAUSAL_MASK_CASES = [(f"cm_{n}_{dt}_{mode}_{'c' if causal else 'n'}_{text}", n, 2, dt, mode, causal, text)
                     for n in (8, 23, 64) for dt in ("fp32", "bf16", "fp16") for mode in ("topk", "energybound")
                     for causal in (True, False) for text in (0, 300)]


def causal_scores(seed: int, H: int, n: int, dtype, causal: bool) -> torch.Tensor:
    """Block scores shaped like the estimator's output: positive rows that sum to about one block's worth of mass,
    zero above the diagonal when causal."""
    rng = np.random.default_rng(seed)
    x = rng.gamma(0.3, 1.0, size=(1, H, n, n)).astype(np.float32) + 1e-4
    if causal:
        x = np.tril(x)
    x = x / x.sum(-1, keepdims=True) * 8.0
    return torch.from_numpy(x).to(dtype)
