"""CPU: the oracle's restatement of the causal (vision-language) call site against the reference's own outputs
(tests/golden/causal_reference_outputs.npz, written by tests/golden/make_golden_causal.py from the unmodified reference)."""
import os

import numpy as np
import pytest
import torch

import cases as C
from oracle import psa_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def golden_causal():
    return np.load(os.path.join(ROOT, "tests", "golden", "causal_reference_outputs.npz"))


@pytest.mark.parametrize("case", C.ANTIDIAG_CASES, ids=lambda c: c[0])
def test_antidiagonal_estimate_matches_reference(golden_causal, case):
    name, L, D, H, block, stride, chunk, causal = case
    q, k, _ = C.qkv(500, 1, H, L, D, torch.float32)
    mine = O.antidiag_block_scores(q, k, block, stride, causal, chunk)
    ref = torch.from_numpy(golden_causal[name]).double()
    assert mine.shape == ref.shape
    assert float((mine - ref).abs().max()) <= 2e-6          # fp32 reference against fp64 restatement


@pytest.mark.parametrize("case", C.CAUSAL_MASK_CASES[::3], ids=lambda c: c[0])
def test_causal_level_mask_matches_reference(golden_causal, case):
    name, n, H, dt, mode, causal, text = case
    attn = C.causal_scores(900 + n, H, n, C.DT[dt], causal)
    ratios = C.RATIOS_CAUSAL if mode == "topk" else C.RATIOS_ENERGY
    mine = O.causal_level_mask(attn, ratios, text, mode, 128, causal)
    assert torch.equal(mine, torch.from_numpy(golden_causal[name]).to(torch.int32))


def test_causal_level_mask_errors():
    attn = C.causal_scores(1, 1, 8, torch.float32, True)
    with pytest.raises(ValueError):
        O.causal_level_mask(attn, {}, 0, "topk", 128, True)
    with pytest.raises(ValueError):
        O.causal_level_mask(attn, C.RATIOS_CAUSAL, 0, "thresholdbound", 128, True)
