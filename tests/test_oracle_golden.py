"""CPU: the oracle (oracle/psa_oracle.py) against the fixtures produced by the reference itself."""
import numpy as np
import pytest
import torch

import cases as C
from oracle import psa_oracle as O


def t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("dt", ["fp32", "bf16", "fp16"])
def test_pyramid_bit_exact(golden, dt):
    x = C.randn(11, (1, 2, 333, 64), C.DT[dt])
    mine = O.pyramid_kv(x, 64)
    for l in (2, 4, 8):
        assert torch.equal(mine[l].float(), t(golden[f"pyramid_{dt}_l{l}"]))


@pytest.mark.parametrize("case", C.SCORE_CASES, ids=lambda c: c[0])
def test_block_scores(golden, case):
    name, S, D, H, bm, bn, dt = case
    q, k, _ = C.qkv(100, 1, H, S, D, C.DT[dt])
    iq, ik = C.sample_idx(7, 1, H, bm, bm // 4), C.sample_idx(8, 1, H, bn, bn // 4)
    mine = O.block_scores(q, k, iq, ik, bm, bn).float()
    ref = t(golden[f"scores_{name}"])
    assert mine.shape == ref.shape
    # fp32 accumulation order of the dot products is the only freedom
    assert float((mine - ref).abs().max()) <= 2e-7 * max(1.0, float(ref.max()) / 1e-2)


@pytest.mark.parametrize("case", C.ASSIGN_CASES, ids=lambda c: c[0])
def test_assign_levels_bit_exact(golden, case):
    name, Mq, Nk, bn, tn, mode, rn, dt, text, ties = case
    po = C.scores_like(sum(map(ord, name)), 1, 2, Mq, Nk, C.DT[dt], ties=ties)
    mine = O.assign_levels(po, getattr(C, rn), mode, bn, tn, text_length=text)
    ref = t(golden[f"assign_{name}"])
    assert torch.equal(mine, ref)
    key = f"density_{name}"
    if key in golden.files:
        d = O.density_newtype(ref) if mode.endswith("newtype") else O.density_old(ref)
        assert abs(d[0] - golden[key][0]) < 1e-6
        assert np.allclose(d[1], golden[key][1:], atol=1e-6)


@pytest.mark.parametrize("case", C.FWD_CASES, ids=lambda c: c[0])
def test_forward_newmask(golden, case):
    name, S, D, H, bm, bn, tn, mode, rn = case
    q, k, v = C.qkv(200, 1, H, S, D)
    mask = t(golden[f"{name}_mask"])
    mine = O.psa_forward_newmask(q, k, v, mask, bm, bn, tn, quirk=True)
    assert float((C.sub(mine) - t(golden[f"{name}_out"])).abs().max()) < 5e-6


@pytest.mark.parametrize("case", C.LEGACY_CASES, ids=lambda c: c[0])
def test_legacy_fwd_bwd(golden, case):
    name, S, D, H, B, causal, diag1 = case
    q, k, v = C.qkv(400, B, H, S, D)
    do = C.randn(404, (B, H, S, D))
    mask = C.legacy_mask(405, B, H, S, causal, diag1)
    o, lse = O.legacy_forward(q, k, v, mask, causal)
    assert float((C.sub(o) - t(golden[f"{name}_out"])).abs().max()) < 5e-6
    dq, dk, dv = O.legacy_backward(q, k, v, mask, o, lse, do, causal)
    for g, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert float((C.sub(g) - t(golden[f"{name}_{n}"])).abs().max()) < 1e-5


@pytest.mark.parametrize("case", C.KSIM_CASES, ids=lambda c: c[0])
def test_ksim(golden, case):
    name, S, D, H, bn = case
    k = ksim_input(S, D, H)
    assert torch.equal(O.k_similarity(k, bn, 0.7, 0.65, 0.6), t(golden[name]))


def ksim_input(S, D, H):
    k = C.randn(500, (1, H, S, D), smooth=12)
    return k * torch.linspace(0.05, 3.0, S).view(1, 1, S, 1) ** 2 + C.randn(501, (1, H, 1, D)) * torch.linspace(
        2.0, 0.0, S).view(1, 1, S, 1)


@pytest.mark.parametrize("case", C.E2E_CASES, ids=lambda c: c[0])
def test_end_to_end(golden, case):
    name, S, D, H, kw, seed = case
    kw = dict(kw)
    if "mask_ratios" in kw:
        kw["mask_ratios"] = getattr(C, kw["mask_ratios"])
    q, k, v = C.qkv(600, 1, H, S, D)
    torch.manual_seed(seed)
    out, mask, _ = O.psa_attention(q, k, v, **kw)
    assert torch.equal(mask, t(golden[f"{name}_mask"]))
    assert float((C.sub(out) - t(golden[f"{name}_out"])).abs().max()) < 5e-6


def test_parse_and_columns_quirk():
    row = [3, 1, -1, -1, -1, 4, 6, 10, 12, -1, 0, 0]
    segs = O.parse_mask_row(row)
    assert segs == {1: [3, 1], 2: [], 4: [], 8: [4, 6, 10, 12]}
    n_ctx = {1: 1024, 2: 512, 4: 256, 8: 128}
    cols = O.row_token_columns(segs, 64, 32, n_ctx, quirk=True)
    assert cols[8] == list(range(32, 40)) + list(range(48, 56)) + list(range(16, 32)) + \
        list(range(80, 88)) + list(range(96, 104)) + list(range(16, 32))
    assert O.row_token_columns(segs, 64, 32, n_ctx, quirk=False)[8] == \
        list(range(32, 40)) + list(range(48, 56)) + list(range(80, 88)) + list(range(96, 104))
