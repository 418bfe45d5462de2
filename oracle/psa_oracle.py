"""CPU restatement of the Pyramid-Sparse-Attention hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker used by the test-suite, by the smoke run and by the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark.  It is never
imported by the product package: the shipped path is CUDA-only.

Every function restates, in plain PyTorch-CPU / numpy, what one stage of the
reference (ziplab/Pyramid-Sparse-Attention) computes, including its rounding
points and its two known quirks.  Citations are ``file:line`` inside the
reference project.

Parity pin: the reference ships no golden vectors or tests.  The restatement is
pinned instead against outputs of the reference's own code executed on CPU
(Triton interpreter, fp32/fp16) by ``tests/golden/make_golden.py``; the
resulting fixtures live in ``tests/golden/*.npz`` and are re-checked by
``tests/test_oracle_golden.py``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

LEVELS = (1, 2, 4, 8)


# --------------------------------------------------------------------------------------
# a1  pyramid K/V builder            src/psa_triton/kernels/psa_kernel.py:318-349, 381-388
# --------------------------------------------------------------------------------------
def pad_replicate(x: torch.Tensor, multiple: int) -> torch.Tensor:
    """Replicate-pad dim 2 of [B,H,L,D] to a multiple (psa_kernel.py:318-329)."""
    L = x.size(2)
    rem = L % multiple
    if rem:
        x = torch.cat([x, x[:, :, -1:, :].expand(-1, -1, multiple - rem, -1)], dim=2)
    return x


def _mean_pairs(x: torch.Tensor) -> torch.Tensor:
    """mean over adjacent token pairs, fp32 add, one rounding into x.dtype
    (what torch.mean over a size-2 dim does; psa_kernel.py:348)."""
    B, H, L, D = x.shape
    xf = x.float().view(B, H, L // 2, 2, D)
    return ((xf[:, :, :, 0] + xf[:, :, :, 1]) * 0.5).to(x.dtype)


def pyramid_kv(x: torch.Tensor, block_n: int) -> Dict[int, torch.Tensor]:
    """Levels 2/4/8 of the mean-pooled pyramid of K or V (psa_kernel.py:381-388).

    The chain is hierarchical: level 4 pools the *rounded* level 2, level 8 the
    rounded level 4.  Level 16 is built by the reference but never read
    (psa_kernel.py:211 stops at 8) and is not restated.
    """
    xp = pad_replicate(x, block_n)
    x2 = _mean_pairs(xp)
    x4 = _mean_pairs(x2)
    x8 = _mean_pairs(x4)
    return {2: x2, 4: x4, 8: x8}


# --------------------------------------------------------------------------------------
# a2  token sampling                               src/psa_triton/attention.py:116-137
# --------------------------------------------------------------------------------------
def draw_sample_indices(B: int, H: int, block: int, keep: int, device="cpu") -> torch.Tensor:
    """idx[b,h,:] = topk(rand(B,H,1,block), keep).indices (attention.py:132-133).
    Consumes the global torch RNG exactly like the reference does."""
    rand_vals = torch.rand(B, H, 1, block, device=device)
    _, idx = torch.topk(rand_vals, keep, dim=3)
    return idx.view(B, H, keep)


def gather_samples(x: torch.Tensor, block: int, idx: torch.Tensor) -> torch.Tensor:
    """Rows idx of every block of the replicate-padded tensor (attention.py:128-137),
    then replicate-padded to a multiple of 64 rows (attention.py:214-215)."""
    xp = pad_replicate(x, block)
    B, H, L, D = xp.shape
    nb = L // block
    keep = idx.shape[-1]
    xb = xp.view(B, H, nb, block, D)
    gi = idx.view(B, H, 1, keep, 1).expand(-1, -1, nb, -1, D)
    s = torch.gather(xb, 3, gi).reshape(B, H, nb * keep, D)
    return pad_replicate(s, 64)


# --------------------------------------------------------------------------------------
# a3  block scores                 src/psa_triton/kernels/attn_pooling_kernel.py:12-116,341-431
# --------------------------------------------------------------------------------------
def block_scores(q, k, idx_q, idx_k, block_m: int, block_n: int) -> torch.Tensor:
    """Po[b,h,r,c]: row-normalised max-pooled softmax numerator on sampled tokens.

    R[i,c]  = max_{j in cell c}(q_i.k_j) * (D^-0.5 * 1.44269504)   -> stored in q.dtype
    m_i     = max_c R[i,c]  (fp32, before the rounding)            (kernel :63-72)
    Po[r,c] = max_{i in group r} exp2(float(R[i,c]) - m_i)         -> q.dtype (:96-112)
    Po     /= sum_c Po  over ALL n_d columns, padded cells included (:428-429)
    and the result is sliced to [:Mq, :Nk] (attention.py:223).
    """
    B, H, S, D = q.shape
    kq, kk = block_m // 4, block_n // 4
    sq = gather_samples(q, block_m, idx_q)
    sk = gather_samples(k, block_n, idx_k)
    Mq = -(-S // block_m)
    Nk = -(-k.shape[2] // block_n)
    n_d = -(-sk.shape[2] // kk)
    m_d = -(-sq.shape[2] // kq)
    sm_scale = np.float32(1.0 / (D ** 0.5))
    qk_scale = float(np.float32(sm_scale * np.float32(1.44269504)))
    s = torch.matmul(sq.float(), sk.float().transpose(-1, -2))          # fp32 accumulate
    Rf = s.view(B, H, sq.shape[2], n_d, kk).amax(dim=-1) * qk_scale      # fp32
    m = Rf.amax(dim=-1, keepdim=True)
    R = Rf.to(q.dtype).float()
    e = torch.exp2(R - m)
    Po = e.view(B, H, m_d, kq, n_d).amax(dim=3).to(q.dtype)
    Sum = torch.sum(Po, dim=-1, keepdim=True)
    Po = Po / Sum
    return Po[:, :, :Mq, :Nk]


# --------------------------------------------------------------------------------------
# a4/a5  level assignment        src/psa_triton/utils/transfer_attn_to_mask.py:6-507
# --------------------------------------------------------------------------------------
def align_multiple(level: int, block_n: int, tile_n: int, topk: bool) -> int:
    """transfer_attn_to_mask.py:65-68 (topk: level 0 -> 1) and :152,382 (threshold: ceil(0/..)=0)."""
    if level == 0 and topk:
        return 1
    return math.ceil(level / (block_n // tile_n))


def topk_intervals(Nk: int, ratios: Dict[int, Tuple[float, float]], block_n: int, tile_n: int,
                   newtype: bool) -> List[Tuple[int, int, int]]:
    """Rank intervals [start,end) per level, identical for every row
    (transfer_attn_to_mask.py:63-120 old format, :282-351 new format)."""
    out = []
    last_end = 0
    for level, (_, end_ratio) in ratios.items():
        a = align_multiple(level, block_n, tile_n, topk=True)
        start = last_end
        init_end = min(Nk, int(Nk * end_ratio))
        length = init_end - start
        if a > 1 and length > 0:
            rem = length % a
            aligned = length + (a - rem) if rem else length
            end = min(start + aligned, Nk)
            if end == Nk:
                end = start + ((end - start) // a) * a
        else:
            end = init_end
        if start < end:
            out.append((level, start, end))
            last_end = end
        else:
            if newtype:
                out.append((level, start, start))     # empty segment, separator still emitted
                last_end = start
            # old format: nothing written, last_end unchanged
    return out


def _cmp_scalar(value: float, dtype: torch.dtype) -> float:
    """`tensor <= python_float` compares in the tensor's dtype: the scalar is rounded
    to that dtype first (observed with torch 2.11 on CPU for bf16/fp16/fp32)."""
    return float(torch.tensor(value, dtype=torch.float64).to(dtype).double())


def threshold_intervals_row(ratio_row: torch.Tensor, levels_sorted, Nk: int, block_n: int, tile_n: int,
                            min_full: float) -> List[Tuple[int, int, int]]:
    """Per-row intervals for the cumulative-energy mode
    (transfer_attn_to_mask.py:150-265 old format, :380-500 new format)."""
    out = []
    last = 0
    for level, (_, end_ratio) in levels_sorted:
        a = align_multiple(level, block_n, tile_n, topk=False)
        thr = _cmp_scalar(end_ratio + 1e-6, ratio_row.dtype)
        cnt = int((ratio_row.double() <= thr).sum())
        init_end = cnt + 1 if cnt > 0 else last
        start = last
        if a > 1:
            length = max(init_end - start, 0)
            rem = length % a
            aligned = length + (a - rem) if rem else length
            end = min(start + aligned, Nk)
            if end == Nk:
                end = start + ((end - start) // a) * a
        else:
            end = max(min(max(init_end, 0), Nk), start)
            if level == 1:
                end = max(end, min(Nk, int(Nk * min_full) + 1))
        out.append((level, start, end))
        last = end
    return out


def assign_levels(Po: torch.Tensor, ratios: Dict[int, Tuple[float, float]], mode: str,
                  block_n: int, tile_n: int, text_length: int = 0,
                  min_full_attn_ratio: float = 0.06) -> torch.Tensor:
    """Restatement of transfer_attn_to_mask for its four modes.

    Sort is descending with ties in ascending index order (what torch.sort gives on
    CPU and what a stable radix sort gives on CUDA).  New format: int32
    [B,H,Mq,Nk+len(ratios)] = sorted indices of each level's rank interval followed
    by a -1 separator; old format: int32 [B,H,Mq,Nk] with values {0,1,2,4,8}.
    """
    B, H, Mq, Nk = Po.shape
    newtype = mode.endswith("_newtype")
    base = mode.replace("_newtype", "")
    if base not in ("topk", "thresholdbound"):
        raise ValueError(f"Unknown mode: {mode}. Must be 'topk' or 'thresholdbound'")
    sorted_w, order = torch.sort(Po, dim=-1, descending=True, stable=True)
    order = order.to(torch.int32)
    W = Nk + len(ratios)
    mask = torch.zeros((B, H, Mq, W if newtype else Nk), dtype=torch.int32)
    if base == "topk":
        iv = topk_intervals(Nk, ratios, block_n, tile_n, newtype)
        for li, (level, s, e) in enumerate(iv):
            if newtype:
                if s < e:
                    mask[..., li + s: li + e] = order[..., s:e]
                mask[..., li + e] = -1
            else:
                idx = order[..., s:e].long()
                mask.scatter_(-1, idx, torch.full_like(idx, level, dtype=torch.int32))
    else:
        cs = torch.cumsum(sorted_w, dim=-1)
        ratio = cs / cs[..., -1:]
        levels_sorted = sorted(ratios.items(), key=lambda x: x[1][1])
        for b in range(B):
            for h in range(H):
                for m in range(Mq):
                    iv = threshold_intervals_row(ratio[b, h, m], levels_sorted, Nk, block_n, tile_n,
                                                 min_full_attn_ratio)
                    row = mask[b, h, m]
                    orow = order[b, h, m]
                    for li, (level, s, e) in enumerate(iv):
                        if newtype:
                            if s < e:
                                row[li + s: li + e] = orow[s:e]
                            row[min(max(li + e, 0), W - 1)] = -1
                        elif s < e:
                            row[orow[s:e].long()] = level
    if not newtype and text_length > 0:
        tb = (text_length + block_n - 1) // block_n
        mask[..., -tb:] = 1                              # transfer_attn_to_mask.py:40-45
    return mask


def density_newtype(mask: torch.Tensor) -> Tuple[float, List[float]]:
    """calc_density_newtype (transfer_attn_to_mask.py:547-622): mean over rows of
    sum_l len_l / l / (W - 5); segments in fixed order 1,2,4,8,0."""
    B, H, Mq, W = mask.shape
    sep = (mask == -1)
    segid = sep.cumsum(-1)
    dens = torch.zeros(B, H, Mq, dtype=torch.float32)
    for si, l in enumerate([1, 2, 4, 8, 0]):
        if l == 0:
            continue
        dens += ((segid == si) & ~sep).sum(-1).float() / l
    dens = dens / (W - 5)
    return dens.mean().item(), [dens[:, h].mean().item() for h in range(H)]


def density_old(mask: torch.Tensor) -> Tuple[float, List[float]]:
    """calc_density (transfer_attn_to_mask.py:510-544)."""
    d = torch.zeros_like(mask, dtype=torch.float32)
    nz = mask > 0
    d[nz] = 1.0 / mask[nz].float()
    return d.mean().item(), [d[:, h].mean().item() for h in range(mask.shape[1])]


# --------------------------------------------------------------------------------------
# a9  K similarity cap             src/psa_triton/kernels/calc_ksim_kernel.py:6-225
# --------------------------------------------------------------------------------------
def k_similarity(k: torch.Tensor, block_n: int, t2: float, t4: float, t8: float) -> torch.Tensor:
    """Per K block: mean cosine of (k[2i],k[2i+1]), (k[4i],k[4i+3]), (k[8i],k[8i+7]);
    8 if s8>t8 else 4 if s4>t4 else 2 if s2>t2 else 1 (kernel :139-147).  Uses the Triton
    kernel's epsilons: norm = sqrt(sum x^2 + 1e-12), cos = dot / (n1*n2 + 1e-6) (:74-80).
    Input is the replicate-padded K (attention.py:196,203)."""
    kp = pad_replicate(k, block_n).float()
    B, H, L, D = kp.shape
    nb = L // block_n
    kb = kp.view(B, H, nb, block_n, D)
    norm = torch.sqrt((kb * kb).sum(-1) + 1e-12)

    def sim(stride, off):
        a, b = kb[..., 0::stride, :], kb[..., off::stride, :]
        na, nb_ = norm[..., 0::stride], norm[..., off::stride]
        cos = (a * b).sum(-1) / (na * nb_ + 1e-6)
        return cos.sum(-1) / cos.shape[-1]

    s2, s4, s8 = sim(2, 1), sim(4, 3), sim(8, 7)
    out = torch.ones(B, H, nb, dtype=torch.int32)
    out[s2 > t2] = 2
    out[s4 > t4] = 4
    out[s8 > t8] = 8
    return out


# --------------------------------------------------------------------------------------
# a6  new-mask multi-level forward          src/psa_triton/kernels/psa_kernel.py:24-316
# --------------------------------------------------------------------------------------
def parse_mask_row(row: Sequence[int]) -> Dict[int, List[int]]:
    """Split one index list at its -1 separators: 1st segment level 1, 2nd level 2, 3rd level 4,
    4th level 8; everything after the 4th separator is ignored (psa_kernel.py:207-217)."""
    out = {1: [], 2: [], 4: [], 8: []}
    level = 1
    for a in row:
        a = int(a)
        if a == -1:
            level *= 2
            if level > 8:
                break
        else:
            out[level].append(a)
    return out


def row_token_columns(segs: Dict[int, List[int]], block_n: int, tile_n: int, n_ctx: Dict[int, int],
                      quirk: bool = True) -> Dict[int, List[int]]:
    """Token positions (inside each level's pooled K/V) that one query block attends to, with
    multiplicity, following the reference's tile walk (psa_kernel.py:261-302).

    P = block_n/level.  P >= tile_n: the block's P tokens.  P < tile_n: entries are consumed in
    PAIRS and each pair's tile has tile_n columns: a0*P+c (c<P), a1*P+(c-P) (P<=c<2P) and — the
    reference's merge loop being hard-coded to 2 — pooled tokens c for 2P <= c < tile_n
    (quirk=True reproduces this).  Columns >= n_ctx[level] are masked out (:54).
    """
    cols = {}
    for level in LEVELS:
        P = block_n // level
        lst = segs[level]
        c = []
        if P >= tile_n:
            for a in lst:
                c.extend(t for t in range(a * P, (a + 1) * P) if t < n_ctx[level])
        else:
            assert len(lst) % 2 == 0, "merged levels need an even number of entries"
            for i in range(0, len(lst), 2):
                a0, a1 = lst[i], lst[i + 1]
                c.extend(t for t in range(a0 * P, (a0 + 1) * P) if t < n_ctx[level])
                c.extend(t for t in range(a1 * P, (a1 + 1) * P) if t < n_ctx[level])
                if quirk:
                    c.extend(t for t in range(2 * P, tile_n) if t < n_ctx[level])
        cols[level] = c
    return cols


def psa_forward_newmask(q, k, v, mask, block_m: int, block_n: int, tile_n: int,
                        sm_scale: float | None = None, quirk: bool = True) -> torch.Tensor:
    """Dense masked-softmax form of the multi-level forward:
    O_i = sum_t softmax_t(q_i.k~_t * scale + ln(level_t)) v~_t over the multiset of
    pooled tokens selected for the row's query block (psa_kernel.py:47-77, 304-316).
    fp64 math; the result is rounded to q.dtype."""
    B, H, S, D = q.shape
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    kp = {1: k, **pyramid_kv(k, block_n)}
    vp = {1: v, **pyramid_kv(v, block_n)}
    n_ctx = {l: kp[l].shape[2] for l in LEVELS}
    out = torch.empty_like(q)
    Mq = -(-S // block_m)
    for b in range(B):
        for h in range(H):
            for m in range(Mq):
                segs = parse_mask_row(mask[b, h, m].tolist())
                cols = row_token_columns(segs, block_n, tile_n, n_ctx, quirk)
                ks, vs, bias = [], [], []
                for l in LEVELS:
                    if cols[l]:
                        ci = torch.tensor(cols[l], dtype=torch.long)
                        ks.append(kp[l][b, h].double()[ci])
                        vs.append(vp[l][b, h].double()[ci])
                        bias.append(torch.full((len(ci),), math.log(l), dtype=torch.float64))
                r0, r1 = m * block_m, min((m + 1) * block_m, S)
                if not ks:
                    out[b, h, r0:r1] = float("nan")      # l_i = 0 -> 0/0 (psa_kernel.py:305)
                    continue
                Kc, Vc, bc = torch.cat(ks), torch.cat(vs), torch.cat(bias)
                logits = q[b, h, r0:r1].double() @ Kc.T * scale + bc
                p = torch.softmax(logits, dim=-1)
                out[b, h, r0:r1] = (p @ Vc).to(q.dtype)
    return out


# --------------------------------------------------------------------------------------
# a7/a8  legacy forward + backward    src/psa_triton/kernels/psa_kernel_legacy.py
# --------------------------------------------------------------------------------------
def legacy_forward(q, k, v, mask, causal: bool = False, sm_scale: float | None = None):
    """Old-format mask forward (psa_kernel_legacy.py:34-101, 580-799), block 128.

    mask[b,h,m,pb] = l > 0: query block m attends pooled tokens [pb*128/l, (pb+1)*128/l) of level l
    with logit + ln(l).  Token j of level l is visible iff j < N_l and, when causal,
    (j+1)*l - 1 <= query position (:78-81).  Causal rows only walk pb < min(cdiv(S,128), m+1)
    (:584-586).  Returns (O in q.dtype, lse fp32 = M + ln(max(L,1e-8)) (:931))."""
    B, H, S, D = q.shape
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    kp = {1: k, **pyramid_kv(k, 128)}
    vp = {1: v, **pyramid_kv(v, 128)}
    out = torch.empty_like(q)
    lse = torch.empty(B, H, S, dtype=torch.float32)
    Mq = -(-S // 128)
    nblk = -(-S // 128)
    for b in range(B):
        for h in range(H):
            for m in range(Mq):
                r0, r1 = m * 128, min((m + 1) * 128, S)
                end = min(nblk, m + 1) if causal else nblk
                qpos = torch.arange(r0, r1)
                logits, vals = [], []
                for pb in range(end):
                    l = int(mask[b, h, m, pb])
                    if l <= 0:
                        continue
                    P = 128 // l
                    n_l = kp[l].shape[2]
                    j = torch.arange(pb * P, (pb + 1) * P)
                    j = j[j < n_l]
                    if len(j) == 0:
                        continue
                    s = q[b, h, r0:r1].double() @ kp[l][b, h].double()[j].T * scale + math.log(l)
                    if causal:
                        vis = ((j + 1) * l - 1)[None, :] <= qpos[:, None]
                        s = s.masked_fill(~vis, float("-inf"))
                    logits.append(s)
                    vals.append(vp[l][b, h].double()[j])
                if not logits:
                    out[b, h, r0:r1] = 0
                    lse[b, h, r0:r1] = float("-inf")
                    continue
                Lg, Vc = torch.cat(logits, dim=1), torch.cat(vals)
                mx = Lg.amax(dim=1, keepdim=True)
                mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
                e = torch.exp(Lg - mx)
                den = e.sum(1, keepdim=True)
                out[b, h, r0:r1] = (e @ Vc / den.clamp_min(1e-8)).to(q.dtype)
                lse[b, h, r0:r1] = (mx + torch.log(den.clamp_min(1e-8))).squeeze(1).float()
    return out, lse


def legacy_backward(q, k, v, mask, o, lse, do, causal: bool = False, sm_scale: float | None = None):
    """Legacy backward (psa_kernel_legacy.py:947-1069, kernels :1072-1234, helpers :1237-1320).

    Per level l present in the mask: K^l = repeat_l(avgpool_l(pad128(K))) at ORIGINAL positions,
    p_ij = exp(q_i.K^l_j*scale - lse_i) (no +ln l: the l repeats supply it), causal uses
    i >= j on original positions (this differs from the forward's rule on diagonal blocks with
    l > 1; reproduced as is).  dV^l = p^T dO, dS = p*(dO V^l^T - delta), dQ += dS K^l scale,
    dK^l = dS^T Q scale; pooled grads are averaged back over the l constituents and the
    replicate-pad tail is folded into token S-1.  fp64 math, cast to input dtypes at the end."""
    B, H, S, D = q.shape
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    S_pad = -(-S // 128) * 128
    qd, dod = q.double(), do.double()
    delta = (o.double() * dod).sum(-1)                                  # [B,H,S]
    dq = torch.zeros(B, H, S, D, dtype=torch.float64)
    dk = torch.zeros(B, H, S, D, dtype=torch.float64)
    dv = torch.zeros(B, H, S, D, dtype=torch.float64)
    pos_q = torch.arange(S)
    for l in LEVELS:
        sel = (mask == l)
        if not bool(sel.any()):
            continue
        if l == 1:
            kl, vl, Lk = k.double(), v.double(), S
        else:
            kl = pyramid_kv(k, 128)[l].double().repeat_interleave(l, dim=2)
            vl = pyramid_kv(v, 128)[l].double().repeat_interleave(l, dim=2)
            Lk = S_pad
        pos_k = torch.arange(Lk)
        # token-level 0/1 visibility from the 128-granular mask
        tok = sel.repeat_interleave(128, dim=2)[:, :, :S].repeat_interleave(128, dim=3)[:, :, :, :Lk]
        if causal:
            tok = tok & (pos_q[:, None] >= pos_k[None, :])
        s = qd @ kl.transpose(-1, -2) * scale
        # pairs outside the mask are never visited by the kernels (a query block that selected nothing has lse = -inf
        # and contributes nothing): exclude them before the exponential instead of multiplying by 0 afterwards
        p = torch.exp((s - lse.double().unsqueeze(-1)).masked_fill(~tok, float("-inf")))
        dvl = p.transpose(-1, -2) @ dod
        dp = dod @ vl.transpose(-1, -2)
        ds = p * (dp - delta.unsqueeze(-1))
        dq += ds @ kl * scale
        dkl = ds.transpose(-1, -2) @ qd * scale
        if l == 1:
            dk += dkl[:, :, :S]
            dv += dvl[:, :, :S]
        else:
            for g, acc in ((dkl, dk), (dvl, dv)):
                gp = g.view(B, H, Lk // l, l, D).sum(3) / l
                gpad = gp.repeat_interleave(l, dim=2)
                acc += gpad[:, :, :S]
                if Lk > S:
                    acc[:, :, S - 1] += gpad[:, :, S:].sum(2)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


# --------------------------------------------------------------------------------------
# whole plug-and-play call                      src/psa_triton/attention.py:261-310
# --------------------------------------------------------------------------------------
def psa_attention(q, k, v, *, block_m=128, block_n=64, tile_n=32, mask_ratios=None, mask_mode="topk",
                  attn_impl="new_mask_type", idx_q=None, idx_k=None, quirk=True):
    """PSAAttention.forward restated end to end.  Draws the sample indices from the global torch
    RNG (Q first, then K) unless they are supplied.  Returns (out, mask, Po)."""
    if mask_ratios is None:
        mask_ratios = {1: (0.0, 0.1), 2: (0.1, 0.15), 4: (0.15, 0.15), 8: (0.15, 0.35), 0: (0.35, 1.0)}
    B, H, S, D = q.shape
    if idx_q is None:
        idx_q = draw_sample_indices(B, H, block_m, block_m // 4)
    if idx_k is None:
        idx_k = draw_sample_indices(B, H, block_n, block_n // 4)
    Po = block_scores(q, k, idx_q, idx_k, block_m, block_n)
    if attn_impl == "new_mask_type":
        mask = assign_levels(Po, mask_ratios, mask_mode + "_newtype", block_n, tile_n)
        out = psa_forward_newmask(q, k, v, mask, block_m, block_n, tile_n, quirk=quirk)
    else:
        mask = assign_levels(Po, mask_ratios, mask_mode, block_n, tile_n, text_length=0)
        out, _ = legacy_forward(q, k, v, mask, causal=False)
    return out, mask, Po


# =====================================================================================================
# Causal (vision-language) call site: antidiagonal block-importance estimate and its level mask.
# =====================================================================================================
def antidiag_block_scores(q: torch.Tensor, k: torch.Tensor, block_size: int, stride: int, causal: bool = True,
                          chunk_size: int = 4096, norm: float = 1.0) -> torch.Tensor:
    """estimate_block_importance with select_mode='inverse', softmax=True, kdb=1
    (qwen2.5-vl-example/src/attention/PSA_casual/utils/block_importance.py:282-562) as exact maths in fp64.

    q, k: [B, H, L, D] with equal lengths.  Tokens are zero-padded to a multiple of chunk_size and grouped by `stride`:
    logit[i, j] = sum_s q[i*stride + stride-1-s] . k[j*stride + s] / sqrt(D) / stride / norm.  Causal: group i sees groups
    j <= i; otherwise every group of the padded length (zero keys included, logit 0), as both of the reference's code
    paths do.  Groups without a valid query token give zero rows.  Result [B, H, ceil(L/block), ceil(L/block)] (fp64) =
    the softmax mass per (query block, key block).  The reference's PyTorch fallback additionally hides all earlier
    chunks when L is a multiple of chunk_size (its '[-0:]' slice); its Triton path, which is what runs on a GPU, does
    not, and neither does this function."""
    B, H, L, D = q.shape
    assert k.shape == q.shape and block_size % stride == 0 and chunk_size % block_size == 0
    Lp = -(-L // chunk_size) * chunk_size
    n = Lp // stride
    qp = F.pad(q.double(), (0, 0, 0, Lp - L)).view(B, H, n, stride, D)
    kp = F.pad(k.double(), (0, 0, 0, Lp - L)).view(B, H, n, stride, D)
    logits = torch.einsum("bhisd,bhjsd->bhij", qp.flip(3), kp) / math.sqrt(D) / stride / norm
    if causal:
        hide = torch.triu(torch.ones(n, n, dtype=torch.bool), diagonal=1)
        logits = logits.masked_fill(hide, float("-inf"))
    p = torch.softmax(logits, dim=-1)
    n_valid = -(-L // stride)
    p[:, :, n_valid:, :] = 0
    rb = block_size // stride
    sums = p.view(B, H, n // rb, rb, n // rb, rb).sum(dim=(3, 5))
    nb = -(-L // block_size)
    return sums[:, :, :nb, :nb]


def causal_level_mask(attn: torch.Tensor, mask_ratios: Dict[int, Tuple[float, float]], text_length: int, mode: str,
                      block_size: int, causal: bool) -> torch.Tensor:
    """transfer_attn_to_mask of the causal call site
    (qwen2.5-vl-example/src/attention/PSA_casual/PyramidAdaptiveBlockSparseAttn.py:85-168), row by row.
    attn [B, H, n, n] -> int32 [B, H, n, n] in {0, 1, 2, 4, 8}.  Equal scores rank in ascending column order.
    'energybound' arithmetic: row sum and running sum are taken sequentially in fp32 (fp64 for fp32 scores) and rounded to
    the score type (the running sum at every element), the ratio is rounded to the score type and compared with the
    bounds rounded to the score type."""
    if not mask_ratios:
        raise ValueError("mask_ratios must not be empty")
    if mode not in {"topk", "energybound"}:
        raise ValueError("mode must be 'topk' or 'energybound'")
    B, H, n, _ = attn.shape
    dt = attn.dtype
    out = torch.zeros((B, H, n, n), dtype=torch.int32)
    f32 = np.float32
    nsb = min(math.ceil(text_length / block_size) if text_length > 0 else 0, n)
    acc_t = np.float64 if dt == torch.float32 else np.float32

    def rnd(x):
        return float(torch.tensor(float(x), dtype=torch.float64).to(dt).double())

    for b in range(B):
        for h in range(H):
            for i in range(n):
                row = attn[b, h, i].double().numpy()
                order = np.lexsort((np.arange(n), -row))          # descending score, ascending column
                m = np.zeros(n, dtype=np.int32)
                if mode == "topk":
                    valid = f32(i + 1) if causal else f32(n)
                    for value, (s_ratio, e_ratio) in mask_ratios.items():
                        s = min(int(f32(valid * f32(s_ratio))), n)
                        e = min(int(f32(valid * f32(e_ratio))), n)
                        if e > s:
                            m[order[s:e]] = value
                else:
                    total = acc_t(0)
                    for x in row:
                        total = acc_t(total + acc_t(x))
                    total = max(rnd(total), rnd(1e-10))
                    run = acc_t(0)
                    prev_upper = 0.0
                    ratio = np.empty(n)
                    for r, c in enumerate(order):
                        run = acc_t(run + acc_t(row[c]))
                        ratio[r] = rnd(rnd(run) / total)
                    for value, (s_ratio, e_ratio) in mask_ratios.items():
                        lower = max(s_ratio, prev_upper)
                        prev_upper = e_ratio
                        sel = (ratio > rnd(lower)) & (ratio <= rnd(e_ratio))
                        m[order[sel]] = value
                out[b, h, i] = torch.from_numpy(m)
    if nsb:
        out[:, :, :, -nsb:] = 1
        out[:, :, -nsb:, :] = 1
    if causal:
        out[:, :, torch.triu(torch.ones(n, n, dtype=torch.bool), diagonal=1)] = 0
    d = torch.arange(n)
    out[:, :, d, d] = 1
    out[:, :, :, 0] = 1
    return out
