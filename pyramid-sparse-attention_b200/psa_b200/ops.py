"""Tensor-level wrappers around the C-ABI kernels.  torch is used for device memory and streams only."""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import check, lib

_DT = {torch.float32: _lib.PSA_F32, torch.float16: _lib.PSA_F16, torch.bfloat16: _lib.PSA_BF16}

IMPL_AUTO, IMPL_SCALAR, IMPL_TENSOR = 0, 1, 2


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("psa_b200 kernels need CUDA tensors; there is no CPU path in this package")


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise ValueError(f"unsupported dtype {t.dtype}; use float32, float16 or bfloat16")
    return _DT[t.dtype]


def _flat_bh(x: torch.Tensor) -> torch.Tensor:
    return x if x.is_contiguous() else x.contiguous()


def _mask32(mask: torch.Tensor) -> torch.Tensor:
    """The kernels read masks as contiguous int32; the reference accepts int32 or int64 and any strides."""
    mask = mask if mask.dtype == torch.int32 else mask.to(torch.int32)
    return mask if mask.is_contiguous() else mask.contiguous()


# One status word per device, shared by every launch of the tensor-core attention kernels: a kernel whose bounded
# device-side wait expired writes PSA_ERR_TIMEOUT into it and nothing ever clears it except check_status().  Calls stay
# free of host synchronisation; a run asks once, at the end (PSAAttention.check_status, close_logger).
_STATUS: Dict[int, torch.Tensor] = {}


def status_word(device) -> torch.Tensor:
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _STATUS:
        _STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _STATUS[idx]


def check_status(device=None, reset: bool = True) -> None:
    """Raise PSAKernelError if any attention kernel launched so far on `device` (default: every device used) gave up
    on a bounded wait - its output is then incomplete.  Synchronises the device."""
    words = list(_STATUS.items()) if device is None else [(None, status_word(device))]
    for _, w in words:
        code = int(w.item())
        if code != 0:
            if reset:
                w.zero_()
            raise _lib.PSAKernelError(f"a PSA kernel on {w.device} reported status {code} (bounded device-side wait expired); "
                                      "outputs produced since the last check are incomplete")


# ------------------------------------------------------------------------------------------------
def pyramid_kv(k: torch.Tensor, v: torch.Tensor, block_n: int):
    """Levels 2/4/8 of the mean-pooled K and V ([B,H,S,D] -> [B,H,S_pad/l,D]) in one pass.
    Mirrors pad_to_multiple + pooling, src/psa_triton/kernels/psa_kernel.py:318-349,381-388."""
    _need_cuda(k, v)
    assert k.shape == v.shape and k.dtype == v.dtype
    k, v = _flat_bh(k), _flat_bh(v)
    B, H, S, D = k.shape
    s_pad = -(-S // block_n) * block_n
    with torch.cuda.device(k.device):
        outs = [torch.empty((B, H, s_pad // l, D), dtype=k.dtype, device=k.device) for l in (2, 4, 8) for _ in (0, 1)]
        k2, v2, k4, v4, k8, v8 = outs
        rc = lib.psa_pyramid_kv(_ptr(k), _ptr(v), _ptr(k2), _ptr(k4), _ptr(k8), _ptr(v2), _ptr(v4), _ptr(v8),
                                B * H, S, D, block_n, _dt(k), _stream(k))
    check(rc, "psa_pyramid_kv")
    return (k2, k4, k8), (v2, v4, v8)


class KVImages:
    """K/V of all four levels in the tile-image layout the tcgen05 forward copies from (see psa_pyramid_kv_images)."""

    def __init__(self, kimg: torch.Tensor, vimg: torch.Tensor, block_n: int):
        self.kimg, self.vimg, self.block_n = kimg, vimg, block_n


def images_supported(k: torch.Tensor, block_m: int, block_n: int, tile_n: int) -> bool:
    return (k.dtype in (torch.float16, torch.bfloat16) and block_m == 128 and tile_n == 32 and block_n in (64, 128)
            and k.shape[-1] in (64, 128))


def _perm32(perm: torch.Tensor, seq: int) -> torch.Tensor:
    if perm.device.type != "cuda" or perm.dtype != torch.int32 or perm.dim() != 1 or perm.numel() != seq:
        raise ValueError(f"perm must be a CUDA int32 tensor of {seq} row numbers")
    return perm.contiguous()


def gather_rows(x: torch.Tensor, perm: Optional[torch.Tensor], rope=None) -> torch.Tensor:
    """x[..., perm, :] for [B,H,S,D] tensors (the q copy of a reordered layer; GilbertRearranger.rearrange_single,
    src/psa_triton/utils/rearranger.py:97-115, with the text move folded into perm).  rope (RotaryTables): the rows are
    rotated on the way (16-bit tensors); perm may then be None (stored order)."""
    _need_cuda(x)
    x = _flat_bh(x)
    B, H, S, D = x.shape
    perm = None if perm is None else _perm32(perm, S)
    with torch.cuda.device(x.device):
        out = torch.empty_like(x)
        if rope is None:
            rc = lib.psa_gather_rows(_ptr(x), _ptr(perm), _ptr(out), B * H, S, D, x.element_size(), _stream(x))
        else:
            rope.check(S, D, x.device)
            rc = lib.psa_gather_rows_rope(_ptr(x), _ptr(perm), _ptr(rope.a), _ptr(rope.b), rope.first, _ptr(out), B * H, S, D,
                                          _dt(x), _stream(x))
    check(rc, "psa_gather_rows")
    return out


def pyramid_kv_images(k: torch.Tensor, v: torch.Tensor, block_n: int, perm: Optional[torch.Tensor] = None, rope=None) -> KVImages:
    """One pass over K and V -> tile images of levels 1/2/4/8 (f16/bf16, block_n 64/128).  perm: build the images of
    k[..., perm, :], v[..., perm, :] without materialising them.  rope (RotaryTables): the keys are rotated as they are
    read."""
    _need_cuda(k, v)
    assert k.shape == v.shape and k.dtype == v.dtype
    k, v = _flat_bh(k), _flat_bh(v)
    B, H, S, D = k.shape
    nbytes = lib.psa_kv_image_bytes(B * H, S, D, block_n)
    if nbytes == 0:
        raise ValueError(f"tile images need head_dim 64/128 and block_n 64/128 (got {D}, {block_n})")
    with torch.cuda.device(k.device):
        kimg = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        vimg = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        if rope is not None:
            rope.check(S, D, k.device)
            perm = None if perm is None else _perm32(perm, S)
            rc = lib.psa_pyramid_kv_images_perm_rope(_ptr(k), _ptr(v), _ptr(perm), _ptr(rope.a), _ptr(rope.b), rope.first,
                                                     _ptr(kimg), _ptr(vimg), B * H, S, D, block_n, _dt(k), _stream(k))
        elif perm is None:
            rc = lib.psa_pyramid_kv_images(_ptr(k), _ptr(v), _ptr(kimg), _ptr(vimg), B * H, S, D, block_n, _dt(k), _stream(k))
        else:
            perm = _perm32(perm, S)
            rc = lib.psa_pyramid_kv_images_perm(_ptr(k), _ptr(v), _ptr(perm), _ptr(kimg), _ptr(vimg), B * H, S, D, block_n,
                                                _dt(k), _stream(k))
    check(rc, "psa_pyramid_kv_images")
    return KVImages(kimg, vimg, block_n)


# ------------------------------------------------------------------------------------------------
# Token-major tensors ([S, H, D], one batch element): what a transformer block's projections produce and consume.
def _tm_check(*ts):
    _need_cuda(*ts)
    x = ts[0]
    for t in ts:
        if t.dim() != 3 or t.shape != x.shape or t.dtype != x.dtype or not t.is_contiguous():
            raise ValueError("token-major operands must be contiguous [S, H, D] tensors of one shape and dtype")
    return x.shape


class RotaryTables:
    """Rotary embedding applied by the kernels while they read q and k rows (token-major route).  a, b: fp32 [S - first,
    D] on the device; stored token s >= first uses row s - first, channel pair (x0, x1) becomes
    (x0*a[even] - x1*b[even], x1*a[odd] + x0*b[odd]) with every product and sum rounded separately."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor, first: int = 0):
        assert a.shape == b.shape and a.dim() == 2, "rotary tables are [tokens, head_dim]"
        self.a = a.to(torch.float32).contiguous()
        self.b = b.to(torch.float32).contiguous()
        self.first = int(first)

    def check(self, S: int, D: int, device) -> None:
        _need_cuda(self.a, self.b)
        if self.a.device != device or tuple(self.a.shape) != (S - self.first, D) or not 0 <= self.first <= S:
            raise ValueError(f"rotary tables of shape {tuple(self.a.shape)} on {self.a.device} do not fit {S} tokens "
                             f"(first rotated token {self.first}), head_dim {D} on {device}")


def rotate_rows(x: torch.Tensor, rope: RotaryTables) -> torch.Tensor:
    """What the fused loads compute, with the framework's element-wise operations: x [B, H, S, D] -> rotated copy.
    (The route for tensors the token-major kernels do not take, and the yardstick of their tests.)"""
    S, D = x.shape[2], x.shape[3]
    a, b = rope.a.to(x.device), rope.b.to(x.device)
    assert tuple(a.shape) == (S - rope.first, D)
    head, tail = x[:, :, :rope.first], x[:, :, rope.first:].float()
    x0, x1 = tail[..., 0::2], tail[..., 1::2]
    out = torch.empty_like(tail)
    out[..., 0::2] = x0 * a[:, 0::2] - x1 * b[:, 0::2]
    out[..., 1::2] = x1 * a[:, 1::2] + x0 * b[:, 1::2]
    return torch.cat([head, out.to(x.dtype)], dim=2)


def gather_heads(x: torch.Tensor, perm: Optional[torch.Tensor] = None, rope: Optional[RotaryTables] = None) -> torch.Tensor:
    """[S, H, D] -> [1, H, S, D] with out[0, h, t] = x[perm[t], h] (perm None: a plain transpose copy), rotated on the
    way if rope is given."""
    S, H, D = _tm_check(x)
    perm = None if perm is None else _perm32(perm, S)
    with torch.cuda.device(x.device):
        out = torch.empty((1, H, S, D), dtype=x.dtype, device=x.device)
        if rope is None:
            rc = lib.psa_gather_heads(_ptr(x), _ptr(perm), _ptr(out), H, S, D, x.element_size(), _stream(x))
        else:
            rope.check(S, D, x.device)
            rc = lib.psa_gather_heads_rope(_ptr(x), _ptr(perm), _ptr(rope.a), _ptr(rope.b), rope.first, _ptr(out), H, S, D,
                                           _dt(x), _stream(x))
    check(rc, "psa_gather_heads")
    return out


def pyramid_kv_images_tm(k: torch.Tensor, v: torch.Tensor, block_n: int, perm: Optional[torch.Tensor] = None,
                         rope: Optional[RotaryTables] = None) -> KVImages:
    """pyramid_kv_images of k, v given token-major ([S, H, D]), optionally read through a row table, the keys
    optionally rotated as they are read."""
    S, H, D = _tm_check(k, v)
    perm = None if perm is None else _perm32(perm, S)
    nbytes = lib.psa_kv_image_bytes(H, S, D, block_n)
    if nbytes == 0:
        raise ValueError(f"tile images need head_dim 64/128 and block_n 64/128 (got {D}, {block_n})")
    with torch.cuda.device(k.device):
        kimg = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        vimg = torch.empty(nbytes, dtype=torch.uint8, device=k.device)
        if rope is None:
            rc = lib.psa_pyramid_kv_images_tm(_ptr(k), _ptr(v), _ptr(perm), _ptr(kimg), _ptr(vimg), H, S, D, block_n, _dt(k),
                                              _stream(k))
        else:
            rope.check(S, D, k.device)
            rc = lib.psa_pyramid_kv_images_tm_rope(_ptr(k), _ptr(v), _ptr(perm), _ptr(rope.a), _ptr(rope.b), rope.first,
                                                   _ptr(kimg), _ptr(vimg), H, S, D, block_n, _dt(k), _stream(k))
    check(rc, "psa_pyramid_kv_images_tm")
    return KVImages(kimg, vimg, block_n)


def block_scores_tm(q, k, idx_q, idx_k, block_m: int, block_n: int, perm: Optional[torch.Tensor] = None,
                    rope: Optional[RotaryTables] = None) -> torch.Tensor:
    """block_scores of q, k given token-major ([S, H, D]); idx_q [H, block_m/4], idx_k [H, block_n/4].  -> [1, H, Mq, Nk].
    With rope the sampled rows of q and k are rotated as they are gathered."""
    S, H, D = _tm_check(q, k)
    _need_cuda(idx_q, idx_k)
    assert idx_q.shape == (H, block_m // 4) and idx_k.shape == (H, block_n // 4)
    perm = None if perm is None else _perm32(perm, S)
    iq = idx_q.to(torch.int32).contiguous()
    ik = idx_k.to(torch.int32).contiguous()
    Mq, Nk = -(-S // block_m), -(-S // block_n)
    with torch.cuda.device(q.device):
        po = torch.empty((1, H, Mq, Nk), dtype=q.dtype, device=q.device)
        nbytes = lib.psa_block_scores_scratch_bytes(H, S, S, block_m, block_n, _dt(q))
        if nbytes == 0:
            raise ValueError(f"psa_block_scores_tm: unsupported block sizes m={block_m} n={block_n}")
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        if rope is None:
            rc = lib.psa_block_scores_tm(_ptr(q), _ptr(k), _ptr(perm), _ptr(iq), _ptr(ik), _ptr(po), _ptr(scratch), nbytes, H,
                                         S, D, block_m, block_n, _dt(q), _stream(q))
        else:
            rope.check(S, D, q.device)
            rc = lib.psa_block_scores_tm_rope(_ptr(q), _ptr(k), _ptr(perm), _ptr(rope.a), _ptr(rope.b), rope.first, _ptr(iq),
                                              _ptr(ik), _ptr(po), _ptr(scratch), nbytes, H, S, D, block_m, block_n, _dt(q),
                                              _stream(q))
    check(rc, "psa_block_scores_tm")
    return po


def psa_forward_tm(q_heads, images: KVImages, mask, out_tm, block_m: int, block_n: int, tile_n: int,
                   sm_scale: Optional[float] = None, compat_quirk: bool = True, out_perm=None) -> torch.Tensor:
    """Tile-image forward with q head-major ([1, H, S, D], from gather_heads) whose output rows are stored token-major
    into out_tm ([S, H, D]), row t at token out_perm[t].  Returns the status word."""
    _need_cuda(q_heads, mask, out_tm)
    _, H, S, D = q_heads.shape
    assert out_tm.shape == (S, H, D) and out_tm.is_contiguous() and out_tm.dtype == q_heads.dtype
    mask = _mask32(mask)
    out_perm = None if out_perm is None else _perm32(out_perm, S)
    if sm_scale is None:
        sm_scale = D ** -0.5
    with torch.cuda.device(q_heads.device):
        status = status_word(q_heads.device)
        rc = lib.psa_fwd_images_tm(_ptr(q_heads), _ptr(images.kimg), _ptr(images.vimg), _ptr(mask), _ptr(out_tm), _ptr(out_perm),
                                   H, S, D, block_m, block_n, tile_n, mask.shape[-1], float(sm_scale), int(compat_quirk),
                                   _dt(q_heads), _ptr(status), _stream(q_heads))
    check(rc, "psa_fwd_images_tm")
    return status


def draw_sample_indices(B: int, H: int, block: int, keep: int, device) -> torch.Tensor:
    """topk(rand(B,H,1,block), keep).indices: the same two torch calls, in the same order on the same
    generator, as _random_sample_tokens (src/psa_triton/attention.py:132-133)."""
    rand_vals = torch.rand(B, H, 1, block, device=device)
    _, idx = torch.topk(rand_vals, keep, dim=3)
    return idx.view(B, H, keep)


def block_scores(q, k, idx_q, idx_k, block_m: int, block_n: int, impl: int = IMPL_AUTO, perm_q=None, perm_k=None,
                 rope=None) -> torch.Tensor:
    """Block-importance scores Po [B,H,Mq,Nk] (q.dtype).  idx_q [B,H,block_m/4], idx_k [B,H,block_n/4].
    perm_q / perm_k (both or neither): the scores of q[..., perm_q, :], k[..., perm_k, :], read in place (f16/bf16).
    rope (RotaryTables; self-attention, perm_q is perm_k or both None): the sampled rows are rotated as they are gathered."""
    _need_cuda(q, k, idx_q, idx_k)
    q, k = _flat_bh(q), _flat_bh(k)
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    assert idx_q.shape == (B, H, block_m // 4) and idx_k.shape == (B, H, block_n // 4)
    iq = idx_q.to(torch.int32).contiguous()
    ik = idx_k.to(torch.int32).contiguous()
    Mq, Nk = -(-Sq // block_m), -(-Sk // block_n)
    with torch.cuda.device(q.device):
        po = torch.empty((B, H, Mq, Nk), dtype=q.dtype, device=q.device)
        nbytes = lib.psa_block_scores_scratch_bytes(B * H, Sq, Sk, block_m, block_n, _dt(q))
        if nbytes == 0:
            raise ValueError(f"psa_block_scores: unsupported block sizes m={block_m} n={block_n}")
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        if rope is not None:
            assert Sq == Sk and perm_q is perm_k, "the rotating score kernel serves self-attention with one row table"
            rope.check(Sq, D, q.device)
            perm = None if perm_q is None else _perm32(perm_q, Sq)
            rc = lib.psa_block_scores_perm_rope(_ptr(q), _ptr(k), _ptr(perm), _ptr(rope.a), _ptr(rope.b), rope.first, _ptr(iq),
                                                _ptr(ik), _ptr(po), _ptr(scratch), nbytes, B * H, Sq, D, block_m, block_n,
                                                _dt(q), _stream(q))
        elif perm_q is None and perm_k is None:
            rc = lib.psa_block_scores(_ptr(q), _ptr(k), _ptr(iq), _ptr(ik), _ptr(po), _ptr(scratch), nbytes, B * H, Sq, Sk,
                                      D, block_m, block_n, _dt(q), impl, _stream(q))
        else:
            perm_q, perm_k = _perm32(perm_q, Sq), _perm32(perm_k, Sk)
            rc = lib.psa_block_scores_perm(_ptr(q), _ptr(k), _ptr(perm_q), _ptr(perm_k), _ptr(iq), _ptr(ik), _ptr(po),
                                           _ptr(scratch), nbytes, B * H, Sq, Sk, D, block_m, block_n, _dt(q), _stream(q))
    check(rc, "psa_block_scores")
    return po


# ------------------------------------------------------------------------------------------------
def _align_multiple(level: int, block_n: int, tile_n: int, topk: bool) -> int:
    if level == 0 and topk:
        return 1
    return math.ceil(level / (block_n // tile_n))


def topk_intervals(nk: int, ratios: Dict[int, Tuple[float, float]], block_n: int, tile_n: int, newtype: bool):
    """Rank interval of every level in dict order, with the reference's Python arithmetic
    (src/psa_triton/utils/transfer_attn_to_mask.py:63-120 old format, :282-351 new format)."""
    out = []
    last_end = 0
    for level, (_, end_ratio) in ratios.items():
        a = _align_multiple(level, block_n, tile_n, True)
        start = last_end
        init_end = min(nk, int(nk * end_ratio))
        length = init_end - start
        if a > 1 and length > 0:
            rem = length % a
            aligned = length + (a - rem) if rem else length
            end = min(start + aligned, nk)
            if end == nk:
                end = start + ((end - start) // a) * a
        else:
            end = init_end
        if start < end:
            out.append((level, start, end))
            last_end = end
        else:
            out.append((level, start, start))   # empty: new format still gets its separator
            if newtype:
                last_end = start
    return out


def _round_to_dtype(x: float, dtype: torch.dtype) -> float:
    return float(torch.tensor(x, dtype=torch.float64).to(dtype).to(torch.float64))


def assign_levels(po: torch.Tensor, mask_ratios: Dict[int, Tuple[float, float]], mode: str, block_n: int,
                  tile_n: int, text_length: int = 0, min_full_attn_ratio: float = 0.06) -> torch.Tensor:
    """Score rows -> level mask.  Same modes, argument meaning and errors as transfer_attn_to_mask
    (src/psa_triton/utils/transfer_attn_to_mask.py:6-507)."""
    if mask_ratios is None:
        raise ValueError("mask_ratios must be provided")
    if mode not in ("topk", "thresholdbound", "topk_newtype", "thresholdbound_newtype"):
        raise ValueError(f"Unknown mode: {mode}. Must be 'topk' or 'thresholdbound'")
    _need_cuda(po)
    po = _flat_bh(po)
    B, H, Mq, Nk = po.shape
    newtype = mode.endswith("_newtype")
    threshold = mode.startswith("thresholdbound")
    n = len(mask_ratios)
    if n > 8:
        raise ValueError("at most 8 levels")
    I32 = C.c_int32 * n
    F32 = C.c_float * n
    if threshold:
        items = sorted(mask_ratios.items(), key=lambda x: x[1][1])
        levels = I32(*[int(l) for l, _ in items])
        thr = F32(*[_round_to_dtype(r[1] + 1e-6, po.dtype) for _, r in items])
        aligns = I32(*[_align_multiple(int(l), block_n, tile_n, False) for l, _ in items])
        starts = ends = None
        min_index = min(Nk, int(Nk * min_full_attn_ratio) + 1)
    else:
        iv = topk_intervals(Nk, mask_ratios, block_n, tile_n, newtype)
        levels = I32(*[int(l) for l, _, _ in iv])
        starts = I32(*[s for _, s, _ in iv])
        ends = I32(*[e for _, _, e in iv])
        thr = aligns = None
        min_index = 0
    text_blocks = 0 if (newtype or text_length == 0) else (text_length + block_n - 1) // block_n
    width = Nk + n if newtype else Nk
    with torch.cuda.device(po.device):
        mask = torch.empty((B, H, Mq, width), dtype=torch.int32, device=po.device)
        rc = lib.psa_assign_levels(_ptr(po), _ptr(mask), B * H * Mq, Nk, _dt(po), int(threshold), int(newtype), n,
                                   levels, starts, ends, thr, aligns, min_index, text_blocks, _stream(po))
    check(rc, "psa_assign_levels")
    return mask


def antidiag_block_scores(q, k, block_size: int, stride: int, chunk_size: int, causal: bool = True,
                          impl: int = 0) -> torch.Tensor:
    """Antidiagonal block-importance estimate [B, H, nb, nb] (q.dtype), nb = ceil(L/block_size): estimate_block_importance
    with select_mode='inverse' (qwen2.5-vl-example/src/attention/PSA_casual/utils/block_importance.py:282-562).
    impl: 0 pick (tcgen05 GEMM when L is a multiple of stride), IMPL_TENSOR, IMPL_WARP_MMA."""
    _need_cuda(q, k)
    q, k = _flat_bh(q), _flat_bh(k)
    B, H, L, D = q.shape
    assert k.shape == q.shape and k.dtype == q.dtype
    nbytes = lib.psa_antidiag_scratch_bytes(B * H, L, D, block_size, stride, chunk_size)
    if nbytes == 0:
        raise ValueError(f"antidiagonal estimate: unsupported sizes (head_dim {D}, block {block_size}, stride {stride}, "
                         f"chunk {chunk_size})")
    nb = -(-L // block_size)
    with torch.cuda.device(q.device):
        out = torch.empty((B, H, nb, nb), dtype=q.dtype, device=q.device)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        status = status_word(q.device)
        rc = lib.psa_antidiag_scores_impl(_ptr(q), _ptr(k), _ptr(out), _ptr(scratch), nbytes, B * H, L, D, block_size, stride,
                                          chunk_size, int(causal), _dt(q), impl, _ptr(status), _stream(q))
    check(rc, "psa_antidiag_scores")
    out._psa_status = status
    return out


def assign_levels_causal(attn: torch.Tensor, mask_ratios: Dict[int, Tuple[float, float]], text_length: int, mode: str,
                         block_size: int, causal: bool) -> torch.Tensor:
    """Square score matrices -> dense level mask of the causal call site; same arguments and errors as its
    transfer_attn_to_mask (qwen2.5-vl-example/src/attention/PSA_casual/PyramidAdaptiveBlockSparseAttn.py:85-168)."""
    if not mask_ratios:
        raise ValueError("mask_ratios must not be empty")
    if mode not in {"topk", "energybound"}:
        raise ValueError("mode must be 'topk' or 'energybound'")
    _need_cuda(attn)
    attn = _flat_bh(attn)
    B, H, n, n2 = attn.shape
    assert n == n2, "the causal call site scores square block matrices"
    nl = len(mask_ratios)
    if nl > 8:
        raise ValueError("at most 8 levels")
    I32, F32 = C.c_int32 * nl, C.c_float * nl
    items = list(mask_ratios.items())              # dict order: later levels overwrite earlier ones
    levels = I32(*[int(l) for l, _ in items])
    rs = re = lo = hi = None
    if mode == "topk":
        rs = F32(*[float(r[0]) for _, r in items])
        re = F32(*[float(r[1]) for _, r in items])
    else:
        lows, prev = [], 0.0
        for _, (s_ratio, e_ratio) in items:
            lows.append(max(s_ratio, prev))
            prev = e_ratio
        lo = F32(*[_round_to_dtype(x, attn.dtype) for x in lows])
        hi = F32(*[_round_to_dtype(r[1], attn.dtype) for _, r in items])
    special = min((text_length + block_size - 1) // block_size if text_length > 0 else 0, n)
    with torch.cuda.device(attn.device):
        mask = torch.empty((B, H, n, n), dtype=torch.int32, device=attn.device)
        rc = lib.psa_assign_levels_causal(_ptr(attn), _ptr(mask), B * H, n, _dt(attn), int(mode == "energybound"), int(causal),
                                          nl, levels, rs, re, lo, hi, special, _stream(attn))
    check(rc, "psa_assign_levels_causal")
    return mask


def density(mask: torch.Tensor, newtype: bool) -> torch.Tensor:
    """Per-(batch, head) mean density [B,H] float32 on the device (no host sync).
    calc_density_newtype / calc_density, src/psa_triton/utils/transfer_attn_to_mask.py:510-622."""
    _need_cuda(mask)
    mask = _flat_bh(mask)
    B, H, Mq, W = mask.shape
    with torch.cuda.device(mask.device):
        out = torch.empty((B, H), dtype=torch.float32, device=mask.device)
        rc = lib.psa_density(_ptr(mask), _ptr(out), B * H, Mq, W, int(newtype), _stream(mask))
    check(rc, "psa_density")
    return out


def k_similarity(k: torch.Tensor, block_n: int, t2: float, t4: float, t8: float, perm: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[B,H,ceil(S/block_n)] int32 in {1,2,4,8}; calc_k_similarity_triton on the replicate-padded K
    (src/psa_triton/kernels/calc_ksim_kernel.py:160-225, src/psa_triton/attention.py:196-204).  perm: the cap of
    k[..., perm, :], read in place."""
    _need_cuda(k)
    k = _flat_bh(k)
    B, H, S, D = k.shape
    assert block_n % 8 == 0, "blocksize must be divisible by 8"
    with torch.cuda.device(k.device):
        out = torch.empty((B, H, -(-S // block_n)), dtype=torch.int32, device=k.device)
        if perm is None:
            rc = lib.psa_ksim(_ptr(k), _ptr(out), B * H, S, D, block_n, t2, t4, t8, _dt(k), _stream(k))
        else:
            perm = _perm32(perm, S)
            rc = lib.psa_ksim_perm(_ptr(k), _ptr(perm), _ptr(out), B * H, S, D, block_n, t2, t4, t8, _dt(k), _stream(k))
    check(rc, "psa_ksim")
    return out


# ------------------------------------------------------------------------------------------------
def psa_forward(q, k, v, mask, block_m: int, block_n: int, tile_n: int, sm_scale: Optional[float] = None,
                compat_quirk: bool = True, impl: int = IMPL_AUTO, pyramid=None, out=None, out_perm=None) -> torch.Tensor:
    """Multi-level block-sparse forward on the separator-format mask
    (_forward, src/psa_triton/kernels/psa_kernel.py:351-432).  out_perm (tile-image path only): output row t is stored
    at row out_perm[t]."""
    _need_cuda(q, k, v, mask)
    assert q.shape[-1] == k.shape[-1] == v.shape[-1]
    assert k.shape[2] == v.shape[2]
    assert q.shape[-1] in [64, 128]
    q, k, v, mask = _flat_bh(q), _flat_bh(k), _flat_bh(v), _mask32(mask)
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if sm_scale is None:
        sm_scale = D ** -0.5
    use_images = isinstance(pyramid, KVImages) or (pyramid is None and impl == IMPL_AUTO and mask.shape[-1] <= 1472
                                                   and images_supported(k, block_m, block_n, tile_n) and sm_scale > 0)
    if use_images:
        if pyramid is None:
            pyramid = pyramid_kv_images(k, v, block_n)
        with torch.cuda.device(q.device):
            o = out if out is not None else torch.empty_like(q)
            status = status_word(q.device)
            if out_perm is None:
                rc = lib.psa_fwd_images(_ptr(q), _ptr(pyramid.kimg), _ptr(pyramid.vimg), _ptr(mask), _ptr(o), B * H, Sq, Sk, D,
                                        block_m, block_n, tile_n, mask.shape[-1], float(sm_scale), int(compat_quirk), _dt(q),
                                        _ptr(status), _stream(q))
            else:
                out_perm = _perm32(out_perm, Sq)
                rc = lib.psa_fwd_images_perm(_ptr(q), _ptr(pyramid.kimg), _ptr(pyramid.vimg), _ptr(mask), _ptr(o),
                                             _ptr(out_perm), B * H, Sq, Sk, D, block_m, block_n, tile_n, mask.shape[-1],
                                             float(sm_scale), int(compat_quirk), _dt(q), _ptr(status), _stream(q))
        check(rc, "psa_fwd_images")
        o._psa_status = status
        return o
    if out_perm is not None:
        raise ValueError("out_perm needs the tile-image forward (f16/bf16, block_m 128, tile_n 32, block_n 64/128)")
    if pyramid is None:
        pyramid = pyramid_kv(k, v, block_n)
    (k2, k4, k8), (v2, v4, v8) = pyramid
    with torch.cuda.device(q.device):
        o = out if out is not None else torch.empty_like(q)
        status = status_word(q.device)
        rc = lib.psa_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(k2), _ptr(k4), _ptr(k8), _ptr(v2), _ptr(v4), _ptr(v8),
                         _ptr(mask), _ptr(o), B * H, Sq, Sk, D, block_m, block_n, tile_n, mask.shape[-1],
                         float(sm_scale), int(compat_quirk), impl, _dt(q), _ptr(status), _stream(q))
    check(rc, "psa_fwd")
    o._psa_status = status     # read lazily by callers that want to check for an expired device wait
    return o


class LegacyKV:
    """Pooled K/V of the legacy kernels (block 128) in the two layouts their kernels read, each built on first use: tile
    images (tcgen05 forward and backward) and row-major levels 2/4/8 (scalar and warp-level-mma kernels)."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, images: Optional[KVImages] = None, rows=None):
        self.k, self.v, self._images, self._rows = k, v, images, rows

    def images(self) -> KVImages:
        if self._images is None:
            self._images = pyramid_kv_images(self.k, self.v, 128)
        return self._images

    def rows(self):
        if self._rows is None:
            self._rows = pyramid_kv(self.k, self.v, 128)
        return self._rows


IMPL_WARP_MMA = 3      # legacy backward only: the warp-level mma.sync kernels


def _legacy_tc_ok(q: torch.Tensor, sm_scale: float) -> bool:
    return q.dtype in (torch.float16, torch.bfloat16) and -(-q.shape[2] // 128) + 5 <= 1472 and sm_scale > 0


def legacy_forward(q, k, v, mask, causal: bool = False, sm_scale: Optional[float] = None, need_lse: bool = False,
                   pyramid=None, impl: int = IMPL_AUTO):
    """Legacy forward on the dense old-format mask (_forward, src/psa_triton/kernels/psa_kernel_legacy.py:837-938).
    Returns (o, lse or None, LegacyKV or None): a training step (need_lse) gets the log-sum-exp rows and the pooled
    K/V for its backward."""
    _need_cuda(q, k, v, mask)
    assert q.shape[-1] == k.shape[-1] == v.shape[-1]
    assert k.shape[2] == v.shape[2]
    assert q.shape[-1] in [64, 128]
    q, k, v, mask = _flat_bh(q), _flat_bh(k), _flat_bh(v), _mask32(mask)
    B, H, S, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    kv = pyramid if isinstance(pyramid, LegacyKV) else LegacyKV(k, v, rows=pyramid)
    if impl != IMPL_SCALAR and _legacy_tc_ok(q, sm_scale):
        # 16-bit tensors: the tcgen05 forward on tile images (which the tcgen05 backward reads again)
        imgs = kv.images()
        with torch.cuda.device(q.device):
            o = torch.empty_like(q)
            lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device) if need_lse else None
            scratch = torch.empty(lib.psa_legacy_index_bytes(B * H, S) // 4, dtype=torch.int32, device=q.device)
            status = status_word(q.device)
            rc = lib.psa_legacy_fwd_images(_ptr(q), _ptr(imgs.kimg), _ptr(imgs.vimg), _ptr(mask), _ptr(scratch), _ptr(o), _ptr(lse),
                                           B * H, S, D, mask.shape[-1], float(sm_scale), int(causal), _dt(q), _ptr(status), _stream(q))
        check(rc, "psa_legacy_fwd_images")
        o._psa_status = status
        return o, lse, (kv if need_lse else None)
    (k2, k4, k8), (v2, v4, v8) = kv.rows()
    with torch.cuda.device(q.device):
        o = torch.empty_like(q)
        lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device) if need_lse else None
        rc = lib.psa_legacy_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(k2), _ptr(k4), _ptr(k8), _ptr(v2), _ptr(v4), _ptr(v8),
                                _ptr(mask), _ptr(o), _ptr(lse), B * H, S, D, mask.shape[-1], float(sm_scale), int(causal),
                                _dt(q), _stream(q))
    check(rc, "psa_legacy_fwd")
    return o, lse, kv


def legacy_forward_reordered(q, k, v, mask, perm: torch.Tensor, sm_scale: Optional[float] = None) -> torch.Tensor:
    """The legacy forward (not causal, inference) of q[..., perm, :], k[..., perm, :], v[..., perm, :] with the result put
    back in the stored order - without reordered copies of k, v or the output: the tile images are built through perm,
    only q is gathered, and the forward stores output row t at row perm[t].  mask: the level mask of the reordered
    sequence (old format)."""
    _need_cuda(q, k, v, mask, perm)
    q, k, v, mask = _flat_bh(q), _flat_bh(k), _flat_bh(v), _mask32(mask)
    B, H, S, D = q.shape
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    if not _legacy_tc_ok(q, sm_scale):
        raise ValueError("the reordered legacy forward needs f16/bf16 tensors, at most 1467 blocks of 128 tokens and a positive scale")
    perm = _perm32(perm, S)
    imgs = pyramid_kv_images(k, v, 128, perm=perm)
    q_r = gather_rows(q, perm)
    with torch.cuda.device(q.device):
        o = torch.empty_like(q)
        scratch = torch.empty(lib.psa_legacy_index_bytes(B * H, S) // 4, dtype=torch.int32, device=q.device)
        status = status_word(q.device)
        rc = lib.psa_legacy_fwd_images_perm(_ptr(q_r), _ptr(imgs.kimg), _ptr(imgs.vimg), _ptr(mask), _ptr(scratch), _ptr(o), _ptr(perm),
                                            B * H, S, D, mask.shape[-1], float(sm_scale), _dt(q), _ptr(status), _stream(q))
    check(rc, "psa_legacy_fwd_images_perm")
    o._psa_status = status
    return o


def legacy_forward_tc(q, k, v, mask, sm_scale: Optional[float] = None, need_lse: bool = True, causal: bool = False):
    """Legacy forward on the tcgen05 kernel (psa_legacy_fwd_images); returns (o, lse or None)."""
    _need_cuda(q, k, v, mask)
    sm_scale = q.shape[-1] ** -0.5 if sm_scale is None else sm_scale
    if not _legacy_tc_ok(q, sm_scale):
        raise ValueError("the tcgen05 legacy forward needs f16/bf16 tensors, at most 1467 blocks of 128 tokens and a positive scale")
    o, lse, _ = legacy_forward(q, k, v, mask, causal, sm_scale, need_lse=need_lse, impl=IMPL_TENSOR)
    return o, lse


def legacy_backward(q, k, v, mask, o, lse, do, causal: bool, sm_scale: float, pyramid=None, impl: int = IMPL_AUTO):
    """dQ, dK, dV of the legacy kernel (_sparse_attention.backward, psa_kernel_legacy.py:947-1069).  16-bit tensors run
    on the tcgen05 kernels (impl IMPL_AUTO / IMPL_TENSOR); IMPL_WARP_MMA selects the warp-level mma kernels, IMPL_SCALAR
    the fp32 ones (the only choice for float32 tensors).  pyramid: the LegacyKV of the forward (rebuilt if None)."""
    _need_cuda(q, k, v, mask, o, lse, do)
    q, k, v, o, do, mask = _flat_bh(q), _flat_bh(k), _flat_bh(v), _flat_bh(o), _flat_bh(do), _mask32(mask)
    B, H, S, D = q.shape
    kv = pyramid if isinstance(pyramid, LegacyKV) else LegacyKV(k, v, rows=pyramid)
    half = q.dtype in (torch.float16, torch.bfloat16)
    if impl == IMPL_AUTO:
        impl = IMPL_TENSOR if (half and _legacy_tc_ok(q, sm_scale)) else IMPL_SCALAR
    with torch.cuda.device(q.device):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if impl == IMPL_TENSOR:
            if not (half and _legacy_tc_ok(q, sm_scale)):
                raise ValueError("the tcgen05 legacy backward needs f16/bf16 tensors, at most 1467 blocks of 128 tokens and a positive scale")
            imgs = kv.images()
            nbytes = lib.psa_legacy_bwd_scratch_bytes(B * H, S, D)
            scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
            status = status_word(q.device)
            rc = lib.psa_legacy_bwd_tcgen05(_ptr(q), _ptr(imgs.kimg), _ptr(imgs.vimg), _ptr(mask), _ptr(o), _ptr(lse), _ptr(do),
                                            _ptr(dq), _ptr(dk), _ptr(dv), _ptr(scratch), nbytes, B * H, S, D, mask.shape[-1],
                                            float(sm_scale), int(causal), _dt(q), _ptr(status), _stream(q))
            check(rc, "psa_legacy_bwd_tcgen05")
            dq._psa_status = status
            return dq, dk, dv
        (k2, k4, k8), (v2, v4, v8) = kv.rows()
        delta = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
        fn = lib.psa_legacy_bwd_tc if impl == IMPL_WARP_MMA else lib.psa_legacy_bwd
        rc = fn(_ptr(q), _ptr(k), _ptr(v), _ptr(k2), _ptr(k4), _ptr(k8), _ptr(v2), _ptr(v4), _ptr(v8),
                _ptr(mask), _ptr(o), _ptr(lse), _ptr(do), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(delta),
                B * H, S, D, mask.shape[-1], float(sm_scale), int(causal), _dt(q), _stream(q))
    check(rc, "psa_legacy_bwd")
    return dq, dk, dv
