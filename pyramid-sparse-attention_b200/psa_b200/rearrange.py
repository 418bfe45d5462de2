"""Token reordering along a generalized Hilbert ("gilbert") curve over the T x H x W latent grid.

Mirrors GilbertRearranger (src/psa_triton/utils/rearranger.py:14-132): video tokens are gathered in curve order, text
tokens (if any) are moved to the END of the sequence; ``reversed_rearrange`` undoes both.  The curve itself is the
published generalized-Hilbert construction for arbitrary cuboids (J. Cerveny, 2018), restated here with integer vector
arithmetic and an explicit work stack; the resulting visiting order is checked against the reference's in the fixtures.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np
import torch


def _sign(v: np.ndarray) -> np.ndarray:
    return np.sign(v).astype(np.int64)


def _half_even(vec: np.ndarray, unit: np.ndarray, extent: int) -> np.ndarray:
    """Half of an axis vector (floor division, as Python does for negatives), bumped by one unit step when the half is
    odd and the full extent exceeds 2 - the curve prefers even splits."""
    h = vec // 2
    if (abs(int(h.sum())) % 2) and extent > 2:
        h = h + unit
    return h


def gilbert_order(width: int, height: int, depth: int) -> np.ndarray:
    """Linear indices x + width*(y + height*z) of the grid cells in curve order."""
    out = np.empty(width * height * depth, dtype=np.int64)
    n = 0
    X = np.array([width, 0, 0], dtype=np.int64)
    Y = np.array([0, height, 0], dtype=np.int64)
    Z = np.array([0, 0, depth], dtype=np.int64)
    if width >= height and width >= depth:
        first = (X, Y, Z)
    elif height >= width and height >= depth:
        first = (Y, X, Z)
    else:
        first = (Z, X, Y)
    stack = [(np.zeros(3, dtype=np.int64),) + first]
    stride = np.array([1, width, width * height], dtype=np.int64)
    while stack:
        pos, a, b, c = stack.pop()
        w, h, d = abs(int(a.sum())), abs(int(b.sum())), abs(int(c.sum()))
        ua, ub, uc = _sign(a), _sign(b), _sign(c)
        # a line of cells along one axis
        line = None
        if h == 1 and d == 1:
            line = (w, ua)
        elif w == 1 and d == 1:
            line = (h, ub)
        elif w == 1 and h == 1:
            line = (d, uc)
        if line is not None:
            cnt, step = line
            cells = pos[None, :] + np.arange(cnt, dtype=np.int64)[:, None] * step[None, :]
            out[n:n + cnt] = cells @ stride
            n += cnt
            continue
        a2, b2, c2 = _half_even(a, ua, w), _half_even(b, ub, h), _half_even(c, uc, d)
        if 2 * w > 3 * h and 2 * w > 3 * d:                       # long box: cut across the major axis only
            parts = [(pos, a2, b, c), (pos + a2, a - a2, b, c)]
        elif 3 * h > 4 * d:                                          # shallow in c: three pieces in the a-b plane
            parts = [(pos, b2, c, a2),
                     (pos + b2, a, b - b2, c),
                     (pos + (a - ua) + (b2 - ub), -b2, c, -(a - a2))]
        elif 3 * d > 4 * h:                                          # shallow in b: three pieces in the a-c plane
            parts = [(pos, c2, a2, b),
                     (pos + c2, a, b, c - c2),
                     (pos + (a - ua) + (c2 - uc), -c2, -(a - a2), b)]
        else:                                                        # general case: five sub-boxes
            parts = [(pos, b2, c2, a2),
                     (pos + b2, c, a2, b - b2),
                     (pos + (b2 - ub) + (c - uc), a, -b2, -(c - c2)),
                     (pos + (a - ua) + b2 + (c - uc), -c, -(a - a2), b - b2),
                     (pos + (a - ua) + (b2 - ub), -b2, c2, -(a - a2))]
        stack.extend(reversed(parts))                                # LIFO: first piece is processed next
    assert n == out.size
    return out


class GilbertRearranger:
    """Same interface as the reference class: rearrange(q, k, v), rearrange_single(x), reversed_rearrange(out)."""

    def __init__(self, width: int, height: int, depth: int, text_length: int = 224):
        self.width, self.height, self.depth = width, height, depth
        self.total_elements = width * height * depth
        self.text_length = text_length
        order = gilbert_order(width, height, depth)                  # curve position -> original linear index
        inverse = np.empty_like(order)
        inverse[order] = np.arange(order.size)
        self.original_order2gilbert_order_cpu = torch.from_numpy(order)      # gather indices, original -> curve
        self.gilbert_order2original_order_cpu = torch.from_numpy(inverse)    # gather indices, curve -> original
        self._device_cache = {}

    def _indices(self, device, forward: bool) -> torch.Tensor:
        key = (str(device), forward)
        if key not in self._device_cache:
            src = self.original_order2gilbert_order_cpu if forward else self.gilbert_order2original_order_cpu
            self._device_cache[key] = src.to(device, non_blocking=True)
        return self._device_cache[key]

    def source_rows(self, device) -> torch.Tensor:
        """int32 [video + text]: row t of the rearranged sequence is row source_rows[t] of the tensor as the model
        holds it (text first).  rearrange_single(x) == x[..., source_rows, :], and writing row t of the attention's
        output to row source_rows[t] is reversed_rearrange - what the kernels that take a row table use."""
        key = (str(device), "rows")
        if key not in self._device_cache:
            video = self.original_order2gilbert_order_cpu.to(torch.int32) + self.text_length
            text = torch.arange(self.text_length, dtype=torch.int32)
            self._device_cache[key] = torch.cat((video, text)).to(device)
        return self._device_cache[key]

    def rearrange_single(self, x: torch.Tensor) -> torch.Tensor:
        idx = self._indices(x.device, True)
        if self.text_length == 0:
            return x.index_select(-2, idx)
        text, video = x[..., :self.text_length, :], x[..., self.text_length:, :]
        return torch.cat((video.index_select(-2, idx), text), dim=-2)

    def rearrange(self, q, k, v) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return self.rearrange_single(q), self.rearrange_single(k), self.rearrange_single(v)

    def reversed_rearrange(self, out: torch.Tensor) -> torch.Tensor:
        idx = self._indices(out.device, False)
        if self.text_length == 0:
            return out.index_select(-2, idx)
        video, text = out[..., :-self.text_length, :], out[..., -self.text_length:, :]
        return torch.cat((text, video.index_select(-2, idx)), dim=-2)
