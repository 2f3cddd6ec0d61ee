"""Numeric helpers used by the tests, the oracle and the benchmarks (plain PyTorch, any device).

Parity: deep_ep/utils/math.py:5-103 of the reference. The block-FP8 helpers restate the
1x128 recipe (amax floor 1e-4, scale = amax / 448) that the fused dispatch kernels implement
on the device; they are eager PyTorch here, not a compiled graph.
"""
from __future__ import annotations

from typing import Tuple

import torch

FP8_MAX = 448.0
FP8_AMAX_FLOOR = 1e-4
FP8_BLOCK = 128


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def safe_div(a, b) -> float:
    if b == 0:
        if a == 0:
            return 0
        raise ZeroDivisionError(f'{a} / 0')
    return a / b


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - cosine-like similarity of (x + 1, y + 1); 0 for identical tensors."""
    a, b = x.double() + 1, y.double() + 1
    denom = (a * a + b * b).sum()
    return float(1 - 2 * (a * b).sum() / denom)


def _pad_to_blocks(x: torch.Tensor) -> Tuple[torch.Tensor, int]:
    n = x.size(1)
    padded = align(n, FP8_BLOCK)
    if padded != n:
        x = torch.nn.functional.pad(x, (0, padded - n))
    return x, n


def per_token_cast_to_fp8(x: torch.Tensor, round_scale: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[m, n]`` → (e4m3 ``[m, n]``, float scales ``[m, ceil(n / 128)]``), one scale per 128 channels.

    With ``round_scale`` the scale is rounded up to a power of two (what a UE8M0 scale can hold).
    """
    assert x.dim() == 2
    m = x.size(0)
    xp, n = _pad_to_blocks(x)
    blocks = xp.view(m, -1, FP8_BLOCK).float()
    amax = blocks.abs().amax(dim=2).clamp(FP8_AMAX_FLOOR)
    if round_scale:
        scale = torch.exp2(torch.ceil(torch.log2(amax / FP8_MAX)))
        q = blocks * (1.0 / scale).unsqueeze(2)
    else:
        # the device kernels compute scale = amax * (1 / 448) and payload * (448 * (1 / amax)) with one correctly
        # rounded reciprocal; the same operations in the same order here give identical bits on CPU and GPU
        scale = amax * torch.tensor(1.0 / FP8_MAX, dtype=torch.float32, device=amax.device)
        q = blocks * (amax.reciprocal() * FP8_MAX).unsqueeze(2)
    q = q.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(m, -1)[:, :n].contiguous()
    return q, scale


def unpack_ue8m0(packed: torch.Tensor) -> torch.Tensor:
    """int32 packs of four UE8M0 exponents → float scales (one per byte, little endian)."""
    exps = packed.contiguous().view(torch.uint8).to(torch.int32)
    return (exps << 23).view(torch.float32)


def per_token_cast_back(x_fp8: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`per_token_cast_to_fp8`; ``scales`` may be float or packed UE8M0 int32."""
    if x_fp8.numel() == 0:
        return x_fp8.to(torch.bfloat16)
    assert x_fp8.dim() == 2
    m = x_fp8.size(0)
    if scales.dtype == torch.int32:
        scales = unpack_ue8m0(scales)
    xp, n = _pad_to_blocks(x_fp8.float())
    num_blocks = xp.size(1) // FP8_BLOCK
    out = xp.view(m, num_blocks, FP8_BLOCK) * scales.reshape(m, -1)[:, :num_blocks].unsqueeze(2).float()
    return out.view(m, -1)[:, :n].to(torch.bfloat16).contiguous()


def inplace_unique(x: torch.Tensor, num_slots: int) -> None:
    """Rewrites every row of ``x`` to its distinct non-negative values (descending), padded with -1."""
    assert x.dim() == 2
    rows = x.size(0)
    present = torch.zeros((rows, num_slots + 1), dtype=torch.bool, device=x.device)
    present.scatter_(1, x.masked_fill(x < 0, num_slots), True)
    present = present[:, :num_slots]
    ids = torch.arange(num_slots, device=x.device, dtype=x.dtype).expand(rows, -1)
    vals = torch.where(present, ids, torch.full_like(ids, -1))
    vals = torch.sort(vals, dim=1, descending=True).values
    width = min(num_slots, x.size(1))
    x.fill_(-1)
    x[:, :width] = vals[:, :width]


def create_grouped_scores(scores: torch.Tensor, group_idx: torch.Tensor, num_groups: int) -> torch.Tensor:
    """Zeroes the scores of every expert group that is not listed in ``group_idx``."""
    tokens, experts = scores.shape
    keep = torch.zeros((tokens, num_groups), dtype=torch.bool, device=scores.device)
    keep.scatter_(1, group_idx, True)
    return (scores.view(tokens, num_groups, -1) * keep.unsqueeze(-1)).view(tokens, experts)


def hash_tensor(t: torch.Tensor) -> int:
    """Order-insensitive 32-bit fingerprint of the raw bytes (for run-to-run equality checks)."""
    raw = t.contiguous().view(torch.uint8)
    pad = (-raw.numel()) % 4
    if pad:
        raw = torch.nn.functional.pad(raw.flatten(), (0, pad))
    return int(raw.view(torch.int32).sum(dtype=torch.int64).item()) & 0xffffffff


def hash_tensors(*tensors) -> int:
    value = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            value ^= hash_tensors(*t)
        elif isinstance(t, torch.Tensor):
            value ^= hash_tensor(t)
    return value


def count_bytes(*tensors) -> int:
    total = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.numel() * t.element_size()
    return total
