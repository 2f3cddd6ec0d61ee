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


def logfmt_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """What a bf16 tensor looks like after the LogFMT-10 wire format of the low-latency combine.

    Per group of 128 channels (last dimension): with ``amax`` / ``amin`` the largest / smallest magnitude, the group
    is encoded only if ``amax < 1`` and ``amin < amax``; then every value becomes its sign and a 9-bit code on a
    logarithmic grid of 510 steps from ``amin`` (clipped to ``amax * 2**-32``) to ``amax``, rounded to the nearest
    grid value in the linear domain; code 0 is an exact zero. Other groups are returned unchanged. The result is
    float32 (the receiver accumulates in float32 before its single rounding to bf16). The GPU kernel uses the
    hardware's approximate ``log2`` / ``exp2``, so a value that sits on a rounding boundary may land one grid step
    away from this restatement. Reference: ``csrc/kernels/legacy/internode_ll.cu:556-712``.
    """
    assert x.size(-1) % 128 == 0
    xf = x.float().reshape(-1, x.size(-1) // 128, 128)
    mag = xf.abs()
    amax = mag.amax(dim=-1, keepdim=True)
    amin = mag.amin(dim=-1, keepdim=True)
    log_amax = torch.log2(amax)
    log_amin = torch.maximum(torch.log2(amin), log_amax - 32.0)
    cast = (log_amax < 0) & (log_amin < log_amax)
    step = (log_amax - log_amin) / 510.0
    safe_step = torch.where(cast, step, torch.ones_like(step))
    rounding = 2.0 - torch.log2((1.0 + torch.exp2(safe_step)) * 0.5) / safe_step
    base = torch.where(cast, log_amin, torch.zeros_like(log_amin))
    code = torch.floor(torch.clamp((torch.log2(mag) - base) / safe_step + rounding, min=0.0)).clamp(max=511.0)
    decoded = torch.where(code == 0, torch.zeros_like(mag), torch.exp2((code - 1.0) * safe_step + base))
    decoded = torch.where(xf < 0, -decoded, decoded)
    return torch.where(cast, decoded, xf).reshape(x.shape)


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
