"""The compute kernels that sit next to the communication in an MoE / tensor-parallel layer.

Thin, typed entry points over the native module (all kernels are hand-written sm_100a CUDA, none calls a
library GEMM), each with the plain PyTorch fp32 function it is tested against (``ref_*``). The reference
library has no compute operators; its tests use ``per_token_cast_to_fp8`` / ``per_token_cast_back``
(``deep_ep/utils/math.py:30-56``), which ``quant_1x128`` / ``dequant_1x128`` reproduce bit for bit.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .._native import require_native

__all__ = ['gemm', 'grouped_gemm', 'router_topk', 'quant_1x128', 'dequant_1x128', 'swiglu', 'swiglu_backward', 'transpose',
           'ref_gemm', 'ref_grouped_gemm', 'ref_router_topk', 'ref_swiglu']


def gemm(a: torch.Tensor, b: torch.Tensor, sfa: Optional[torch.Tensor] = None, sfb: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, num_sms: int = 0) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T -> bf16 [M, N]`` on the tcgen05 tensor cores.

    bf16 operands, or e4m3 operands with ``sfa [M, K/128]`` (1x128) and ``sfb [N/128, K/128]`` (128x128) fp32
    block scales. ``K`` must be a multiple of 64 (bf16) or 128 (fp8), ``N`` of 128.
    """
    C = require_native()
    return C.gemm(a, b, sfa, sfb, None, 1, out, num_sms)


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, group_end: torch.Tensor, group_alignment: int = 128,
                 sfa: Optional[torch.Tensor] = None, sfb: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 num_sms: int = 0) -> torch.Tensor:
    """Expert-major grouped GEMM: rows ``[start_g, group_end[g])`` of ``a`` multiply ``b[g] [N, K]``, where
    ``start_0 = 0`` and ``start_g = align(group_end[g-1], group_alignment)``.

    ``group_end`` is a device int32 tensor, e.g. ``EPHandle.psum_num_recv_tokens_per_expert`` of an expanded
    dispatch: no host synchronisation sits between the dispatch and the expert GEMM. Rows in the alignment gaps
    are written as zeros when ``group_alignment`` is a multiple of 128, otherwise left untouched.
    """
    C = require_native()
    assert b.dim() == 3 and group_end.dtype == torch.int32 and group_end.numel() == b.size(0)
    return C.gemm(a, b, sfa, sfb, group_end, group_alignment, out, num_sms)


def router_topk(logits: torch.Tensor, num_topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k experts per token (descending logits, int64) and the softmax over the selected logits (fp32)."""
    return require_native().router_topk(logits, num_topk)


def quant_1x128(x: torch.Tensor, pow2_scales: bool = False, col_major_sf: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[M, H]`` -> e4m3 ``[M, H]`` and fp32 scales ``[M, H/128]`` (``amax / 448`` per 128 channels, optionally
    rounded up to a power of two; ``col_major_sf`` returns the scales with unit stride along tokens, padded to 4)."""
    return require_native().quant_1x128(x, pow2_scales, col_major_sf)


def dequant_1x128(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`quant_1x128` (bf16 result)."""
    return require_native().dequant_1x128(q, sf)


def swiglu(x: torch.Tensor, row_weight: Optional[torch.Tensor] = None, num_valid_rows: Optional[torch.Tensor] = None,
           quant: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``silu(x[:, :I]) * x[:, I:] * row_weight`` for bf16 ``x [M, 2I]``; with ``quant`` the result leaves as e4m3 with
    1x128 scales (the cast is fused). ``num_valid_rows`` (device int32 scalar) bounds the rows that are computed."""
    return require_native().swiglu(x, row_weight, num_valid_rows, quant)


def swiglu_backward(x: torch.Tensor, dout: torch.Tensor, row_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gradient of :func:`swiglu` with respect to ``x``."""
    return require_native().swiglu_backward(x, dout, row_weight)


def transpose(x: torch.Tensor) -> torch.Tensor:
    """bf16 ``[M, N]`` -> contiguous ``[N, M]`` through shared-memory tiles (weight-gradient GEMMs need K-major operands)."""
    return require_native().transpose_bf16(x)


# ------------------------------------------------------------------ plain PyTorch fp32 references
def ref_gemm(a: torch.Tensor, b: torch.Tensor, sfa: Optional[torch.Tensor] = None, sfb: Optional[torch.Tensor] = None) -> torch.Tensor:
    af, bf = a.float(), b.float()
    if sfa is not None:
        af = af * sfa.float().repeat_interleave(128, dim=1)[:, :a.size(1)]
        bf = bf * sfb.float().repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)[:b.size(0), :b.size(1)]
    return af @ bf.t()


def ref_grouped_gemm(a: torch.Tensor, b: torch.Tensor, group_end: torch.Tensor, group_alignment: int = 128) -> torch.Tensor:
    out = torch.zeros((a.size(0), b.size(1)), dtype=torch.float32, device=a.device)
    start = 0
    for g, end in enumerate(group_end.tolist()):
        out[start:end] = a[start:end].float() @ b[g].float().t()
        start = -(-end // group_alignment) * group_alignment
    return out


def ref_router_topk(logits: torch.Tensor, num_topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    vals, idx = torch.topk(logits.float(), num_topk, dim=1, sorted=True)
    return idx, torch.softmax(vals, dim=1)


def ref_swiglu(x: torch.Tensor, row_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    half = x.size(1) // 2
    out = torch.nn.functional.silu(x[:, :half].float()) * x[:, half:].float()
    return out if row_weight is None else out * row_weight.float()[:, None]
