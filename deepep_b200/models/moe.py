"""Fused expert-parallel MoE layer (forward and backward) on the kernels of this library.

Forward, per rank::

    router logits --router_topk--> (topk_idx, topk_weights)
    x --dispatch (expanded, expert-major, 128-aligned; optional in-kernel e4m3 cast)--> rows
    rows --grouped tcgen05 GEMM (W13: gate|up)--> h1 --SwiGLU * gate weight (optional fused cast)--> a
    a --grouped tcgen05 GEMM (W2)--> h2 --combine (sum over experts, fp32 accumulate)--> y

The expert GEMMs read the dispatch's device-resident prefix array as their group table, so nothing
but the dispatch itself synchronises with the host. The gate weight is applied inside the SwiGLU
kernel, which makes the combine a plain sum. Backward reverses the same pipeline: the gradient of
the combine is a cached (replayed) dispatch, the gradient of the dispatch is a combine, the data
gradients are grouped GEMMs with the transposed weights, the weight gradients are two GEMM launches
grouped along the contraction dimension (all experts at once, segment bounds read on the device), and
the gradient of the gate weights rides back with the combine. The router runs on the same tensor-core
GEMM (``_RouterFunction``).

The reference library has no model code; this is the "fused MoE layer fwd+bwd" workload that its
kernels exist to serve. Everything is written over LISTS of ranks so that the single-GPU emulation
(``LocalCluster``) and the real one-rank-per-process case share one code path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional, Sequence, Tuple

import torch

from .._native import _C, require_native


@dataclass
class MoEConfig:
    hidden: int
    intermediate: int
    num_experts: int
    num_topk: int
    use_fp8: bool = False          # e4m3 dispatch + e4m3 expert GEMMs (weights 128x128 block scaled), bf16 gradients
    pow2_scales: bool = False      # with use_fp8: every scale is a power of two (UE8M0), applied by the tensor core itself
    expert_alignment: int = 128
    num_sms: int = 24


def quantize_weight_128x128(w: torch.Tensor, pow2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[G, N, K]`` -> (e4m3 ``[G, N, K]``, fp32 scales ``[G, N / 128, K / 128]``); ``pow2`` rounds the scales up to
    powers of two."""
    G, N, K = w.shape
    blocks = w.float().view(G, N // 128, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(2, 4)).clamp(1e-4)
    scale = torch.div(amax, torch.full_like(amax, 448.0))
    if pow2:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (blocks / scale[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(G, N, K)
    return q, scale.contiguous()


class ExpertWeights:
    """This rank's experts: ``w13 [local experts, 2 * intermediate, hidden]`` (gate rows first, then up) and
    ``w2 [local experts, hidden, intermediate]`` in bf16, plus the derived copies the kernels read."""

    def __init__(self, w13: torch.Tensor, w2: torch.Tensor, use_fp8: bool, pow2_scales: bool = False):
        self.w13, self.w2, self.use_fp8, self.pow2_scales = w13.contiguous(), w2.contiguous(), use_fp8, pow2_scales
        self.refresh()

    def refresh(self) -> None:
        """Rebuilds the transposed (for data gradients) and quantised (for FP8 forward) copies after an update."""
        self.w13_t = self.w13.transpose(1, 2).contiguous()     # [EL, hidden, 2I]
        self.w2_t = self.w2.transpose(1, 2).contiguous()       # [EL, I, hidden]
        if self.use_fp8:
            self.w13_q, self.w13_sf = quantize_weight_128x128(self.w13, self.pow2_scales)
            self.w2_q, self.w2_sf = quantize_weight_128x128(self.w2, self.pow2_scales)


class _SingleRankComm:
    """Gives one ``ElasticBuffer`` the list interface of ``LocalCluster``."""

    def __init__(self, buffer):
        self.buffers = [buffer]

    def dispatch(self, per_rank_kwargs):
        return [self.buffers[0].dispatch(**per_rank_kwargs[0])]

    def combine(self, per_rank_kwargs):
        return [self.buffers[0].combine(**per_rank_kwargs[0])]


def route(logits: torch.Tensor, num_topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k experts and softmax weights over the selected logits (hand-written kernel)."""
    require_native()
    return _C.router_topk(logits.float().contiguous(), num_topk)


def moe_forward(comm, weights: Sequence[ExpertWeights], xs: Sequence[torch.Tensor], topk_idx: Sequence[torch.Tensor],
                topk_weights: Sequence[torch.Tensor], cfg: MoEConfig):
    """Expert part of the layer for all ranks of ``comm``. Returns ``(ys, contexts)``."""
    R = len(xs)
    out = comm.dispatch([dict(x=xs[r], topk_idx=topk_idx[r], topk_weights=topk_weights[r], num_experts=cfg.num_experts,
                              expert_alignment=cfg.expert_alignment, do_expand=True, do_zero_padding=True, num_sms=cfg.num_sms,
                              fused_fp8=cfg.use_fp8, round_scale=cfg.use_fp8 and cfg.pow2_scales) for r in range(R)])
    ctxs, h2s = [], []
    for r in range(R):
        recv_x, _, recv_w, handle, _ = out[r]
        w = weights[r]
        ends = handle.psum_num_recv_tokens_per_expert
        if cfg.use_fp8:
            xq, xsf = recv_x
            pow2 = cfg.pow2_scales and w.pow2_scales
            h1 = _C.gemm(xq, w.w13_q, sfa=xsf, sfb=w.w13_sf, group_end=ends, group_alignment=cfg.expert_alignment, pow2_scales=pow2)
            aq, asf = _C.swiglu(h1, recv_w, None, True, pow2)
            h2 = _C.gemm(aq, w.w2_q, sfa=asf, sfb=w.w2_sf, group_end=ends, group_alignment=cfg.expert_alignment, pow2_scales=pow2)
        else:
            h1 = _C.gemm(recv_x, w.w13, group_end=ends, group_alignment=cfg.expert_alignment)
            a, _ = _C.swiglu(h1, recv_w)
            h2 = _C.gemm(a, w.w2, group_end=ends, group_alignment=cfg.expert_alignment)
        h2s.append(h2)
        ctxs.append(dict(recv_x=recv_x, recv_w=recv_w, handle=handle, h1=h1))
    comb = comm.combine([dict(x=h2s[r], handle=ctxs[r]['handle']) for r in range(R)])
    return [c[0] for c in comb], ctxs


def moe_backward(comm, weights: Sequence[ExpertWeights], ctxs, dys: Sequence[torch.Tensor], cfg: MoEConfig):
    """Gradients of :func:`moe_forward`: ``(dxs, d_topk_weights, dW13s, dW2s)`` (bf16 / fp32 weights grads).

    Nothing here synchronises with the host: the expert segments are read on the device from the dispatch's prefix
    array, both by the grouped data-gradient GEMMs and by the two weight-gradient launches (one GEMM over all experts
    each, grouped along the contraction dimension). The SwiGLU backward kernel also produces the weighted activation
    (operand of the W2 gradient) and the gradient of the gate weights in the same pass.
    """
    R = len(dys)
    # gradient of the combine (a sum): replay the dispatch routing with dy as payload
    out = comm.dispatch([dict(x=dys[r].contiguous(), handle=ctxs[r]['handle'], do_expand=True, do_zero_padding=True,
                              num_sms=cfg.num_sms, fused_fp8=False) for r in range(R)])
    dx_rows, dw_rows, dW13s, dW2s = [], [], [], []
    for r in range(R):
        dh2 = out[r][0]
        c, w = ctxs[r], weights[r]
        handle, h1, recv_w = c['handle'], c['h1'], c['recv_w']
        ends = handle.psum_num_recv_tokens_per_expert
        el = w.w13.size(0)
        x_rows = c['recv_x']
        if cfg.use_fp8:
            x_rows = _C.dequant_1x128(x_rows[0], x_rows[1].contiguous())
        # data gradients
        da = _C.gemm(dh2, w.w2_t, group_end=ends, group_alignment=cfg.expert_alignment)           # [rows, I]
        dh1, a_w, dw_row = _C.swiglu_backward(h1, da, recv_w, True)                                 # [rows, 2I], [rows, I], [rows]
        dw_rows.append(dw_row)
        dx_rows.append(_C.gemm(dh1, w.w13_t, group_end=ends, group_alignment=cfg.expert_alignment))
        # weight gradients: contraction over every expert's (zero padded) rows, all experts in one launch each
        dh2_t, a_t = _C.transpose_bf16(dh2), _C.transpose_bf16(a_w)
        dh1_t, x_t = _C.transpose_bf16(dh1), _C.transpose_bf16(x_rows)
        dW2s.append(_C.gemm_k_grouped(dh2_t, a_t, ends, el, cfg.expert_alignment))               # [EL, hidden, I]
        dW13s.append(_C.gemm_k_grouped(dh1_t, x_t, ends, el, cfg.expert_alignment))              # [EL, 2I, hidden]
    # gradient of the dispatch: a combine that also carries the gate-weight gradients back
    comb = comm.combine([dict(x=dx_rows[r], handle=ctxs[r]['handle'], topk_weights=dw_rows[r].contiguous()) for r in range(R)])
    return [c[0] for c in comb], [c[1] for c in comb], dW13s, dW2s


class _RouterFunction(torch.autograd.Function):
    """Router of the layer on this library's kernels: logits = x @ W_r^T on the tcgen05 GEMM (bf16 operands, fp32
    accumulation), top-k and softmax over the selected logits in ``router_topk``; the backward pass turns the gradient
    of the top-k weights into the gradient of the logits (softmax Jacobian over the selected experts, zero elsewhere)
    and into two more tensor-core GEMMs for dW_r and dx."""

    @staticmethod
    def forward(ctx, x, router, num_topk):
        E = router.size(0)
        router_bf16 = router.detach().to(torch.bfloat16)
        if E % 128 != 0:                                                        # the GEMM tiles N in multiples of 128: zero rows
            router_bf16 = torch.nn.functional.pad(router_bf16, (0, 0, 0, -(-E // 128) * 128 - E))
        router_bf16 = router_bf16.contiguous()
        logits = _C.gemm(x.detach().contiguous(), router_bf16)[:, :E]          # [T, E] bf16
        topk_idx, topk_weights = _C.router_topk(logits.float().contiguous(), num_topk)
        ctx.save_for_backward(x, router_bf16, topk_idx, topk_weights)
        ctx.router_dtype, ctx.num_experts = router.dtype, E
        ctx.mark_non_differentiable(topk_idx)
        return topk_idx, topk_weights

    @staticmethod
    def backward(ctx, _d_idx, d_weights):
        x, router_bf16, topk_idx, w = ctx.saved_tensors
        T, E = x.size(0), router_bf16.size(0)                                  # E: padded to a multiple of 128
        # d logit_k = w_k * (dw_k - sum_j w_j dw_j) on the selected experts
        inner = (w * d_weights).sum(dim=1, keepdim=True)
        d_sel = (w * (d_weights - inner)).to(torch.bfloat16)
        d_logits = torch.zeros((T, E), dtype=torch.bfloat16, device=x.device)
        d_logits.scatter_(1, topk_idx.clamp(min=0), torch.where(topk_idx >= 0, d_sel, torch.zeros_like(d_sel)))
        pad_t = -(-T // 64) * 64                                               # the GEMM wants K (here: tokens) in multiples of 64
        if pad_t != T:
            d_logits = torch.nn.functional.pad(d_logits, (0, 0, 0, pad_t - T))
            x_p = torch.nn.functional.pad(x.detach(), (0, 0, 0, pad_t - T))
        else:
            x_p = x.detach()
        dx = _C.gemm(d_logits[:T].contiguous(), _C.transpose_bf16(router_bf16))                         # [T, H] = dlogits @ W_r
        d_router = _C.gemm(_C.transpose_bf16(d_logits), _C.transpose_bf16(x_p.contiguous()))             # [E, H] = dlogits^T @ x
        return dx, d_router[:ctx.num_experts].to(ctx.router_dtype), None


class _MoEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_weights, w13, w2, layer, topk_idx):
        ys, ctxs = moe_forward(layer.comm, [layer.weights], [x], [topk_idx], [topk_weights.detach()], layer.cfg)
        ctx.layer, ctx.saved = layer, ctxs
        return ys[0]

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        dxs, dws, dW13s, dW2s = moe_backward(layer.comm, [layer.weights], ctx.saved, [dy], layer.cfg)
        return dxs[0], dws[0], dW13s[0], dW2s[0], None, None


class FusedMoE(torch.nn.Module):
    """Expert-parallel MoE layer of one rank: ``y = sum_k w_k * Expert_k(x)`` with SwiGLU experts.

    Arguments:
        buffer: the rank's ``ElasticBuffer`` (sized for the layer's tokens / hidden / top-k).
        cfg: layer shape.
    Weights are initialised N(0, 0.02).
    """

    def __init__(self, buffer, cfg: MoEConfig, device='cuda', seed: int = 0):
        super().__init__()
        require_native()
        self.cfg, self.buffer = cfg, buffer
        self.comm = _SingleRankComm(buffer)
        el = cfg.num_experts // buffer.num_ranks
        g = torch.Generator(device='cpu').manual_seed(seed + buffer.rank_idx)
        self.router = torch.nn.Parameter((torch.randn((cfg.num_experts, cfg.hidden), generator=g) * 0.02).to(device))
        self.w13 = torch.nn.Parameter((torch.randn((el, 2 * cfg.intermediate, cfg.hidden), generator=g) * 0.02).bfloat16().to(device))
        self.w2 = torch.nn.Parameter((torch.randn((el, cfg.hidden, cfg.intermediate), generator=g) * 0.02).bfloat16().to(device))
        self.weights = ExpertWeights(self.w13.data, self.w2.data, cfg.use_fp8, cfg.pow2_scales)

    def refresh_weights(self) -> None:
        """Call after an optimizer step: rebuilds the transposed / quantised weight copies."""
        self.weights = ExpertWeights(self.w13.data, self.w2.data, self.cfg.use_fp8, self.cfg.pow2_scales)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        topk_idx, topk_weights = _RouterFunction.apply(x, self.router, self.cfg.num_topk)
        return _MoEFunction.apply(x, topk_weights, self.w13, self.w2, self, topk_idx)


def reference_moe(xs, topk_idx, topk_weights, w13_all: torch.Tensor, w2_all: torch.Tensor):
    """Dense fp32 reference over ALL experts (``w13_all [E, 2I, H]``, ``w2_all [E, H, I]``): per-rank outputs."""
    outs = []
    inter = w13_all.size(1) // 2
    for x, idx, w in zip(xs, topk_idx, topk_weights):
        y = torch.zeros_like(x, dtype=torch.float32)
        for k in range(idx.size(1)):
            e = idx[:, k]
            ok = e >= 0
            ee = e.clamp(min=0)
            h = torch.einsum('th,tfh->tf', x.float(), w13_all[ee].float())
            a = torch.nn.functional.silu(h[:, :inter]) * h[:, inter:]
            o = torch.einsum('ti,thi->th', a, w2_all[ee].float())
            y = y + torch.where(ok[:, None], o * w[:, k:k + 1].float(), torch.zeros_like(o))
        outs.append(y)
    return outs
