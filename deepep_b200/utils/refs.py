"""Pure-PyTorch oracle for expert-parallel dispatch / combine (any device, any backend).

Two levels:

* ``*_local`` functions take the inputs of ALL ranks as lists and return what one rank must
  receive. They need no process group, which is what the single-GPU emulation tests use.
* ``dispatch`` / ``combine`` are the collective forms: they all-gather the inputs as Python
  objects over the given process group (works with ``gloo`` on CPU and with ``nccl``), then
  call the local functions. A plain ``all_to_all_single`` formulation of the same exchange
  lives in :func:`nccl_all_to_all_dispatch`; it is the "library collective" baseline.

Ordering contract (identical to the device kernels): received rows are grouped by source
rank in ascending order and keep token order inside a group; combine accumulates in fp32 in
ascending order of the contributing rank (or of the top-k slot), then adds ``bias_0`` and
``bias_1`` and rounds to bf16 once.

Parity: deep_ep/utils/refs.py:10-243 of the reference (dispatch :10-123, combine :177-243).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .math import align


def rank_membership(topk_idx: torch.Tensor, num_ranks: int, num_experts: int) -> torch.Tensor:
    """bool ``[tokens, ranks]``: does the token select at least one expert of that rank."""
    per_rank = num_experts // num_ranks
    hit = torch.zeros((topk_idx.size(0), num_ranks + 1), dtype=torch.bool, device=topk_idx.device)
    rank_of = torch.where(topk_idx >= 0, topk_idx // per_rank, torch.full_like(topk_idx, num_ranks))
    hit.scatter_(1, rank_of, True)   # unused lanes land in the extra column
    return hit[:, :num_ranks].contiguous()


def dispatch_layout(topk_idx: torch.Tensor, num_ranks: int, num_experts: int):
    """(tokens per rank, pairs per expert, membership) — the legacy ``get_dispatch_layout`` result."""
    member = rank_membership(topk_idx, num_ranks, num_experts)
    per_expert = torch.zeros(num_experts, dtype=torch.int32, device=topk_idx.device)
    flat = topk_idx[topk_idx >= 0]
    per_expert.scatter_add_(0, flat, torch.ones_like(flat, dtype=torch.int32))
    return member.sum(dim=0).to(torch.int32), per_expert, member


def dispatch_local(xs: Sequence[torch.Tensor], topk_idxs: Sequence[torch.Tensor],
                   topk_weights: Sequence[Optional[torch.Tensor]], rank: int, num_experts: int,
                   num_max_tokens_per_rank: int, sfs: Optional[Sequence[torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """What ``rank`` receives when every rank ``s`` dispatches ``xs[s]`` with ``topk_idxs[s]``."""
    num_ranks = len(xs)
    per_rank = num_experts // num_ranks
    lo, hi = rank * per_rank, (rank + 1) * per_rank
    out_x, out_sf, out_idx, out_w, out_src, counts = [], [], [], [], [], []
    for s in range(num_ranks):
        idx = topk_idxs[s]
        mine = ((idx >= lo) & (idx < hi))
        rows = mine.any(dim=1).nonzero(as_tuple=True)[0]
        counts.append(rows.numel())
        out_x.append(xs[s][rows])
        if sfs is not None:
            out_sf.append(sfs[s][rows])
        sel = idx[rows]
        out_idx.append(torch.where(mine[rows], sel - lo, torch.full_like(sel, -1)))
        if topk_weights[s] is not None:
            out_w.append(topk_weights[s][rows])
        out_src.append(rows.to(torch.int32) + s * num_max_tokens_per_rank)
    res = {
        'recv_x': torch.cat(out_x, dim=0),
        'recv_topk_idx': torch.cat(out_idx, dim=0),
        'recv_src_token_idx': torch.cat(out_src, dim=0),
        'num_recv_tokens_per_rank': torch.tensor(counts, dtype=torch.int32),
    }
    if sfs is not None:
        res['recv_sf'] = torch.cat(out_sf, dim=0)
    if out_w:
        res['recv_topk_weights'] = torch.cat(out_w, dim=0)
    return res


def expand_local(recv: Dict[str, torch.Tensor], num_local_experts: int, expert_alignment: int = 1) -> Dict[str, torch.Tensor]:
    """Expert-major expansion of a non-expanded receive result.

    Expert ``e`` owns rows ``[start_e, start_e + count_e)`` with ``start_e`` the aligned
    running total; inside an expert rows keep the order of the non-expanded result.
    Returns the expanded rows as indices into the non-expanded ones (``row_of``), the starts,
    the counts, and per received token the expanded row of each top-k lane (-1 when unused).
    """
    idx = recv['recv_topk_idx']
    n, k = idx.shape
    starts, counts, row_of = [], [], []
    lane_rows = torch.full((n, k), -1, dtype=torch.int64)
    cursor = 0
    for e in range(num_local_experts):
        hit = (idx == e)
        tok, lane = hit.nonzero(as_tuple=True)
        starts.append(cursor)
        counts.append(tok.numel())
        lane_rows[tok, lane] = cursor + torch.arange(tok.numel())
        row_of.append(tok)
        cursor = align(cursor + tok.numel(), expert_alignment)
    return {'starts': torch.tensor(starts), 'counts': torch.tensor(counts), 'row_of': row_of,
            'lane_rows': lane_rows, 'num_rows': cursor}


def combine_local(ys: Sequence[torch.Tensor], srcs: Sequence[torch.Tensor], rank: int, num_tokens: int,
                  num_max_tokens_per_rank: int, bias: Sequence[torch.Tensor] = ()) -> torch.Tensor:
    """Sum, per original token of ``rank``, the rows that every rank ``r`` holds for it.

    ``ys[r]`` is rank r's bf16 ``[N_r, hidden]`` (one row per received token) and ``srcs[r]`` the
    matching global source indices ``src_rank * num_max_tokens_per_rank + token``.
    """
    hidden = ys[0].size(1)
    acc = torch.zeros((num_tokens, hidden), dtype=torch.float32, device=ys[0].device)
    for r in range(len(ys)):
        src = srcs[r].long()
        mine = (src // num_max_tokens_per_rank) == rank
        tok = src[mine] % num_max_tokens_per_rank
        acc.index_add_(0, tok, ys[r][mine].float())   # a token appears at most once per rank: order is fixed
    for b in bias:
        acc += b.float()
    return acc.to(torch.bfloat16)


# ---------------------------------------------------------------------------- collective forms
def _gather(obj, group):
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


def dispatch(x, topk_idx: torch.Tensor, topk_weights: Optional[torch.Tensor], num_max_tokens_per_rank: int,
             num_experts: int, group: Optional[dist.ProcessGroup] = None):
    """Collective oracle: returns ``(recv_x, recv_topk_idx, recv_topk_weights, recv_src_token_idx, counts)``.

    ``x`` may be a tensor or an ``(x_fp8, scales)`` tuple, in which case ``recv_x`` is a tuple too.
    """
    use_fp8 = isinstance(x, tuple)
    xs, sf = x if use_fp8 else (x, None)
    dev = xs.device
    payload = (xs.cpu() if not use_fp8 else xs.view(torch.uint8).cpu(), None if sf is None else sf.cpu(),
               topk_idx.cpu(), None if topk_weights is None else topk_weights.cpu())
    everyone = _gather(payload, group)
    rank = dist.get_rank(group)
    res = dispatch_local([e[0] for e in everyone], [e[2] for e in everyone], [e[3] for e in everyone], rank,
                         num_experts, num_max_tokens_per_rank, sfs=[e[1] for e in everyone] if use_fp8 else None)
    recv_x = res['recv_x'].to(dev)
    if use_fp8:
        recv_x = (recv_x.view(torch.float8_e4m3fn), res['recv_sf'].to(dev))
    return (recv_x, res['recv_topk_idx'].to(dev), res.get('recv_topk_weights', torch.empty(0)).to(dev),
            res['recv_src_token_idx'].to(dev), res['num_recv_tokens_per_rank'])


def combine(y: torch.Tensor, recv_src_token_idx: torch.Tensor, num_tokens: int, num_max_tokens_per_rank: int,
            bias: Sequence[torch.Tensor] = (), group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Collective oracle of the (unweighted) combine for the calling rank."""
    dev = y.device
    everyone = _gather((y.cpu(), recv_src_token_idx.cpu()), group)
    rank = dist.get_rank(group)
    out = combine_local([e[0] for e in everyone], [e[1] for e in everyone], rank, num_tokens, num_max_tokens_per_rank,
                        [b.cpu() for b in bias])
    return out.to(dev)


def nccl_all_to_all_dispatch(x: torch.Tensor, topk_idx: torch.Tensor, num_experts: int,
                             group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, List[int]]:
    """Baseline (not the product): the same token exchange with ``dist.all_to_all_single``.

    Needs a backend that implements all-to-all (NCCL). Returns the received rows and the split sizes.
    """
    world = dist.get_world_size(group)
    member = rank_membership(topk_idx, world, num_experts)
    order = [member[:, r].nonzero(as_tuple=True)[0] for r in range(world)]
    send = torch.cat([x[o] for o in order], dim=0)
    send_counts = torch.tensor([o.numel() for o in order], dtype=torch.int64, device=x.device)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    recv_list, send_list = recv_counts.tolist(), send_counts.tolist()
    recv = torch.empty((sum(recv_list), x.size(1)), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, send, recv_list, send_list, group=group)
    return recv, recv_list


def generate_pre_combine_data(src_token_global_idx: torch.Tensor, hidden: int, rank: int) -> torch.Tensor:
    """Deterministic bf16 rows keyed on (global source token, holder rank): the same value on every run."""
    base = src_token_global_idx.double().unsqueeze(1) * 0.37 + rank * 1.3
    cols = torch.arange(hidden, dtype=torch.float64, device=src_token_global_idx.device).unsqueeze(0) * 0.011
    return torch.sin(base + cols).to(torch.bfloat16)
