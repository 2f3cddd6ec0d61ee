"""Shared pytest configuration: the ``gpu`` marker and helpers to build routed test inputs."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')
    config.addinivalue_line('markers', 'multigpu: needs at least two CUDA devices')


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _poison_free_gpu_memory(request):
    """Before every GPU test the caching allocator's free blocks are filled with NaN bit patterns (0xFF bytes), so a
    kernel that reads a row nobody wrote shows up in the comparison instead of happening to read zeros."""
    if 'gpu' in request.keywords and torch.cuda.is_available():
        junk = torch.full((192 << 20,), 0xFF, dtype=torch.uint8, device='cuda')
        del junk
    yield


def make_routed_inputs(num_ranks, num_tokens, hidden, num_experts, num_topk, seed=0, device='cpu', masked_ratio=0.0,
                       vary_tokens=True, dtype=torch.bfloat16):
    """Per-rank (x, topk_idx, topk_weights) lists with seeded N(0,1) tokens and softmax top-k routing."""
    from deepep_b200.utils import gate
    g = torch.Generator().manual_seed(seed)
    xs, idxs, ws = [], [], []
    for r in range(num_ranks):
        t = max(0, num_tokens - (r * 3 if vary_tokens else 0))
        x = torch.randn((t, hidden), generator=g).to(dtype)
        idx, w = gate.topk_from_scores(gate.get_balanced_scores(t, num_experts, generator=g), num_topk,
                                       masked_ratio=masked_ratio, generator=g)
        xs.append(x.to(device))
        idxs.append(idx.to(device))
        ws.append(w.to(device))
    return xs, idxs, ws
