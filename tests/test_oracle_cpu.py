"""CPU-only checks: the pure-torch oracle over gloo with world_size 2 (128 tokens per rank, hidden
256, 16 experts, top-2: combine(dispatch(x)) == sum_k w_k * x), the gate generators, the FP8
helpers, the layout reference and the analytical SM model. No GPU, no native kernel launch."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _gloo_worker(rank: int, world: int, port: int):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    from deepep_b200.utils import gate, refs
    T, H, E, K, T_max = 128, 256, 16, 2, 128
    g = torch.Generator().manual_seed(7 + rank)
    x = torch.randn((T, H), generator=g)
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K)
    assert torch.allclose(w.sum(dim=1), torch.ones(T), atol=1e-6)
    recv_x, recv_idx, recv_w, recv_src, counts = refs.dispatch(x, idx, w, T_max, E)
    assert recv_x.size(0) == int(counts.sum())
    # every received row is the source row it claims to be, and carries a local expert
    src_rank = recv_src // T_max
    assert torch.equal(src_rank, torch.repeat_interleave(torch.arange(world), counts.long()).int())
    assert bool(((recv_idx >= 0).any(dim=1)).all()) and int(recv_idx.max()) < E // world
    # expert compute = identity weighted by the local experts' weights; combine sums the partial results
    local_w = torch.where(recv_idx >= 0, recv_w, torch.zeros_like(recv_w)).sum(dim=1, keepdim=True)
    y = (recv_x * local_w).to(torch.bfloat16)
    out = refs.combine(y, recv_src, T, T_max)
    ref = x   # sum_k w_k * x with sum_k w_k == 1
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_world2_dispatch_combine_roundtrip():
    mp.spawn(_gloo_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_fp8_cast_roundtrip_and_pow2_scales():
    from deepep_b200.utils.math import calc_diff, per_token_cast_back, per_token_cast_to_fp8
    x = torch.randn((33, 384), generator=torch.Generator().manual_seed(0)).bfloat16()
    q, s = per_token_cast_to_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (33, 3)
    assert calc_diff(per_token_cast_back(q, s).float(), x.float()) < 1e-3
    q2, s2 = per_token_cast_to_fp8(x, round_scale=True)
    assert torch.equal(torch.log2(s2), torch.log2(s2).round())     # powers of two
    assert bool((s2 >= s * (1 - 1e-6)).all())                      # rounded up
    assert calc_diff(per_token_cast_back(q2, s2).float(), x.float()) < 2e-3


def test_layout_reference_and_membership():
    from deepep_b200.utils import refs
    idx = torch.tensor([[0, 5, -1], [15, 14, 2], [-1, -1, -1]])
    per_rank, per_expert, member = refs.dispatch_layout(idx, 4, 16)
    assert per_rank.tolist() == [2, 1, 0, 1]
    assert per_expert.sum().item() == 5 and per_expert[15].item() == 1
    assert member.tolist() == [[True, True, False, False], [True, False, False, True], [False] * 4]


def test_gate_generators():
    from deepep_b200.utils import gate
    g = torch.Generator().manual_seed(3)
    scores = gate.get_unbalanced_scores(4096, 64, 8, 4, 2.5, generator=g)
    ratio = gate.measure_unbalanced_ratio(torch.topk(scores, 4).indices, 64, 8)
    assert 2.2 < ratio < 2.8
    idx, w = gate.topk_from_scores(gate.get_zipf_scores(2048, 64, 1.2, generator=g), 4)
    counts = torch.bincount(idx.flatten(), minlength=64)
    assert counts[0] > 4 * counts[32]       # Zipf skew
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(256, 64, generator=g), 8, num_groups=8, num_topk_groups=3)
    assert int((torch.div(idx, 8, rounding_mode='floor')).unique(dim=1).size(1)) <= 8
    for row in idx.tolist():
        assert len({e // 8 for e in row}) <= 3   # group-limited routing


def test_sm_model_matches_published_row():
    """EP8 / 256 experts / top-8 with 810 GB/s of NVLink gives 24 SMs (the reference's "min #SM" row)."""
    from deepep_b200.buffers.elastic import ElasticBuffer

    class FakeBuffer:
        num_ranks = 8
        prefer_overlap_with_compute = True

    f = ElasticBuffer.get_theoretical_num_sms.__wrapped__
    assert f(FakeBuffer(), 256, 8, nvlink_gbs=810.0) == 24
    FakeBuffer.prefer_overlap_with_compute = False
    assert f(FakeBuffer(), 256, 8, nvlink_gbs=810.0) == 64
    FakeBuffer.num_ranks = 1
    assert f(FakeBuffer(), 256, 8) >= 100


def test_event_overlap_hook_runs_once():
    from deepep_b200.utils.event import EventOverlap
    calls = []
    ev = EventOverlap(None)
    ev.register_hook_after_wait(lambda: calls.append(1))
    with ev:
        pass
    ev.current_stream_wait()
    assert calls == [1]


def test_nvlink_status_parser():
    from deepep_b200.utils.envs import parse_nvlink_status
    text = 'GPU 0: NVIDIA B200\n\t Link 0: 53.125 GB/s\n\t Link 1: 53.125 GB/s\n'
    assert parse_nvlink_status(text) == (2, 53.125)
    assert parse_nvlink_status('nothing') == (0, 0.0)


def test_logfmt_roundtrip_oracle():
    """The torch restatement of the LogFMT-10 wire format: which groups are encoded, exact values, error bound."""
    from deepep_b200.utils.math import logfmt_roundtrip
    torch.manual_seed(3)
    x = (torch.randn(8, 512) * 0.1).bfloat16()
    x[:, 128:256] *= 40          # amax >= 1: stays bf16
    x[:, 256:384] = 0            # all zero: stays as is
    x[:, 384:512] = -0.25        # single magnitude: stays as is
    x[0, 5] = 0
    y = logfmt_roundtrip(x)
    assert torch.equal(y[:, 128:], x[:, 128:].float())
    assert y[0, 5] == 0
    a, b = y[:, :128], x[:, :128].float()
    assert not torch.equal(a, b)
    assert torch.equal(torch.sign(a), torch.sign(b))
    nz = b != 0
    assert ((a - b).abs()[nz] / b.abs()[nz]).max() < 0.025       # half a grid step of at most 32 / 510 octaves
    # the extreme values of a group are grid points
    amax = b.abs().amax(dim=1)
    assert torch.allclose(a.abs().amax(dim=1), amax, rtol=1e-5)


def test_numa_helpers(tmp_path):
    """CPU-list parsing and the sysfs lookups of utils/numa.py against a fake /sys tree."""
    from deepep_b200.utils import numa
    assert numa.parse_cpu_list('0-3,8,10-11\n') == [0, 1, 2, 3, 8, 10, 11]
    assert numa.parse_cpu_list('') == []
    dev = tmp_path / 'bus/pci/devices/0000:1b:00.0'
    dev.mkdir(parents=True)
    (dev / 'numa_node').write_text('1\n')
    node = tmp_path / 'devices/system/node/node1'
    node.mkdir(parents=True)
    (node / 'cpulist').write_text('32-63\n')
    assert numa.pci_numa_node('0000:1B:00.0', str(tmp_path)) == 1
    assert numa.pci_numa_node('00000000:1b:00.0', str(tmp_path)) == 1      # NVML spelling
    assert numa.pci_numa_node('0000:2c:00.0', str(tmp_path)) is None
    (dev / 'numa_node').write_text('-1\n')
    assert numa.pci_numa_node('0000:1b:00.0', str(tmp_path)) is None
    assert numa.node_cpus(1, str(tmp_path)) == list(range(32, 64))
    assert numa.node_cpus(7, str(tmp_path)) == []


def test_ops_references_cpu():
    """The fp32 reference functions of deepep_b200.ops are plain torch and run anywhere."""
    from deepep_b200 import ops
    torch.manual_seed(0)
    a, b = torch.randn(5, 256), torch.randn(128, 256)
    assert torch.allclose(ops.ref_gemm(a, b), a @ b.t())
    sfa, sfb = torch.full((5, 2), 2.0), torch.full((1, 2), 0.5)
    assert torch.allclose(ops.ref_gemm(a, b, sfa, sfb), a @ b.t(), rtol=1e-5, atol=1e-4)
    ends = torch.tensor([3, 5], dtype=torch.int32)
    w = torch.randn(2, 4, 256)
    out = ops.ref_grouped_gemm(a, w, ends, 1)
    assert torch.allclose(out[:3], a[:3] @ w[0].t()) and torch.allclose(out[3:], a[3:] @ w[1].t())
    idx, wt = ops.ref_router_topk(torch.randn(7, 16), 3)
    assert idx.shape == (7, 3) and torch.allclose(wt.sum(1), torch.ones(7))
    x = torch.randn(4, 8)
    assert torch.allclose(ops.ref_swiglu(x), torch.nn.functional.silu(x[:, :4]) * x[:, 4:])


def test_weight_quantisation_pow2_scales_cpu():
    """128x128 weight quantisation: with ``pow2`` every scale is an exact power of two (what a UE8M0 scale factor of the
    block-scaled tensor-core instruction can hold), never smaller than the exact scale, and the dequantised weights
    stay within e4m3 rounding of the originals."""
    from deepep_b200.models.moe import quantize_weight_128x128
    g = torch.Generator().manual_seed(3)
    w = torch.randn((2, 256, 384), generator=g) * torch.exp2(torch.randint(-5, 6, (2, 2, 1, 3, 1), generator=g).float()).expand(2, 2, 128, 3, 128).reshape(2, 256, 384)
    q, sf = quantize_weight_128x128(w)
    q2, sf2 = quantize_weight_128x128(w, pow2=True)
    assert sf.shape == sf2.shape == (2, 2, 3)
    assert bool((torch.frexp(sf2)[0] == 0.5).all())
    assert bool((sf2 >= sf).all()) and bool((sf2 < 2 * sf).all())
    for qq, ss in ((q, sf), (q2, sf2)):
        deq = (qq.float().view(2, 2, 128, 3, 128) * ss[:, :, None, :, None]).view(2, 256, 384)
        assert ((deq - w).norm() / w.norm()).item() < 0.04


def test_bench_reference_arm_reports_unavailable():
    """`bench.py --impl reference` must answer with one JSON line and exit 0 where the reference cannot be installed."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if os.path.isdir(os.path.join(root, 'baseline', '_ref', 'deep_ep')):
        pytest.skip('the reference is installed here')
    res = subprocess.run([sys.executable, os.path.join(root, 'bench.py'), '--impl', 'reference'], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line['impl'] == 'reference' and isinstance(line.get('unavailable'), str) and line['unavailable']
