"""Run-time compiler: the disk cache (CPU, nvcc cross-compiles without a GPU), header-content
invalidation, and on a GPU loading + launching a specialised kernel."""
import os
import shutil

import pytest
import torch


def test_jit_cache_and_header_invalidation(tmp_path):
    from deepep_b200 import jit
    import deepep_b200
    if shutil.which('nvcc') is None and not os.path.exists('/usr/local/cuda/bin/nvcc'):
        pytest.skip('no nvcc')
    jit.init(str(tmp_path / 'cache'))
    C = deepep_b200._C
    code = jit.combine_reduce_source(256, 4)
    before = C.jit_num_compilations()
    cubin = jit.build('combine_reduce', code)
    assert os.path.exists(cubin) and C.jit_num_compilations() == before + 1
    assert jit.build('combine_reduce', code) == cubin and C.jit_num_compilations() == before + 1      # cache hit
    other = jit.build('combine_reduce', jit.combine_reduce_source(512, 4))
    assert other != cubin and C.jit_num_compilations() == before + 2                                  # new constants, new entry
    assert 'sm_100a' in C.jit_flags()
    with pytest.raises(Exception):
        jit.build('broken', 'extern "C" __global__ void ep_jit_entry() { this does not compile }')


@pytest.mark.gpu
def test_jit_specialised_combine_reduce(tmp_path):
    from deepep_b200 import jit
    jit.init(str(tmp_path / 'cache'))
    hidden, lanes, T, T_max = 512, 4, 100, 128
    g = torch.Generator(device='cuda').manual_seed(0)
    region = torch.randn((lanes, T_max, hidden), device='cuda', generator=g).bfloat16()
    mask = torch.randint(1, 1 << lanes, (T,), device='cuda', generator=g, dtype=torch.int32)
    out = torch.zeros((T, hidden), device='cuda', dtype=torch.bfloat16)
    cubin = jit.build('combine_reduce', jit.combine_reduce_source(hidden, lanes))
    params = jit.pack('PPPii', region.data_ptr(), mask.data_ptr(), out.data_ptr(), T, T_max)
    jit.launch(cubin, (32,), (256,), params)
    torch.cuda.synchronize()
    bits = ((mask.unsqueeze(1) >> torch.arange(lanes, device='cuda')) & 1).bool()       # [T, lanes]
    ref = (region[:, :T].float() * bits.t().unsqueeze(-1)).sum(dim=0).bfloat16()
    assert torch.equal(out, ref)
