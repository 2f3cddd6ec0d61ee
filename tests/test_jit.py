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


def test_jit_rebuilds_when_an_included_header_changes(tmp_path):
    """The cache key covers the CONTENT of the library headers a source includes (directly or through other headers):
    the same source compiled against an edited copy of the header tree is a cache miss, against the unchanged copy a hit."""
    from deepep_b200 import jit
    import deepep_b200
    if shutil.which('nvcc') is None and not os.path.exists('/usr/local/cuda/bin/nvcc'):
        pytest.skip('no nvcc')
    C = deepep_b200._C
    root = tmp_path / 'csrc'
    shutil.copytree(jit.INCLUDE_ROOT, root, ignore=shutil.ignore_patterns('*.cu', '*.cpp', '*.o'))
    try:
        # make the include chain two levels deep: source -> kernels/jit/combine_reduce_jit.cuh -> kernels/jit/probe_extra.cuh
        header = root / 'kernels' / 'jit' / 'probe_extra.cuh'
        header.write_text('// a header that the specialised kernel pulls in indirectly\n')
        top = root / 'kernels' / 'jit' / 'combine_reduce_jit.cuh'
        top.write_text(top.read_text().replace('#include <cstdint>', '#include <cstdint>\n#include "probe_extra.cuh"', 1))
        jit.init(str(tmp_path / 'cache'), include_root=str(root))
        code = jit.combine_reduce_source(256, 4)
        before = C.jit_num_compilations()
        first = jit.build('combine_reduce', code)
        assert C.jit_num_compilations() == before + 1
        assert jit.build('combine_reduce', code) == first and C.jit_num_compilations() == before + 1
        header.write_text(header.read_text() + '\n// edited\n')
        second = jit.build('combine_reduce', code)
        assert second != first and C.jit_num_compilations() == before + 2
        # back to the old content: the old entry is found again
        header.write_text(header.read_text().replace('\n// edited\n', ''))
        assert jit.build('combine_reduce', code) == first and C.jit_num_compilations() == before + 2
    finally:
        jit.init(str(tmp_path / 'cache2'))       # later tests use the package's own headers again


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
