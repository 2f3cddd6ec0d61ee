"""The allocation-free dispatch entry point, called through its exported C symbol.

Some embedders of this library may not take device memory when they need a dispatch (their
memory pool belongs to a serving runtime, or an allocation would stall the other streams of the
process). ``deepep_b200_dispatch_local_noalloc`` serves them from a fixed device array inside the
library. This test calls it with ctypes exactly as such an embedder would (raw device pointers,
no Python wrapper) and requires bit-identical results to ``ElasticBuffer.dispatch`` on a one-rank
group, on two calls in a row that share the scratch array. It sits in a file of its own that is
collected last, so a failure here cannot hide the result of any other test.
"""
import ctypes

import pytest
import torch

gpu = pytest.mark.gpu


def _lib():
    import deepep_b200
    lib = ctypes.CDLL(deepep_b200._C.__file__)
    fn = lib.deepep_b200_dispatch_local_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.deepep_b200_noalloc_status.restype = ctypes.c_int
    lib.deepep_b200_noalloc_status.argtypes = [ctypes.POINTER(ctypes.c_ulonglong)]
    lib.deepep_b200_noalloc_scratch_bytes.restype = ctypes.c_size_t
    return lib


def _inputs(seed, T, H, E, K):
    from deepep_b200.utils import gate
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, H), generator=g).bfloat16().cuda()
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K, masked_ratio=0.15, generator=g)
    return x, idx.cuda(), w.cuda()


def _call(lib, x, idx, w, E, do_expand, alignment, rows):
    T, H = x.shape
    K = idx.size(1)
    recv_x = torch.zeros((rows, H), dtype=torch.bfloat16, device='cuda')
    recv_idx = torch.full((T, K), -7, dtype=torch.int64, device='cuda')
    recv_w = torch.zeros((rows if do_expand else T, K) if not do_expand else (rows,), dtype=torch.float32, device='cuda')
    meta = torch.full((T, K + 2), -7, dtype=torch.int32, device='cuda')
    psum = torch.zeros(E + 1, dtype=torch.int32, device='cuda')
    n = torch.zeros(1, dtype=torch.int32, device='cuda')
    rc = lib.deepep_b200_dispatch_local_noalloc(
        x.data_ptr(), x.stride(0) * 2, H * 2, idx.data_ptr(), w.data_ptr(), T, K, E, int(do_expand), alignment, 6,
        recv_x.data_ptr(), rows, recv_idx.data_ptr(), recv_w.data_ptr(), meta.data_ptr(), psum.data_ptr(), n.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f'entry point returned {rc}'
    torch.cuda.synchronize()
    record = ctypes.c_ulonglong(1)
    assert lib.deepep_b200_noalloc_status(ctypes.byref(record)) == 0 and record.value == 0
    return recv_x, recv_idx, recv_w, meta, psum, int(n.item())


@gpu
@pytest.mark.parametrize('do_expand,alignment', [(False, 1), (True, 8)])
def test_noalloc_matches_regular_dispatch(do_expand, alignment):
    import deepep_b200
    from deepep_b200.parallel.local_cluster import SingleProcessGroup
    lib = _lib()
    assert 0 < lib.deepep_b200_noalloc_scratch_bytes() < 32 << 20
    T, H, E, K = 300, 1024, 32, 4
    buf = deepep_b200.ElasticBuffer(SingleProcessGroup(), num_max_tokens_per_rank=T, hidden=H, num_topk=K,
                                    num_gpu_timeout_secs=10)
    for call in range(2):   # two calls in a row share the scratch array
        x, idx, w = _inputs(40 + call, T - 17 * call, H, E, K)
        ref_x, ref_idx, ref_w, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=6,
                                                        do_expand=do_expand, expert_alignment=alignment)
        torch.cuda.synchronize()
        buf.check_status()
        rows = x.size(0) * K + E * (alignment - 1) if do_expand else x.size(0)
        got_x, got_idx, got_w, meta, psum, n = _call(lib, x, idx, w, E, do_expand, alignment, rows)
        assert n == handle.num_recv_tokens
        assert torch.equal(meta[:n], handle.recv_src_metadata)
        assert torch.equal(psum[:E], handle.psum_num_recv_tokens_per_expert)
        if do_expand:
            total = handle.num_expanded_tokens
            assert int(psum[E].item()) == total
            # compare the rows that hold tokens (alignment gaps are not written by either path)
            for e in range(E):
                end = int(psum[e].item())
                begin = 0 if e == 0 else -(-int(psum[e - 1].item()) // alignment) * alignment
                assert torch.equal(got_x[begin:end], ref_x[begin:end])
                assert torch.equal(got_w[begin:end], ref_w[begin:end])
        else:
            assert torch.equal(got_x[:n], ref_x)
            assert torch.equal(got_idx[:n], ref_idx)
            assert torch.equal(got_w[:n], ref_w)
    buf.destroy()


@gpu
def test_noalloc_rejects_sizes_beyond_the_scratch():
    lib = _lib()
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device='cuda')
    idx = torch.zeros((4, 2), dtype=torch.int64, device='cuda')
    out = torch.zeros((4, 64), dtype=torch.bfloat16, device='cuda')
    meta = torch.zeros((4, 4), dtype=torch.int32, device='cuda')
    psum = torch.zeros(9, dtype=torch.int32, device='cuda')
    n = torch.zeros(1, dtype=torch.int32, device='cuda')
    args = lambda T, rb, K, E: (x.data_ptr(), 128, rb, idx.data_ptr(), None, T, K, E, 0, 1, 4, out.data_ptr(), 4, None, None,
                                meta.data_ptr(), psum.data_ptr(), n.data_ptr(), None)
    assert lib.deepep_b200_dispatch_local_noalloc(*args(1 << 20, 128, 2, 8)) == 1    # too many tokens
    assert lib.deepep_b200_dispatch_local_noalloc(*args(4, 1 << 20, 2, 8)) == 2      # row too wide
    assert lib.deepep_b200_dispatch_local_noalloc(*args(4, 120, 2, 8)) == 2          # not a multiple of 16
    assert lib.deepep_b200_dispatch_local_noalloc(*args(4, 128, 64, 8)) == 3         # top-k beyond the maximum
    assert lib.deepep_b200_dispatch_local_noalloc(*args(4, 128, 2, 4096)) == 4       # too many experts


def test_noalloc_rejects_an_output_that_is_too_small():
    """An embedder that sizes recv_x too small gets an error code, not an out-of-bounds write. The check runs before
    anything touches the device, so this test needs no GPU: the pointers are never dereferenced."""
    lib = _lib()
    fake = 1 << 20            # any non-null, 16-byte aligned address
    T, K, E = 64, 4, 8

    def call(do_expand, alignment, rows):
        return lib.deepep_b200_dispatch_local_noalloc(fake, 256, 256, fake, None, T, K, E, do_expand, alignment, 4, fake, rows,
                                                      None, None, fake, fake, fake, None)

    assert call(0, 1, T - 1) == 5                                  # non-expanded output needs one row per token
    assert call(1, 1, T * K - 1) == 5                              # expanded: one row per token and expert ...
    assert call(1, 16, T * K + E * 15 - 1) == 5                    # ... plus the alignment slack of every expert
    assert call(0, 0, T) == 5                                      # an alignment of zero


@gpu
def test_noalloc_reset_clears_the_status():
    """deepep_b200_noalloc_reset() is the way back after a wait that ran out: here it is simply called on a healthy
    device and a dispatch after it must still be correct."""
    lib = _lib()
    lib.deepep_b200_noalloc_reset.restype = ctypes.c_int
    x, idx, w = _inputs(7, 64, 256, 8, 2)
    _call(lib, x, idx, w, 8, False, 1, 64)
    assert lib.deepep_b200_noalloc_reset() == 0
    record = ctypes.c_ulonglong(1)
    assert lib.deepep_b200_noalloc_status(ctypes.byref(record)) == 0 and record.value == 0
    got_x, got_idx, _, _, _, n = _call(lib, x, idx, w, 8, False, 1, 64)
    sel = (idx >= 0).any(dim=1)
    assert n == int(sel.sum()) and torch.equal(got_x[:n], x[sel])
