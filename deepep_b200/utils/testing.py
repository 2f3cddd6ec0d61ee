"""Timing helpers: CUDA-event benchmarks with an L2 flush, and per-kernel device times from the
PyTorch profiler with the pre-synchronisation the reference uses for its published numbers.

Parity: deep_ep/utils/testing.py:12-219 of the reference (``bench``, ``bench_kineto``).
"""
from __future__ import annotations

import os
import sys
from contextlib import contextmanager
from typing import Callable, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

_L2_FLUSH_BYTES = 256 << 20
_flush_buffer = {}


def flush_l2_cache(enabled: bool = True) -> None:
    """Overwrites a 256 MB buffer (larger than the 126 MB L2 of a B200)."""
    if not enabled:
        return
    dev = torch.cuda.current_device()
    if dev not in _flush_buffer:
        _flush_buffer[dev] = torch.empty(_L2_FLUSH_BYTES // 4, dtype=torch.int32, device='cuda')
    _flush_buffer[dev].zero_()


def bench(fn: Callable, num_warmups: int = 50, num_tests: int = 50, post_fn: Optional[Callable] = None,
          flush_l2: bool = True) -> Tuple[float, float, float]:
    """(mean, min, max) seconds of ``fn`` over ``num_tests`` runs, each timed with its own CUDA event pair."""
    torch.cuda.synchronize()
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(num_tests)]
    for i in range(num_tests):
        flush_l2_cache(flush_l2)
        starts[i].record()
        fn()
        ends[i].record()
        if post_fn is not None:
            post_fn()
    torch.cuda.synchronize()
    times = [s.elapsed_time(e) / 1e3 for s, e in zip(starts, ends)][1:] or [starts[0].elapsed_time(ends[0]) / 1e3]
    return sum(times) / len(times), min(times), max(times)


@contextmanager
def suppress_stdout_stderr():
    with open(os.devnull, 'w') as devnull:
        old_out, old_err = sys.stdout, sys.stderr
        sys.stdout, sys.stderr = devnull, devnull
        try:
            yield
        finally:
            sys.stdout, sys.stderr = old_out, old_err


def presync(group: Optional[dist.ProcessGroup] = None, sleep_cycles: int = int(4e6)) -> None:
    """Queues a long GPU sleep and a tiny all-reduce: the host runs ahead and enqueues the kernels under
    test, the all-reduce then releases all ranks at the same moment, so launch skew is not timed."""
    torch.cuda._sleep(sleep_cycles)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(torch.ones(1, device='cuda'), group=group)


def bench_kineto(fn: Callable, kernel_names: Union[str, Sequence[str]], num_tests: int = 30, suppress_kineto_output: bool = True,
                 trace_path: Optional[str] = None, flush_l2: bool = True, barrier_comm_profiling: bool = False,
                 group: Optional[dist.ProcessGroup] = None):
    """Mean device duration (seconds) of the kernels whose names contain ``kernel_names``.

    With ``EP_USE_NVIDIA_TOOLS=1`` (running under ncu / compute-sanitizer) the profiler is skipped, ``fn`` runs
    once and 1.0 is returned for every name.
    """
    single = isinstance(kernel_names, str)
    names = (kernel_names,) if single else tuple(kernel_names)
    if int(os.environ.get('EP_USE_NVIDIA_TOOLS', '0')):
        fn()
        torch.cuda.synchronize()
        return 1.0 if single else (1.0,) * len(names)
    fn()
    torch.cuda.synchronize()
    use_barrier = barrier_comm_profiling and not int(os.environ.get('EP_DISABLE_BARRIER_PROFILING', '0'))
    ctx = suppress_stdout_stderr if suppress_kineto_output else (lambda: contextmanager(lambda: (yield))())
    with ctx():
        schedule = torch.profiler.schedule(wait=0, warmup=1, active=1, repeat=1)
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA], schedule=schedule) as prof:
            for _ in range(2):
                for _ in range(num_tests):
                    flush_l2_cache(flush_l2)
                    if use_barrier:
                        presync(group)
                    fn()
                torch.cuda.synchronize()
                prof.step()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    totals = {n: [0.0, 0] for n in names}
    for evt in prof.key_averages():
        for n in names:
            if n in evt.key:
                dev_time = getattr(evt, 'device_time_total', None)
                if dev_time is None:
                    dev_time = getattr(evt, 'cuda_time_total', 0.0)
                totals[n][0] += dev_time / 1e6
                totals[n][1] += evt.count
    out = tuple(totals[n][0] / totals[n][1] if totals[n][1] else 0.0 for n in names)
    return out[0] if single else out
