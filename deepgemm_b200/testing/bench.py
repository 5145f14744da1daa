"""Device timing helpers.

`bench_events` times with CUDA events on the current stream and flushes L2 between iterations.  `bench_kineto`
keeps the name and arguments of the reference's profiler-based timer (deep_gemm/testing/bench.py:79-146) so
that its test scripts run unchanged: kernel time summed by the torch profiler for the kernels whose names contain
the given substrings, a 256 MB memset between runs, an optional barrier + long spin before each run to line the
ranks of a multi-GPU job up.
"""
import os
from typing import Callable, Optional

import torch


def get_arch_major() -> int:
    return torch.cuda.get_device_capability()[0]


def bench(fn, num_warmups: int = 5, num_tests: int = 10, high_precision: bool = False):
    """Average device time (seconds) of `num_tests` back-to-back calls (deep_gemm/testing/bench.py:7-33)."""
    torch.cuda.synchronize()
    torch.empty(int(256e6), dtype=torch.int8, device="cuda").zero_()
    for _ in range(num_warmups):
        fn()
    if high_precision:
        torch.cuda._sleep(int(2e6))   # the host runs ahead of the device: launch latency stays out of the interval
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(num_tests):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / num_tests / 1e3


def test_filter(condition: Callable):
    """Decorator: run the test only where condition() holds (deep_gemm/testing/utils.py:11-23)."""
    import functools

    def decorator(func):
        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            if condition():
                return func(*args, **kwargs)
            print(f"{func.__name__}:\n > Filtered by {condition}\n")
        return wrapper
    return decorator


def bench_events(fn, num_warmups: int = 3, num_tests: int = 10, flush_l2: bool = True):
    """Median, min and all per-call device times (seconds) of fn()."""
    flush = torch.empty(int(256e6), dtype=torch.int8, device="cuda") if flush_l2 else None
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(num_tests):
        if flush is not None:
            flush.zero_()
        # Keep the GPU busy while the host enqueues fn(), so that host latency is not timed
        torch.cuda._sleep(int(2e5))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end) * 1e-3)
    times.sort()
    return times[len(times) // 2], times[0], times


def bench_kineto(fn, kernel_names, num_tests: int = 30, suppress_kineto_output: bool = False,
                 trace_path: Optional[str] = None, flush_l2: bool = True, with_multiple_kernels: bool = False,
                 barrier: Optional[Callable] = None):
    """Average device time (seconds) per launch of the kernels whose names contain `kernel_names` (a string, or a
    tuple of strings -> a tuple of times), measured by the torch profiler over `num_tests` calls of fn()."""
    names = (kernel_names,) if isinstance(kernel_names, str) else tuple(kernel_names)
    if int(os.environ.get("DG_USE_NVIDIA_TOOLS", 0)):    # under ncu / a sanitizer the profiler must stay off
        return (1,) * len(names) if isinstance(kernel_names, tuple) else 1
    fn()
    flush = torch.empty(int(256e6), dtype=torch.int8, device="cuda") if flush_l2 else None
    schedule = torch.profiler.schedule(wait=0, warmup=1, active=1, repeat=1)
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA], schedule=schedule,
                                acc_events=True) as prof:
        for _ in range(2):
            for _ in range(num_tests):
                if flush is not None:
                    flush.zero_()
                if barrier is not None:
                    torch.cuda._sleep(int(2e7))
                    barrier()
                fn()
            torch.cuda.synchronize()
            prof.step()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    totals = []
    for name in names:
        hits = [e for e in prof.key_averages() if name in e.key]
        assert with_multiple_kernels or len(hits) <= 1, f"several kernels match `{name}`: {[e.key for e in hits]}"
        time_us = sum(getattr(e, "self_device_time_total", 0.0) for e in hits)
        count = sum(e.count for e in hits)
        totals.append(time_us / count * 1e-6 if count else 0)
    return tuple(totals) if isinstance(kernel_names, tuple) else totals[0]
