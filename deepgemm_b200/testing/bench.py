"""Device timing with CUDA events and an L2 flush between iterations.

The reference times kernels through the torch profiler with a 256 MB memset between runs
(deep_gemm/testing/bench.py:79-146); this does the same with CUDA events on the current stream.
"""
import torch


def get_arch_major() -> int:
    return torch.cuda.get_device_capability()[0]


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
