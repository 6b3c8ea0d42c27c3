"""CUDA-event timing with an L2 flush between calls (the reference's ``bench``, deep_gemm/testing/bench.py:7-33)."""
import torch


def bench(fn, num_warmups: int = 5, num_tests: int = 10, flush_l2_bytes: int = 256 * 1024 * 1024) -> float:
    """Average seconds per call of ``fn`` on the current stream."""
    flush = torch.empty(flush_l2_bytes, dtype=torch.int8, device='cuda')
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()
    total_ms = 0.0
    for _ in range(num_tests):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total_ms += start.elapsed_time(end)
    return total_ms / num_tests / 1e3


def bench_kineto(fn, kernel_names, num_tests: int = 30, suppress_kineto_output: bool = False, trace_path: str = None,
                 flush_l2: bool = True, with_multiple_kernels: bool = False, barrier=None):
    """Average device time in seconds of the kernels whose names contain ``kernel_names`` (a string, or a tuple of
    strings for a tuple of times) over ``num_tests`` calls of ``fn``, read from the CUDA activity records of
    torch.profiler. Same arguments as the reference's helper (deep_gemm/testing/bench.py:79-146); the kernels of this
    library are named ``dgb200_*``. ``flush_l2`` writes a buffer larger than L2 before every call; ``barrier`` (a
    callable) runs before every call behind a ~10 ms spin kernel so that ranks launch together."""
    import os
    names = (kernel_names,) if isinstance(kernel_names, str) else tuple(kernel_names)
    if int(os.environ.get('DG_USE_NVIDIA_TOOLS', 0)):  # a CUDA profiler is attached: two profilers cannot share the device
        return (1,) * len(names) if isinstance(kernel_names, tuple) else 1
    del suppress_kineto_output
    flush = torch.empty(512 << 20, dtype=torch.int8, device='cuda') if flush_l2 else None
    fn()
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(num_tests):
            if flush is not None:
                flush.zero_()
            if barrier is not None:
                torch.cuda._sleep(int(2e7))
                barrier()
            fn()
        torch.cuda.synchronize()
    if trace_path is not None:
        prof.export_chrome_trace(trace_path)
    averages = prof.key_averages()
    times = []
    for name in names:
        hits = [ev for ev in averages if name in ev.key]
        assert with_multiple_kernels or len(hits) <= 1, f'`{name}` matches {len(hits)} kernels: {[ev.key for ev in hits]}'
        total_us = sum(ev.device_time_total for ev in hits)
        count = sum(ev.count for ev in hits)
        times.append(total_us / count / 1e6 if count else 0.0)
    return tuple(times) if isinstance(kernel_names, tuple) else times[0]
