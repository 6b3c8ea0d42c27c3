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
