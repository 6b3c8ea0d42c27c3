"""Small helpers of the reference's test drivers (deep_gemm/testing/utils.py:6-40, deep_gemm/testing/numeric.py:24-30)."""
import functools
import os
from typing import Callable

import torch


def get_arch_major() -> int:
    """Compute-capability major of the current device (10 on B200)."""
    return torch.cuda.get_device_capability()[0]


def test_filter(condition: Callable):
    """Decorator: the wrapped test runs only where ``condition()`` holds, otherwise it prints that it was skipped."""
    def decorator(func):
        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            if condition():
                return func(*args, **kwargs)
            print(f'{func.__name__}: skipped\n')
            return None
        return wrapper
    return decorator


def ignore_env(name: str, condition: Callable):
    """Decorator: while ``condition()`` holds the environment variable ``name`` is hidden from the wrapped call."""
    def decorator(func):
        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            saved = os.environ.pop(name, None) if condition() else None
            try:
                return func(*args, **kwargs)
            finally:
                if saved is not None:
                    os.environ[name] = saved
        return wrapper
    return decorator


def assert_bitwise_equal(x: torch.Tensor, y: torch.Tensor, label: str = '') -> None:
    """Same shape, dtype and bytes (NaN payloads included)."""
    assert x.shape == y.shape and x.dtype == y.dtype, f'{label}: shape or dtype differs'
    same = torch.equal(x.contiguous().view(torch.uint8), y.contiguous().view(torch.uint8))
    assert same, f'{label}: tensors differ bitwise'
