"""Quantisers and dequantisers with the reference's names and return conventions (deep_gemm/utils/math.py).

The quantisers run as CUDA kernels of libdgb200.so (fused amax / UE8M0 scale / cast); inputs must be CUDA BF16
tensors. The dequantisers and the packing helpers are plain tensor expressions: the reference uses them only to
build test inputs and expected values, and they work on any device.
"""
import ctypes
from typing import Tuple

import torch

from .. import _lib


def ceil_div(x: int, y: int) -> int:
    return (x + y - 1) // y


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= |x| (reference: deep_gemm/utils/math.py:13-16)."""
    bits = x.abs().float().contiguous().view(torch.int32)
    exponent = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (exponent.clamp(1, 254) << 23).view(torch.float32)


def pack_ue8m0_to_int(x: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales [..., 4n] -> int32 [..., n] (reference: deep_gemm/utils/math.py:19-23)."""
    assert x.dtype == torch.float32 and x.size(-1) % 4 == 0
    bits = x.contiguous().view(torch.int32)
    assert bool((bits >= 0).all()) and bool(((bits & 0x7FFFFF) == 0).all())
    return (bits >> 23).to(torch.uint8).view(torch.int32)


def unpack_ue8m0_from_int(packed_sf: torch.Tensor) -> torch.Tensor:
    return (packed_sf.contiguous().view(torch.uint8).to(torch.int32) << 23).view(torch.float32)


def _cast(x: torch.Tensor, gran_k: int, fp4: bool, want_f32: bool, packed_layout: str):
    """Runs the fused cast kernel. ``packed_layout``: None, 'token' (int32 [M, Kp] contiguous) or 'mn'
    (int32 [M, Kp] with strides (1, align(M, 4)), the layout the GEMMs consume)."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2):
        raise RuntimeError('expected a 2-D CUDA bfloat16 tensor')
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    if k % 16 != 0:
        raise RuntimeError(f'k ({k}) must be a multiple of 16')
    q = torch.empty((m, k // 2 if fp4 else k), dtype=torch.int8 if fp4 else torch.float8_e4m3fn, device=x.device)
    num_sf = ceil_div(k, gran_k)
    sf = torch.empty((m, num_sf), dtype=torch.float32, device=x.device) if want_f32 else None
    packed = None
    k_stride = row_stride = 0
    packed_k = ceil_div(num_sf, 4)
    if packed_layout == 'token':
        packed = torch.empty((m, packed_k), dtype=torch.int32, device=x.device)
        k_stride, row_stride = 1, packed_k
    elif packed_layout == 'mn':
        packed = torch.empty((packed_k, align(m, 4)), dtype=torch.int32, device=x.device).t()[:m]
        k_stride, row_stride = align(m, 4), 1
    fn = _lib.lib().dgb200_per_token_cast_to_fp4 if fp4 else _lib.lib().dgb200_per_token_cast_to_fp8
    with torch.cuda.device(x.device):
        _lib.check(fn(_ptr(x), x.stride(0), m, k, gran_k, _ptr(q), q.stride(0), _ptr(sf), _ptr(packed), k_stride, row_stride,
                      _lib.current_stream_ptr()))
    return q, sf, packed


def per_token_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128,
                          use_packed_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 [M, K], scales): fp32 [M, K / gran_k] or, packed, int32 [M, ceil(K / gran_k / 4)] (token-major).
    Reference: per_token_cast_to_fp8, deep_gemm/utils/math.py:26-49. Only power-of-two (UE8M0) scales exist on
    this path, so ``use_ue8m0`` must be True."""
    if not use_ue8m0:
        raise RuntimeError('only UE8M0 (power-of-two) scales are supported on sm_100a')
    q, sf, packed = _cast(x, gran_k, False, not use_packed_ue8m0, 'token' if use_packed_ue8m0 else None)
    return q, (packed if use_packed_ue8m0 else sf)


def per_channel_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """x bfloat16 [K, MN] -> (e4m3 [K, MN], fp32 [K / gran_k, MN]): one scale per ``gran_k`` K rows and channel, the
    operand format of the K-grouped GEMM. Reference: per_channel_cast_to_fp8, deep_gemm/utils/math.py:52-59."""
    if not use_ue8m0:
        raise RuntimeError('only UE8M0 (power-of-two) scales are supported on sm_100a')
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()):
        raise RuntimeError('x must be a contiguous CUDA bfloat16 [K, MN] tensor')
    k, mn = x.shape
    if k % gran_k != 0:
        raise RuntimeError(f'K ({k}) must be a multiple of gran_k ({gran_k})')
    q = torch.empty((k, mn), dtype=torch.float8_e4m3fn, device=x.device)
    sf = torch.empty((k // gran_k, mn), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().dgb200_per_channel_cast_to_fp8(_ptr(x), k, mn, gran_k, _ptr(q), _ptr(sf), _lib.current_stream_ptr()))
    return q, sf


def per_token_cast_to_fp4(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128,
                          use_packed_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """(int8 [M, K / 2] packed E2M1, scales). Reference: per_token_cast_to_fp4, deep_gemm/utils/math.py:96-122."""
    if not use_ue8m0:
        raise RuntimeError('only UE8M0 (power-of-two) scales are supported on sm_100a')
    q, sf, packed = _cast(x, gran_k, True, not use_packed_ue8m0, 'token' if use_packed_ue8m0 else None)
    return q, (packed if use_packed_ue8m0 else sf)


def per_token_cast_to_fp8_mn_major(x: torch.Tensor, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fused variant with no reference counterpart: scales come out already packed in the MN-major, TMA-aligned
    layout of ``transform_sf_into_required_layout`` (one kernel instead of cast + pack)."""
    q, _, packed = _cast(x, gran_k, False, False, 'mn')
    return q, packed


def per_token_cast_to_fp4_mn_major(x: torch.Tensor, gran_k: int = 32) -> Tuple[torch.Tensor, torch.Tensor]:
    q, _, packed = _cast(x, gran_k, True, False, 'mn')
    return q, packed


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def cast_back_from_fp4(packed: torch.Tensor, sf: torch.Tensor, gran_k: int = 128,
                       use_packed_ue8m0: bool = False) -> torch.Tensor:
    """Reference: cast_back_from_fp4, deep_gemm/utils/math.py:152-164."""
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    raw = packed.contiguous().view(torch.uint8)
    codes = torch.stack([raw & 0xF, raw >> 4], dim=-1).reshape(raw.shape[0], -1).to(torch.int64)
    table = torch.tensor(_E2M1 + (0.0,) + tuple(-v for v in _E2M1[1:]), dtype=torch.float32, device=packed.device)
    values = table[codes]
    block = torch.arange(values.shape[1], device=packed.device) // gran_k
    return values * sf[:, block]


def cast_back_from_fp8(x_fp8: torch.Tensor, sf: torch.Tensor, gran_k: int = 128,
                       use_packed_ue8m0: bool = False) -> torch.Tensor:
    """Reference: cast_back_from_fp8, deep_gemm/utils/math.py:167-173."""
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    block = torch.arange(x_fp8.shape[1], device=x_fp8.device) // gran_k
    return x_fp8.float() * sf[:, block]


def per_token_cast_to_fp8_into(x: torch.Tensor, q_out: torch.Tensor, sf_packed_out: torch.Tensor, gran_k: int = 32) -> None:
    """Quantises ``x`` straight into caller-owned views (e.g. ``SymmBuffer.x`` / ``SymmBuffer.x_sf``): e4m3
    [M, K] and token-major packed UE8M0 int32 [M, ceil(K / gran_k / 4)]. Allocates nothing. The reference has its
    callers run per_token_cast_to_fp8 and then copy into the buffer (tests/test_mega_moe.py:53-59, README)."""
    m, k = x.shape
    packed_k = ceil_div(ceil_div(k, gran_k), 4)
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.stride(1) == 1):
        raise RuntimeError('x must be a CUDA bfloat16 tensor with unit inner stride')
    if not (q_out.dtype == torch.float8_e4m3fn and q_out.shape[0] >= m and q_out.shape[1] == k and q_out.stride(1) == 1):
        raise RuntimeError('q_out must be float8_e4m3fn [>= M, K]')
    if not (sf_packed_out.dtype == torch.int32 and sf_packed_out.shape[0] >= m and sf_packed_out.shape[1] == packed_k and
            sf_packed_out.stride(1) == 1):
        raise RuntimeError('sf_packed_out must be int32 [>= M, ceil(K / gran_k / 4)], token-major')
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().dgb200_per_token_cast_to_fp8(
            _ptr(x), x.stride(0), m, k, gran_k, _ptr(q_out), q_out.stride(0), None, _ptr(sf_packed_out), 1,
            sf_packed_out.stride(0), _lib.current_stream_ptr()))
