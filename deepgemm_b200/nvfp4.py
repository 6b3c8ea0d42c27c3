"""NVFP4 x NVFP4 operators: packed E2M1 values, one UE4M3 scale per 16 elements along K, one FP32 scale per tensor.

The reference package has no NVFP4 operators (its FP4 operand is MXFP4 with UE8M0 per-32 scales); the names below
follow its conventions for the FP8 x FP4 path (tuples of (values, scales), outputs written in place,
``use_psum_layout``), with the per-tensor scale added as a third tuple element. Everything runs in libdgb200.so
(tcgen05 ``kind::mxf4nvf4`` with ``scale_vec::4X``); there is no fallback.
"""
import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .runtime import get_mk_alignment_for_contiguous_layout
from .utils.math import align


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _check_x(x: torch.Tensor) -> torch.Tensor:
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2):
        raise RuntimeError('expected a 2-D CUDA bfloat16 tensor')
    if x.size(1) % 64 != 0:
        raise RuntimeError(f'k ({x.size(1)}) must be a multiple of 64')
    return x if x.stride(1) == 1 else x.contiguous()


def nvfp4_tensor_scale(x: torch.Tensor) -> torch.Tensor:
    """FP32 scalar amax(|x|) / (6 * 448) (1.0 for an all-zero tensor), on the device."""
    x = _check_x(x)
    out = torch.empty((), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().dgb200_nvfp4_tensor_scale(_p(x), x.stride(0), x.size(0), x.size(1), _p(out),
                                                        _lib.current_stream_ptr()))
    return out


def per_token_cast_to_nvfp4(x: torch.Tensor, tensor_scale: Optional[torch.Tensor] = None,
                            sf_layout: str = 'token') -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """BF16 [M, K] -> (packed E2M1 int8 [M, K / 2], block scales, FP32 tensor scale).

    ``tensor_scale`` fixes the per-tensor scale (a calibrated scale; block scales then saturate at 448); by default
    it is computed from ``x``. ``sf_layout``: 'token' returns float8_e4m3fn [M, K / 16]; 'mn' returns the packed
    int32 [M, K / 64] view with strides (1, align(M, 4)) that the GEMM consumes directly."""
    x = _check_x(x)
    m, k = x.shape
    if tensor_scale is None:
        tensor_scale = nvfp4_tensor_scale(x)
    if not (tensor_scale.is_cuda and tensor_scale.dtype == torch.float32 and tensor_scale.numel() == 1):
        raise RuntimeError('tensor_scale must be a CUDA float32 scalar')
    q = torch.empty((m, k // 2), dtype=torch.int8, device=x.device)
    if sf_layout == 'token':
        packed = torch.empty((m, k // 64), dtype=torch.int32, device=x.device)
        k_stride, row_stride = 1, k // 64
    elif sf_layout == 'mn':
        packed = torch.zeros((k // 64, align(m, 4)), dtype=torch.int32, device=x.device).t()[:m]
        k_stride, row_stride = align(m, 4), 1
    else:
        raise RuntimeError(f'unknown sf_layout `{sf_layout}`')
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().dgb200_per_token_cast_to_nvfp4(_p(x), x.stride(0), m, k, _p(tensor_scale), _p(q), q.stride(0),
                                                             _p(packed), k_stride, row_stride, _lib.current_stream_ptr()))
    sf = packed.view(torch.uint8).view(torch.float8_e4m3fn) if sf_layout == 'token' else packed
    return q, sf, tensor_scale


def per_token_cast_to_nvfp4_into(x: torch.Tensor, tensor_scale: torch.Tensor, q_out: torch.Tensor,
                                 sf_packed_out: torch.Tensor) -> None:
    """Quantises straight into caller-owned views (the layer buffer's ``x`` int8 [>= M, K / 2] and ``x_sf`` int32
    [>= M, K / 64], token-major) against the given tensor scale. Allocates nothing."""
    x = _check_x(x)
    m, k = x.shape
    if not (q_out.dtype == torch.int8 and q_out.shape[0] >= m and q_out.shape[1] == k // 2 and q_out.stride(1) == 1):
        raise RuntimeError('q_out must be int8 [>= M, K / 2]')
    if not (sf_packed_out.dtype == torch.int32 and sf_packed_out.shape[0] >= m and sf_packed_out.shape[1] == k // 64 and
            sf_packed_out.stride(1) == 1):
        raise RuntimeError('sf_packed_out must be int32 [>= M, K / 64], token-major')
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().dgb200_per_token_cast_to_nvfp4(_p(x), x.stride(0), m, k, _p(tensor_scale), _p(q_out),
                                                             q_out.stride(0), _p(sf_packed_out), 1, sf_packed_out.stride(0),
                                                             _lib.current_stream_ptr()))


def pack_nvfp4_sf_mn_major(sf: torch.Tensor) -> torch.Tensor:
    """UE4M3 block scales float8_e4m3fn [..., MN, K / 16] -> packed int32 [..., MN, K / 64] whose MN dimension has
    stride 1 and whose K dimension has stride align(MN, 4) (one int = the four scales of 64 K elements). Weight
    preparation, done once: plain tensor copies."""
    if sf.dtype != torch.float8_e4m3fn or sf.size(-1) % 4 != 0:
        raise RuntimeError('expected float8_e4m3fn scales with a multiple of 4 blocks per row')
    ints = sf.contiguous().view(torch.uint8).view(torch.int32)  # [..., MN, K / 64]
    mn, kq = ints.shape[-2], ints.shape[-1]
    out = torch.zeros(ints.shape[:-2] + (kq, align(mn, 4)), dtype=torch.int32, device=sf.device)
    out[..., :mn] = ints.transpose(-1, -2)
    return out.transpose(-1, -2)[..., :mn, :]


def _sf_mn_major(sf: torch.Tensor, mn: int, k: int, lead: Tuple[int, ...], name: str) -> torch.Tensor:
    if sf.dtype == torch.float8_e4m3fn:
        if tuple(sf.shape) != lead + (mn, k // 16):
            raise RuntimeError(f'{name} scales must have shape {lead + (mn, k // 16)}')
        sf = pack_nvfp4_sf_mn_major(sf)
    if not (sf.dtype == torch.int32 and tuple(sf.shape) == lead + (mn, k // 64) and sf.stride(-2) == 1 and
            sf.stride(-1) >= mn):
        raise RuntimeError(f'{name} scales must be float8_e4m3fn {lead + (mn, k // 16)} or packed MN-major int32 '
                           f'{lead + (mn, k // 64)}')
    if lead and sf.stride(0) != sf.stride(-1) * sf.size(-1) and sf.size(0) > 1:
        raise RuntimeError(f'{name} packed scales must be dense across groups')
    return sf


def m_grouped_nvfp4_gemm_nt_contiguous(a: Tuple[torch.Tensor, torch.Tensor, torch.Tensor],
                                       b: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], d: torch.Tensor,
                                       grouped_layout: torch.Tensor, use_psum_layout: bool = False) -> None:
    """D[m] = a_scale * b_scales[g(m)] * (A[m] @ B[g(m)].T with UE4M3 block scales).

    a = (int8 [M, K / 2], scales, FP32 scalar); b = (int8 [G, N, K / 2], scales, FP32 [G]); scales as accepted by
    ``pack_nvfp4_sf_mn_major`` or already packed. ``d`` is bfloat16 or float32 [M, N]. The grouped layouts are the
    ones of ``m_grouped_fp8_fp4_gemm_nt_contiguous``."""
    a_q, a_sf, a_scale = a
    b_q, b_sf, b_scales = b
    for t, rank, name in ((a_q, 2, 'a'), (b_q, 3, 'b')):
        if not (t.is_cuda and t.dtype == torch.int8 and t.dim() == rank and t.is_contiguous()):
            raise RuntimeError(f'{name} must be a contiguous {rank}-D CUDA int8 (packed E2M1) tensor')
    m, k = a_q.size(0), a_q.size(1) * 2
    num_groups, n = b_q.size(0), b_q.size(1)
    if b_q.size(2) * 2 != k:
        raise RuntimeError(f'K mismatch: a has {k}, b has {b_q.size(2) * 2}')
    if tuple(d.shape) != (m, n) or d.dtype not in (torch.bfloat16, torch.float32) or d.stride(1) != 1 or not d.is_cuda:
        raise RuntimeError(f'd must be a CUDA bfloat16 / float32 [{m}, {n}] tensor with unit stride on N')
    if not (a_scale.dtype == torch.float32 and a_scale.numel() == 1 and a_scale.is_cuda):
        raise RuntimeError('the scale of a must be a CUDA float32 scalar')
    if not (b_scales.dtype == torch.float32 and b_scales.numel() == num_groups and b_scales.is_contiguous() and b_scales.is_cuda):
        raise RuntimeError('the scales of b must be a contiguous CUDA float32 [num_groups] tensor')
    if grouped_layout.dtype != torch.int32 or not grouped_layout.is_contiguous() or not grouped_layout.is_cuda:
        raise RuntimeError('grouped_layout must be a contiguous CUDA int32 tensor')
    if grouped_layout.numel() != (num_groups if use_psum_layout else m):
        raise RuntimeError('grouped_layout needs one entry per group (psum) or per row')
    if m == 0:
        return
    sfa = _sf_mn_major(a_sf, m, k, (), 'a')
    sfb = _sf_mn_major(b_sf, n, k, (num_groups,), 'b')
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_m_grouped_nvfp4_gemm_nt_contiguous(
            _p(a_q), _p(sfa), sfa.stride(-1), _p(a_scale), _p(b_q), _p(sfb), sfb.stride(-1), sfb.stride(0) if num_groups > 1 else
            sfb.stride(-1) * sfb.size(-1), _p(b_scales), _p(d), d.stride(0), _p(grouped_layout), m, n, k, num_groups,
            int(d.dtype == torch.float32), 1 if use_psum_layout else 0, get_mk_alignment_for_contiguous_layout(),
            _lib.current_stream_ptr()))
