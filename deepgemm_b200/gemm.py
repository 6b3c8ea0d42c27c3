"""m-grouped FP8 x FP4 (or FP8 x FP8) GEMMs with the reference's Python signatures
(csrc/apis/gemm.hpp:166-297, pybind defaults at :673-694). Outputs are written in place; nothing is returned."""
import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from .layout import transform_sf_pair_into_required_layout
from .runtime import get_mk_alignment_for_contiguous_layout

kPackedFP4 = torch.int8  # two E2M1 codes per byte, logical K = 2 x last dim (reference: csrc/utils/math.hpp:11)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _check_ab(t: torch.Tensor, rank: int, name: str):
    if not t.is_cuda or t.dim() != rank:
        raise RuntimeError(f'{name} must be a {rank}-D CUDA tensor')
    if t.dtype not in (torch.float8_e4m3fn, kPackedFP4):
        raise RuntimeError(f'{name} must be float8_e4m3fn or packed FP4 (int8)')
    if t.stride(-1) != 1 or not t.is_contiguous():
        raise RuntimeError(f'{name} must be K-major and contiguous')
    k = t.size(-1) * (2 if t.dtype == kPackedFP4 else 1)
    return tuple(t.shape[:-1]) + (k,)


def _check_grouped_b(t: torch.Tensor):
    """b of the m-grouped contiguous GEMM, logically [G, N, K]: K-major and contiguous, or MN-major, i.e. a transposed
    view of contiguous [G, K, N] storage (FP8) or [G, K, N / 2] storage (packed FP4, two N elements per byte, logical
    shape [G, N / 2, K]), as the reference accepts on SM100 (csrc/apis/gemm.hpp:181-183, tests/generators.py:282-292).
    Returns (num_groups, n, k, mn_major)."""
    if not t.is_cuda or t.dim() != 3:
        raise RuntimeError('b must be a 3-D CUDA tensor')
    if t.dtype not in (torch.float8_e4m3fn, kPackedFP4):
        raise RuntimeError('b must be float8_e4m3fn or packed FP4 (int8)')
    fp4 = t.dtype == kPackedFP4
    if t.is_contiguous():
        return t.size(0), t.size(1), t.size(2) * (2 if fp4 else 1), False
    if t.transpose(1, 2).is_contiguous():
        return t.size(0), t.size(1) * (2 if fp4 else 1), t.size(2), True
    raise RuntimeError('b must be K-major and contiguous, or the transposed view of a contiguous [G, K, N] tensor')


def _prepare_accumulator(c, d):
    """The reference's accumulator input (csrc/apis/gemm.hpp:73-124, :404-438; its tests pass c with a float32 d):
    d = c + a @ b.T. The kernel adds into d, so c is first copied there unless it is d itself. Returns the flag."""
    if c is None:
        return 0
    if d.dtype != torch.float32 or c.dtype != torch.float32 or tuple(c.shape) != tuple(d.shape) or not c.is_cuda:
        raise RuntimeError('c must be a CUDA float32 tensor of the shape of a float32 d')
    if c.data_ptr() != d.data_ptr():
        d.copy_(c)
    return 1


def _check_d(d: torch.Tensor, shape):
    if tuple(d.shape) != tuple(shape):
        raise RuntimeError(f'd has shape {tuple(d.shape)}, expected {tuple(shape)}')
    if d.dtype != torch.bfloat16 or not d.is_cuda or d.stride(-1) != 1:
        raise RuntimeError('d must be a CUDA bfloat16 tensor with unit stride on N')


def fp8_fp4_gemm_nt(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor], d: torch.Tensor,
                    c: Optional[torch.Tensor] = None, recipe: Optional[Tuple[int, int, int]] = None,
                    recipe_a: Optional[Tuple[int, int]] = None, recipe_b: Optional[Tuple[int, int]] = None,
                    compiled_dims: str = 'nk', disable_ue8m0_cast: bool = False) -> None:
    """Dense D = A @ B.T with a [M, K] FP8 and b [N, K] FP8 or packed FP4; d bfloat16 or float32.
    With ``c`` (float32, float32 d): d = c + a @ b.T. Reference: fp8_fp4_gemm_nt, csrc/apis/gemm.hpp:73-124."""
    del compiled_dims
    a_q, a_sf = a
    b_q, b_sf = b
    if a_q.dtype != torch.float8_e4m3fn:
        raise RuntimeError('a must be float8_e4m3fn')
    m, k = _check_ab(a_q, 2, 'a')
    n, k_ = _check_ab(b_q, 2, 'b')
    if k != k_:
        raise RuntimeError(f'K mismatch: a has {k}, b has {k_}')
    if tuple(d.shape) != (m, n) or d.dtype not in (torch.bfloat16, torch.float32) or not d.is_cuda or d.stride(-1) != 1:
        raise RuntimeError(f'd must be a CUDA bfloat16 / float32 [{m}, {n}] tensor with unit stride on N')
    if m == 0:
        return
    accumulate = _prepare_accumulator(c, d)
    sfa, sfb, gran_a, gran_b = transform_sf_pair_into_required_layout(
        a_sf, b_sf, m, n, k, recipe, recipe_a, recipe_b, None, None, disable_ue8m0_cast)
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_fp8_fp4_gemm_nt(
            _p(a_q), _p(sfa), sfa.stride(-1), _p(b_q), _p(sfb), sfb.stride(-1), _p(d), d.stride(0), m, n, k, gran_a, gran_b,
            int(b_q.dtype == kPackedFP4), int(d.dtype == torch.float32), accumulate, _lib.current_stream_ptr()))


def fp8_fp4_gemm_nn(a, b, d, c=None, recipe=None, recipe_a=None, recipe_b=None, compiled_dims: str = 'nk',
                    disable_ue8m0_cast: bool = False) -> None:
    """b given as [K, N] over K-major storage (reference: csrc/apis/gemm.hpp:126-137 transposes and calls the NT form)."""
    fp8_fp4_gemm_nt(a, (b[0].transpose(0, 1), b[1].transpose(0, 1)), d, c, recipe, recipe_a, recipe_b, compiled_dims,
                    disable_ue8m0_cast)


def m_grouped_fp8_fp4_gemm_nt_contiguous(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                         d: torch.Tensor, grouped_layout: torch.Tensor,
                                         recipe: Optional[Tuple[int, int, int]] = None,
                                         recipe_a: Optional[Tuple[int, int]] = None,
                                         recipe_b: Optional[Tuple[int, int]] = None,
                                         compiled_dims: str = 'nk', disable_ue8m0_cast: bool = False,
                                         use_psum_layout: bool = False, ensure_zero_padding: bool = True,
                                         expected_m_for_psum_layout: Optional[int] = None) -> None:
    """D[m] = A[m] @ B[group(m)].T; reference: m_grouped_fp8_fp4_gemm_nt_contiguous, csrc/apis/gemm.hpp:166-232."""
    del compiled_dims
    a_q, a_sf = a
    b_q, b_sf = b
    if a_q.dtype != torch.float8_e4m3fn:
        raise RuntimeError('a must be float8_e4m3fn')
    m, k = _check_ab(a_q, 2, 'a')
    num_groups, n, k_, b_mn_major = _check_grouped_b(b_q)
    if k != k_:
        raise RuntimeError(f'K mismatch: a has {k}, b has {k_}')
    if b_mn_major and n % 32 != 0:
        raise RuntimeError('an MN-major b needs N to be a multiple of 32')
    _check_d(d, (m, n))
    if d.stride(0) * 2 % 16 != 0:
        raise RuntimeError('d rows must be 16-byte aligned')
    if grouped_layout.dtype != torch.int32 or not grouped_layout.is_contiguous() or not grouped_layout.is_cuda:
        raise RuntimeError('grouped_layout must be a contiguous CUDA int32 tensor')
    if use_psum_layout:
        if grouped_layout.numel() != num_groups:
            raise RuntimeError('psum layout needs one entry per group')
    else:
        if grouped_layout.numel() != m:
            raise RuntimeError('grouped_layout needs one entry per row')
        if expected_m_for_psum_layout is not None:
            raise RuntimeError('expected_m_for_psum_layout is only valid with use_psum_layout')
    if m == 0:
        return
    sfa, sfb, gran_a, gran_b = transform_sf_pair_into_required_layout(
        a_sf, b_sf, m, n, k, recipe, recipe_a, recipe_b, None, num_groups, disable_ue8m0_cast,
        grouped_layout if use_psum_layout else None)
    entry = _lib.lib().dgb200_m_grouped_fp8_fp4_gemm_nn_contiguous if b_mn_major else \
        _lib.lib().dgb200_m_grouped_fp8_fp4_gemm_nt_contiguous
    with torch.cuda.device(d.device):
        _lib.check(entry(
            _p(a_q), _p(sfa), sfa.stride(-1), _p(b_q), _p(sfb), sfb.stride(-1), sfb.stride(0),
            _p(d), d.stride(0), _p(grouped_layout), m, n, k, num_groups, gran_a, gran_b,
            int(b_q.dtype == kPackedFP4), 0, 1 if use_psum_layout else 0,
            get_mk_alignment_for_contiguous_layout(), int(bool(ensure_zero_padding and use_psum_layout)),
            _lib.current_stream_ptr()))


def m_grouped_fp8_fp4_gemm_nn_contiguous(a, b, d, grouped_layout, recipe=None, recipe_a=None, recipe_b=None,
                                         compiled_dims: str = 'nk', disable_ue8m0_cast: bool = False,
                                         use_psum_layout: bool = False, ensure_zero_padding: bool = True) -> None:
    """B given as [G, K, N] (packed FP4: [G, K, N / 2]); reference: csrc/apis/gemm.hpp:234-248 (transposes the views and
    calls the NT form, which reads a contiguous [G, K, N] tensor as an MN-major operand)."""
    m_grouped_fp8_fp4_gemm_nt_contiguous(a, (b[0].transpose(1, 2), b[1].transpose(1, 2)), d, grouped_layout, recipe,
                                         recipe_a, recipe_b, compiled_dims, disable_ue8m0_cast, use_psum_layout,
                                         ensure_zero_padding, None)


def m_grouped_fp8_fp4_gemm_nt_masked(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                     d: torch.Tensor, masked_m: torch.Tensor, expected_m: int,
                                     recipe: Optional[Tuple[int, int, int]] = None,
                                     recipe_a: Optional[Tuple[int, int]] = None,
                                     recipe_b: Optional[Tuple[int, int]] = None,
                                     compiled_dims: str = 'nk', disable_ue8m0_cast: bool = False) -> None:
    """Per group g only rows < masked_m[g]; reference: m_grouped_fp8_fp4_gemm_nt_masked, csrc/apis/gemm.hpp:250-297."""
    del compiled_dims
    a_q, a_sf = a
    b_q, b_sf = b
    if a_q.dtype != torch.float8_e4m3fn:
        raise RuntimeError('a must be float8_e4m3fn')
    num_groups, m, k = _check_ab(a_q, 3, 'a')
    num_groups_b, n, k_ = _check_ab(b_q, 3, 'b')
    if num_groups != num_groups_b or k != k_ or masked_m.numel() != num_groups:
        raise RuntimeError('group count or K mismatch between a, b and masked_m')
    _check_d(d, (num_groups, m, n))
    if not d.is_contiguous():
        raise RuntimeError('d must be contiguous')
    if not (expected_m > 0 and m > 0 and n > 0 and k > 0 and num_groups > 0):
        raise RuntimeError('expected_m, m, n, k and num_groups must be positive')
    if masked_m.dtype != torch.int32 or not masked_m.is_contiguous() or not masked_m.is_cuda:
        raise RuntimeError('masked_m must be a contiguous CUDA int32 tensor')
    sfa, sfb, gran_a, gran_b = transform_sf_pair_into_required_layout(
        a_sf, b_sf, m, n, k, recipe, recipe_a, recipe_b, num_groups, num_groups, disable_ue8m0_cast)
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_m_grouped_fp8_fp4_gemm_nt_masked(
            _p(a_q), _p(sfa), sfa.stride(-1), sfa.stride(0), _p(b_q), _p(sfb), sfb.stride(-1), sfb.stride(0),
            _p(d), d.stride(1), _p(masked_m), num_groups, m, n, k, int(expected_m), gran_a, gran_b,
            int(b_q.dtype == kPackedFP4), 0, _lib.current_stream_ptr()))


# FP8-only names are the same entry points (reference: csrc/apis/gemm.hpp:711-717)
fp8_gemm_nt = fp8_fp4_gemm_nt
fp8_gemm_nn = fp8_fp4_gemm_nn
m_grouped_fp8_gemm_nt_contiguous = m_grouped_fp8_fp4_gemm_nt_contiguous
m_grouped_fp8_gemm_nn_contiguous = m_grouped_fp8_fp4_gemm_nn_contiguous
m_grouped_fp8_gemm_nt_masked = m_grouped_fp8_fp4_gemm_nt_masked
