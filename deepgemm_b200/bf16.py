"""BF16 x BF16 GEMMs with the reference's Python signatures (csrc/apis/gemm.hpp:404-564, pybind defaults at
:722-753): the same persistent tcgen05 kernel as the FP8 x FP4 family, issued as kind::f16 without scale factors.
Outputs are written in place; nothing is returned."""
import ctypes
from typing import Optional

import torch

from . import _lib
from .gemm import _prepare_accumulator
from .runtime import get_mk_alignment_for_contiguous_layout


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _check_bf16(t: torch.Tensor, rank: int, name: str, allow_mn_major: bool = False):
    if not t.is_cuda or t.dim() != rank or t.dtype != torch.bfloat16:
        raise RuntimeError(f'{name} must be a {rank}-D CUDA bfloat16 tensor')
    if t.stride(-1) != 1 and not (allow_mn_major and t.stride(-2) == 1):
        raise RuntimeError(f'{name} must be K-major')
    return tuple(t.shape)


def _b_major(b: torch.Tensor, name: str):
    """(mn_major flag, row stride in elements) of a weight operand [.., N, K]: K contiguous, or N contiguous (a transposed
    view of [.., K, N] storage, the operand of the reference's "nn" forms)."""
    if b.stride(-1) == 1:
        return 0, b.stride(-2)
    if b.stride(-2) == 1:
        return 1, b.stride(-1)
    raise RuntimeError(f'{name} must be contiguous along K or along N')


def _check_out(d: torch.Tensor, shape, allow_fp32: bool):
    ok_types = (torch.bfloat16, torch.float32) if allow_fp32 else (torch.bfloat16,)
    if tuple(d.shape) != tuple(shape) or d.dtype not in ok_types or not d.is_cuda or d.stride(-1) != 1:
        raise RuntimeError(f'd must be a CUDA {"bfloat16 / float32" if allow_fp32 else "bfloat16"} {tuple(shape)} tensor '
                           'with unit stride on N')


def bf16_gemm_nt(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, c: Optional[torch.Tensor] = None,
                 compiled_dims: str = 'nk') -> None:
    """Dense D = A @ B.T, a [M, K], b [N, K] bfloat16, d bfloat16 or float32.
    With ``c`` (float32, float32 d): d = c + a @ b.T. Reference: bf16_gemm_nt, csrc/apis/gemm.hpp:404-438."""
    del compiled_dims
    m, k = _check_bf16(a, 2, 'a', allow_mn_major=True)
    n, k_ = _check_bf16(b, 2, 'b', allow_mn_major=True)
    if k != k_:
        raise RuntimeError(f'K mismatch: a has {k}, b has {k_}')
    _check_out(d, (m, n), True)
    if m == 0:
        return
    accumulate = _prepare_accumulator(c, d)
    a_mn, a_stride = _b_major(a, 'a')
    b_mn, b_stride = _b_major(b, 'b')
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_bf16_gemm_nt(_p(a), a_stride, a_mn, _p(b), b_stride, b_mn, _p(d), d.stride(0), m, n, k,
                                                  int(d.dtype == torch.float32), accumulate, _lib.current_stream_ptr()))


def bf16_gemm_nn(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, c: Optional[torch.Tensor] = None,
                 compiled_dims: str = 'nk') -> None:
    """b given as [K, N] (reference: csrc/apis/gemm.hpp:440-446 transposes the view and calls the NT form): a row-major
    [K, N] tensor is an MN-major operand and is read as such."""
    bf16_gemm_nt(a, b.transpose(0, 1), d, c, compiled_dims)


def bf16_gemm_tn(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, c: Optional[torch.Tensor] = None,
                 compiled_dims: str = 'nk') -> None:
    """a given as [K, M], b as [K, N] (reference: csrc/apis/gemm.hpp:448-454)."""
    bf16_gemm_nt(a.transpose(0, 1), b.transpose(0, 1), d, c, compiled_dims)


def bf16_gemm_tt(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, c: Optional[torch.Tensor] = None,
                 compiled_dims: str = 'nk') -> None:
    """a given as [K, M], b as [N, K] (reference: csrc/apis/gemm.hpp:456-462)."""
    bf16_gemm_nt(a.transpose(0, 1), b, d, c, compiled_dims)


def m_grouped_bf16_gemm_nt_contiguous(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, grouped_layout: torch.Tensor,
                                      compiled_dims: str = 'nk', use_psum_layout: bool = False,
                                      ensure_zero_padding: bool = True,
                                      expected_m_for_psum_layout: Optional[int] = None) -> None:
    """D[m] = A[m] @ B[group(m)].T; reference: m_grouped_bf16_gemm_nt_contiguous, csrc/apis/gemm.hpp:464-517."""
    del compiled_dims
    m, k = _check_bf16(a, 2, 'a')
    num_groups, n, k_ = _check_bf16(b, 3, 'b', allow_mn_major=True)
    if k != k_:
        raise RuntimeError(f'K mismatch: a has {k}, b has {k_}')
    b_mn, b_stride = _b_major(b, 'b')
    if not (b.is_contiguous() or (b_mn and b.transpose(1, 2).is_contiguous())):
        raise RuntimeError('b must be contiguous ([G, N, K], or [G, K, N] storage viewed as [G, N, K])')
    _check_out(d, (m, n), False)
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
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_m_grouped_bf16_gemm_nt_contiguous(
            _p(a), a.stride(0), _p(b), b_stride, b_mn, _p(d), d.stride(0), _p(grouped_layout), m, n, k, num_groups, 0,
            1 if use_psum_layout else 0, get_mk_alignment_for_contiguous_layout(),
            int(bool(ensure_zero_padding and use_psum_layout)), _lib.current_stream_ptr()))


def m_grouped_bf16_gemm_nn_contiguous(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, grouped_layout: torch.Tensor,
                                      compiled_dims: str = 'nk', use_psum_layout: bool = False,
                                      ensure_zero_padding: bool = True) -> None:
    """B given as [G, K, N] (contiguous: an MN-major operand; or a view of [G, N, K] storage); reference:
    csrc/apis/gemm.hpp:519-526."""
    m_grouped_bf16_gemm_nt_contiguous(a, b.transpose(1, 2), d, grouped_layout, compiled_dims, use_psum_layout,
                                      ensure_zero_padding, None)


def m_grouped_bf16_gemm_nt_masked(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, masked_m: torch.Tensor,
                                  expected_m: int, compiled_dims: str = 'nk') -> None:
    """Per group g only rows < masked_m[g]; reference: m_grouped_bf16_gemm_nt_masked, csrc/apis/gemm.hpp:528-564."""
    del compiled_dims
    num_groups, m, k = _check_bf16(a, 3, 'a')
    num_groups_b, n, k_ = _check_bf16(b, 3, 'b')
    if num_groups != num_groups_b or k != k_ or masked_m.numel() != num_groups:
        raise RuntimeError('group count or K mismatch between a, b and masked_m')
    if not a.is_contiguous() or not b.is_contiguous() or not d.is_contiguous():
        raise RuntimeError('a, b and d must be contiguous')
    _check_out(d, (num_groups, m, n), False)
    if not (expected_m > 0 and m > 0 and n > 0 and k > 0 and num_groups > 0):
        raise RuntimeError('expected_m, m, n, k and num_groups must be positive')
    if masked_m.dtype != torch.int32 or not masked_m.is_contiguous() or not masked_m.is_cuda:
        raise RuntimeError('masked_m must be a contiguous CUDA int32 tensor')
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_m_grouped_bf16_gemm_nt_masked(
            _p(a), _p(b), _p(d), d.stride(1), _p(masked_m), num_groups, m, n, k, int(expected_m), 0,
            _lib.current_stream_ptr()))
