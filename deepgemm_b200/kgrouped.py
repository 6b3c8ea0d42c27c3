"""K-grouped GEMMs (MoE weight gradient) with the reference's Python signatures (k_grouped_fp8_gemm_tn_contiguous,
csrc/apis/gemm.hpp:299-346, and k_grouped_bf16_gemm_tn_contiguous, :566-608; pybind defaults at :695-701 and :752-757).
d is written in place."""
import ctypes
from typing import List, Optional, Tuple

import torch

from . import _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def k_grouped_fp8_gemm_tn_contiguous(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                     d: torch.Tensor, ks_cpu: Optional[List[int]], grouped_layout: torch.Tensor,
                                     c: Optional[torch.Tensor] = None, recipe: Tuple[int, int, int] = (1, 1, 128),
                                     compiled_dims: str = 'mn', use_psum_layout: bool = False) -> None:
    """For every group g: d[g] = c[g] + a[rows of g].T @ b[rows of g].

    a = (float8_e4m3fn [sum_k, m], float32 [sum_k / 128, m]), b = (float8_e4m3fn [sum_k, n], float32 [sum_k / 128, n]):
    the K rows of the groups concatenated, one power-of-two scale per 128 K rows and channel (the reference's
    k_grouped_per_channel_cast_to_fp8, tests/generators.py:413-435). ``grouped_layout`` is the int32 CUDA tensor of the
    groups' K extents and ``ks_cpu`` the same numbers on the host; d and c are float32 [G, m, n] (c may be d).
    Built: recipe (1, 1, 128), K extents that are multiples of 128, the plain (non-psum) layout."""
    del compiled_dims
    if tuple(recipe) != (1, 1, 128):
        raise RuntimeError('only recipe (1, 1, 128) is built')
    if use_psum_layout:
        raise RuntimeError('the psum layout of the K-grouped GEMM is not built')
    (a_q, a_sf), (b_q, b_sf) = a, b
    if d.dim() != 3 or d.dtype != torch.float32 or not d.is_cuda or not d.is_contiguous():
        raise RuntimeError('d must be a contiguous CUDA float32 [G, m, n] tensor')
    num_groups, m, n = d.shape
    if c is None or tuple(c.shape) != tuple(d.shape) or c.dtype != torch.float32 or not c.is_contiguous():
        raise RuntimeError('c must be a contiguous float32 tensor of the shape of d (it may be d itself)')
    if grouped_layout.dtype != torch.int32 or not grouped_layout.is_contiguous() or not grouped_layout.is_cuda or \
            grouped_layout.numel() != num_groups:
        raise RuntimeError('grouped_layout must be a contiguous CUDA int32 tensor with one K extent per group')
    if ks_cpu is None or len(ks_cpu) != num_groups:
        raise RuntimeError('ks_cpu must list one K extent per group')
    if any(k % 128 != 0 or k < 0 for k in ks_cpu):
        raise RuntimeError('every K extent must be a non-negative multiple of 128')
    sum_k = int(sum(ks_cpu))
    for q, sf, mn, name in ((a_q, a_sf, m, 'a'), (b_q, b_sf, n, 'b')):
        if q.dtype != torch.float8_e4m3fn or tuple(q.shape) != (sum_k, mn) or not q.is_contiguous() or not q.is_cuda:
            raise RuntimeError(f'{name} must be a contiguous CUDA float8_e4m3fn [{sum_k}, {mn}] tensor')
        if sf.dtype != torch.float32 or tuple(sf.shape) != (sum_k // 128, mn) or not sf.is_contiguous():
            raise RuntimeError(f'scale factors of {name} must be contiguous float32 [{sum_k // 128}, {mn}]')
    with torch.cuda.device(d.device):
        nbytes = _lib.lib().dgb200_k_grouped_sf_workspace_bytes(num_groups, m, n, sum_k)
        workspace = torch.empty(max(int(nbytes), 16), dtype=torch.int8, device=d.device)
        _lib.check(_lib.lib().dgb200_k_grouped_fp8_gemm_tn_contiguous(
            _p(a_q), _p(a_sf), _p(b_q), _p(b_sf), _p(c), _p(d), _p(grouped_layout), num_groups, m, n, sum_k,
            _p(workspace), _lib.current_stream_ptr()))


def k_grouped_bf16_gemm_tn_contiguous(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, ks_cpu: Optional[List[int]],
                                      grouped_layout: torch.Tensor, c: Optional[torch.Tensor] = None,
                                      compiled_dims: str = 'mn', use_psum_layout: bool = False) -> None:
    """For every group g: d[g] = c[g] + a[rows of g].T @ b[rows of g] with a bfloat16 [sum_k, m], b bfloat16 [sum_k, n].
    Built: K extents that are multiples of 64, the plain (non-psum) layout."""
    del compiled_dims
    if use_psum_layout:
        raise RuntimeError('the psum layout of the K-grouped GEMM is not built')
    if d.dim() != 3 or d.dtype != torch.float32 or not d.is_cuda or not d.is_contiguous():
        raise RuntimeError('d must be a contiguous CUDA float32 [G, m, n] tensor')
    num_groups, m, n = d.shape
    if c is None or tuple(c.shape) != tuple(d.shape) or c.dtype != torch.float32 or not c.is_contiguous():
        raise RuntimeError('c must be a contiguous float32 tensor of the shape of d (it may be d itself)')
    if grouped_layout.dtype != torch.int32 or not grouped_layout.is_contiguous() or not grouped_layout.is_cuda or \
            grouped_layout.numel() != num_groups:
        raise RuntimeError('grouped_layout must be a contiguous CUDA int32 tensor with one K extent per group')
    if ks_cpu is None or len(ks_cpu) != num_groups:
        raise RuntimeError('ks_cpu must list one K extent per group')
    if any(k % 64 != 0 or k < 0 for k in ks_cpu):
        raise RuntimeError('every K extent must be a non-negative multiple of 64')
    sum_k = int(sum(ks_cpu))
    for t, mn, name in ((a, m, 'a'), (b, n, 'b')):
        if t.dtype != torch.bfloat16 or tuple(t.shape) != (sum_k, mn) or not t.is_contiguous() or not t.is_cuda:
            raise RuntimeError(f'{name} must be a contiguous CUDA bfloat16 [{sum_k}, {mn}] tensor')
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_k_grouped_bf16_gemm_tn_contiguous(
            _p(a), _p(b), _p(c), _p(d), _p(grouped_layout), num_groups, m, n, sum_k, _lib.current_stream_ptr()))
