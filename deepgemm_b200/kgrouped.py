"""K-grouped GEMMs (MoE weight gradient) with the reference's Python signatures (k_grouped_fp8_gemm_tn_contiguous,
csrc/apis/gemm.hpp:299-346, and k_grouped_bf16_gemm_tn_contiguous, :566-608; pybind defaults at :695-701 and :752-757).
d is written in place."""
import ctypes
from typing import List, Optional, Tuple

import torch

from . import _lib
from .runtime import get_mk_alignment_for_contiguous_layout


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _check_ks(ks_cpu, num_groups, use_psum_layout, block_k, rows_of_a):
    """(rows of a and b, K rows the scale factors cover or None if unknown) after the reference's argument rules
    (check_k_grouped_args, csrc/apis/gemm.hpp:48-69): the plain layout needs ks_cpu; with the psum layout the operand's
    own row count is taken and ks_cpu, when given, holds each group's K extent rounded up to the alignment."""
    if use_psum_layout:
        alignment = get_mk_alignment_for_contiguous_layout()
        if alignment % block_k != 0:
            raise RuntimeError(f'the psum layout needs a K alignment that is a multiple of {block_k}, got {alignment}')
        if rows_of_a % block_k != 0:
            raise RuntimeError(f'a and b must have a multiple of {block_k} rows')
        return rows_of_a, None
    if ks_cpu is None or len(ks_cpu) != num_groups:
        raise RuntimeError('ks_cpu must list one K extent per group')
    if any(k % block_k != 0 or k < 0 for k in ks_cpu):
        raise RuntimeError(f'every K extent must be a non-negative multiple of {block_k}')
    return int(sum(ks_cpu)), int(sum(ks_cpu))


def k_grouped_fp8_gemm_tn_contiguous(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                     d: torch.Tensor, ks_cpu: Optional[List[int]], grouped_layout: torch.Tensor,
                                     c: Optional[torch.Tensor] = None, recipe: Tuple[int, int, int] = (1, 1, 128),
                                     compiled_dims: str = 'mn', use_psum_layout: bool = False) -> None:
    """For every group g: d[g] = c[g] + a[rows of g].T @ b[rows of g].

    a = (float8_e4m3fn [sum_k, m], float32 [sum_k / g, m]), b = (float8_e4m3fn [sum_k, n], float32 [sum_k / g, n]) with
    g = recipe[2]: the K rows of the groups concatenated, one power-of-two scale per g K rows and channel (the reference's
    k_grouped_per_channel_cast_to_fp8, tests/generators.py:413-435). ``grouped_layout`` is the int32 CUDA tensor of the
    groups' K extents and ``ks_cpu`` the same numbers on the host; d and c are float32 [G, m, n] (c may be d).
    With ``use_psum_layout`` ``grouped_layout`` holds the groups' end rows instead: group g starts at
    align(end[g - 1], get_mk_alignment_for_contiguous_layout()), the rows in the gaps are zero, and ``ks_cpu`` may be None
    (tests/generators.py:482-533). Built: recipes (1, 1, 128) and (1, 1, 32); plain layout with K extents that are multiples of 128;
    psum layout with a K alignment that is a multiple of 128."""
    del compiled_dims
    if tuple(recipe) not in ((1, 1, 128), (1, 1, 32)):
        raise RuntimeError('the recipe must be (1, 1, 128) or (1, 1, 32)')
    gran_k = recipe[2]
    (a_q, a_sf), (b_q, b_sf) = a, b
    if d.dim() != 3 or d.dtype != torch.float32 or not d.is_cuda or not d.is_contiguous():
        raise RuntimeError('d must be a contiguous CUDA float32 [G, m, n] tensor')
    num_groups, m, n = d.shape
    if c is None or tuple(c.shape) != tuple(d.shape) or c.dtype != torch.float32 or not c.is_contiguous():
        raise RuntimeError('c must be a contiguous float32 tensor of the shape of d (it may be d itself)')
    if grouped_layout.dtype != torch.int32 or not grouped_layout.is_contiguous() or not grouped_layout.is_cuda or \
            grouped_layout.numel() != num_groups:
        raise RuntimeError('grouped_layout must be a contiguous CUDA int32 tensor with one K extent per group')
    sum_k, sf_rows = _check_ks(ks_cpu, num_groups, use_psum_layout, 128, a_q.size(0))
    sf_rows = a_sf.size(0) if sf_rows is None else sf_rows // gran_k
    for q, sf, mn, name in ((a_q, a_sf, m, 'a'), (b_q, b_sf, n, 'b')):
        if q.dtype != torch.float8_e4m3fn or tuple(q.shape) != (sum_k, mn) or not q.is_contiguous() or not q.is_cuda:
            raise RuntimeError(f'{name} must be a contiguous CUDA float8_e4m3fn [{sum_k}, {mn}] tensor')
        if sf.dtype != torch.float32 or tuple(sf.shape) != (sf_rows, mn) or not sf.is_contiguous():
            raise RuntimeError(f'scale factors of {name} must be contiguous float32 [{sf_rows}, {mn}]')
    with torch.cuda.device(d.device):
        nbytes = _lib.lib().dgb200_k_grouped_sf_workspace_bytes(num_groups, m, n, sum_k)
        workspace = torch.empty(max(int(nbytes), 16), dtype=torch.int8, device=d.device)
        _lib.check(_lib.lib().dgb200_k_grouped_fp8_gemm_tn_contiguous(
            _p(a_q), _p(a_sf), sf_rows, _p(b_q), _p(b_sf), _p(c), _p(d), _p(grouped_layout), int(use_psum_layout),
            get_mk_alignment_for_contiguous_layout(), gran_k, num_groups, m, n, sum_k, _p(workspace),
            _lib.current_stream_ptr()))


def k_grouped_bf16_gemm_tn_contiguous(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, ks_cpu: Optional[List[int]],
                                      grouped_layout: torch.Tensor, c: Optional[torch.Tensor] = None,
                                      compiled_dims: str = 'mn', use_psum_layout: bool = False) -> None:
    """For every group g: d[g] = c[g] + a[rows of g].T @ b[rows of g] with a bfloat16 [sum_k, m], b bfloat16 [sum_k, n].
    Built: plain layout with K extents that are multiples of 64; psum layout with a K alignment that is one."""
    del compiled_dims
    if d.dim() != 3 or d.dtype != torch.float32 or not d.is_cuda or not d.is_contiguous():
        raise RuntimeError('d must be a contiguous CUDA float32 [G, m, n] tensor')
    num_groups, m, n = d.shape
    if c is None or tuple(c.shape) != tuple(d.shape) or c.dtype != torch.float32 or not c.is_contiguous():
        raise RuntimeError('c must be a contiguous float32 tensor of the shape of d (it may be d itself)')
    if grouped_layout.dtype != torch.int32 or not grouped_layout.is_contiguous() or not grouped_layout.is_cuda or \
            grouped_layout.numel() != num_groups:
        raise RuntimeError('grouped_layout must be a contiguous CUDA int32 tensor with one K extent per group')
    sum_k, _ = _check_ks(ks_cpu, num_groups, use_psum_layout, 64, a.size(0))
    for t, mn, name in ((a, m, 'a'), (b, n, 'b')):
        if t.dtype != torch.bfloat16 or tuple(t.shape) != (sum_k, mn) or not t.is_contiguous() or not t.is_cuda:
            raise RuntimeError(f'{name} must be a contiguous CUDA bfloat16 [{sum_k}, {mn}] tensor')
    with torch.cuda.device(d.device):
        _lib.check(_lib.lib().dgb200_k_grouped_bf16_gemm_tn_contiguous(
            _p(a), _p(b), _p(c), _p(d), _p(grouped_layout), int(use_psum_layout), get_mk_alignment_for_contiguous_layout(),
            num_groups, m, n, sum_k, _lib.current_stream_ptr()))
