"""Scale-factor layout transforms (reference: csrc/apis/layout.hpp:14-90, csrc/utils/layout.hpp:74-127)."""
import ctypes
from typing import Optional, Tuple, Union

import torch

from . import _lib
from .utils.math import align, ceil_div


def get_tma_aligned_size(x: int, element_size: int) -> int:
    """Reference: csrc/utils/math.hpp:23-26."""
    return align(x, 16 // element_size)


def _recipe_grans(recipe, is_sfa) -> Tuple[int, int]:
    if len(recipe) == 3:
        if is_sfa is None:
            raise RuntimeError('a 3-element recipe needs is_sfa')
        return (recipe[0] if is_sfa else recipe[1]), recipe[2]
    if len(recipe) == 2:
        if is_sfa is not None:
            raise RuntimeError('a 2-element recipe must not pass is_sfa')
        return recipe[0], recipe[1]
    raise RuntimeError('invalid recipe')


def check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups, tma_stride_check=False, type_check=None):
    """Reference: check_sf_layout, csrc/utils/layout.hpp:90-127."""
    if type_check is not None and sf.dtype != type_check:
        raise RuntimeError(f'scale factors must be {type_check}')
    if sf.dtype not in (torch.float32, torch.int32):
        raise RuntimeError('scale factors must be float32 or int32')
    if sf.dim() != (3 if num_groups is not None else 2):
        raise RuntimeError('scale-factor rank does not match num_groups')
    if num_groups is not None and sf.size(-3) != num_groups:
        raise RuntimeError('scale-factor group count mismatch')
    if sf.size(-2) != ceil_div(mn, gran_mn):
        raise RuntimeError(f'scale-factor MN extent {sf.size(-2)} != ceil({mn} / {gran_mn})')
    per_elem = 1 if sf.dtype == torch.float32 else 4
    if sf.size(-1) != ceil_div(k, gran_k * per_elem):
        raise RuntimeError(f'scale-factor K extent {sf.size(-1)} != ceil({k} / {gran_k * per_elem})')
    if tma_stride_check:
        if num_groups is not None and sf.stride(-3) != sf.stride(-1) * sf.size(-1):
            raise RuntimeError('packed scale factors: group stride must be K extent x K stride')
        if not (sf.stride(-2) == 1 or mn == 1):
            raise RuntimeError('packed scale factors must be MN-major')
        if sf.stride(-1) != get_tma_aligned_size(mn, sf.element_size()):
            raise RuntimeError('packed scale factors: K stride must be the TMA-aligned MN size')
    return sf


def get_mn_major_tma_aligned_packed_ue8m0_tensor(sf: torch.Tensor, psum_layout: Optional[torch.Tensor] = None,
                                                 psum_alignment: Optional[int] = None) -> torch.Tensor:
    """fp32 power-of-two scales [G?, MN, SFK] -> int32 [G?, MN, ceil(SFK / 4)], MN-major, MN stride align(MN, 4).
    Reference: csrc/jit_kernels/impls/smxx_layout.hpp:180-253."""
    if not (sf.is_cuda and sf.dtype == torch.float32 and sf.dim() in (2, 3)):
        raise RuntimeError('expected a 2-D or 3-D CUDA float32 tensor')
    squeeze = sf.dim() == 2
    sf3 = sf.unsqueeze(0) if squeeze else sf
    g, mn, sf_k = sf3.shape
    packed_k, aligned_mn = ceil_div(sf_k, 4), align(mn, 4)
    out = torch.empty((g, packed_k, aligned_mn), dtype=torch.int32, device=sf.device)
    from .runtime import get_mk_alignment_for_contiguous_layout
    with torch.cuda.device(sf.device):
        _lib.check(_lib.lib().dgb200_transform_sf_into_required_layout(
            ctypes.c_void_p(sf3.data_ptr()), sf3.stride(0), sf3.stride(1), sf3.stride(2), ctypes.c_void_p(out.data_ptr()),
            g, mn, sf_k, 1,
            ctypes.c_void_p(psum_layout.data_ptr()) if psum_layout is not None else None,
            psum_layout.numel() if psum_layout is not None else 0,
            (psum_alignment or get_mk_alignment_for_contiguous_layout()) if psum_layout is not None else 0,
            _lib.current_stream_ptr()))
    view = out.transpose(1, 2)[:, :mn, :]
    return view[0] if squeeze else view


def transform_sf_into_required_layout(sf: torch.Tensor, mn: int, k: int,
                                      recipe: Union[Tuple[int, int, int], Tuple[int, int]],
                                      num_groups: Optional[int] = None, is_sfa: Optional[bool] = None,
                                      disable_ue8m0_cast: bool = False,
                                      psum_layout: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Reference: transform_sf_into_required_layout, csrc/apis/layout.hpp:14-61 (the sm_100 branches)."""
    gran_mn, gran_k = _recipe_grans(tuple(recipe), is_sfa)
    check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups)
    if sf.dtype == torch.float32 and gran_k in (32, 128):
        if disable_ue8m0_cast:
            raise RuntimeError('sm_100a kernels need UE8M0 scales: disable_ue8m0_cast is not supported')
        if gran_mn != 1:
            index = torch.arange(mn, device=sf.device) // gran_mn
            sf = sf.index_select(-2, index)
        return get_mn_major_tma_aligned_packed_ue8m0_tensor(sf, psum_layout)
    if sf.dtype == torch.int32 and gran_mn == 1 and gran_k in (32, 128):
        return check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups, tma_stride_check=True, type_check=torch.int32)
    raise RuntimeError('Unknown SF transformation')


def get_default_recipe(sfa_dtype, sfb_dtype) -> Tuple[int, int, int]:
    """Reference: get_default_recipe, csrc/utils/layout.hpp:74-87 (arch 10)."""
    if sfb_dtype not in (torch.float32, torch.int32):
        raise RuntimeError('unsupported scale-factor dtype')
    return (1, 128, 128) if sfb_dtype == torch.float32 else (1, 1, 128)


def transform_sf_pair_into_required_layout(sfa, sfb, m, n, k, recipe, recipe_a, recipe_b, num_groups_a, num_groups_b,
                                           disable_ue8m0_cast=False, psum_layout=None):
    """Reference: transform_sf_pair_into_required_layout, csrc/apis/layout.hpp:63-90."""
    if recipe_a is None and recipe is None:
        recipe = get_default_recipe(sfa.dtype, sfb.dtype)
    if (recipe_a is None) != (recipe_b is None):
        raise RuntimeError('recipe_a and recipe_b must be given together')
    if (recipe_a is None) == (recipe is None):
        raise RuntimeError('give either recipe or the recipe_a / recipe_b pair')
    if recipe is not None:
        ta = transform_sf_into_required_layout(sfa, m, k, recipe, num_groups_a, True, disable_ue8m0_cast, psum_layout)
        tb = transform_sf_into_required_layout(sfb, n, k, recipe, num_groups_b, False, disable_ue8m0_cast)
        return ta, tb, recipe[2], recipe[2]
    ta = transform_sf_into_required_layout(sfa, m, k, recipe_a, num_groups_a, None, disable_ue8m0_cast, psum_layout)
    tb = transform_sf_into_required_layout(sfb, n, k, recipe_b, num_groups_b, None, disable_ue8m0_cast)
    return ta, tb, recipe_a[1], recipe_b[1]
