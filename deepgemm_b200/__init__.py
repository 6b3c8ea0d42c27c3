"""deepgemm_b200: the Mega-MoE hot path of DeepGEMM rebuilt for B200 (sm_100a).

Same operator names and argument conventions as the reference package (deep_gemm/__init__.py:17-97) for the
path it covers; use ``import deepgemm_b200 as deep_gemm``. Every operator calls libdgb200.so through its C ABI
(include/dgb200.h); there is no CPU or PyTorch fallback.
"""
from . import _lib, testing, utils  # noqa: F401
from .bf16 import (  # noqa: F401
    bf16_gemm_nn,
    bf16_gemm_nt,
    bf16_gemm_tn,
    bf16_gemm_tt,
    m_grouped_bf16_gemm_nn_contiguous,
    m_grouped_bf16_gemm_nt_contiguous,
    m_grouped_bf16_gemm_nt_masked,
)
from .gemm import (  # noqa: F401
    fp8_fp4_gemm_nn,
    fp8_fp4_gemm_nt,
    fp8_gemm_nn,
    fp8_gemm_nt,
    m_grouped_fp8_fp4_gemm_nn_contiguous,
    m_grouped_fp8_fp4_gemm_nt_contiguous,
    m_grouped_fp8_fp4_gemm_nt_masked,
    m_grouped_fp8_gemm_nn_contiguous,
    m_grouped_fp8_gemm_nt_contiguous,
    m_grouped_fp8_gemm_nt_masked,
)
from .kgrouped import k_grouped_bf16_gemm_tn_contiguous, k_grouped_fp8_gemm_tn_contiguous  # noqa: F401
from .layout import (  # noqa: F401
    get_mn_major_tma_aligned_packed_ue8m0_tensor,
    get_tma_aligned_size,
    transform_sf_into_required_layout,
)
from .mega import (  # noqa: F401
    SymmBuffer,
    bf16_mega_moe,
    fp8_fp4_mega_moe,
    fp8_fp4_mega_moe_bf16_input,
    get_block_m_for_mega_moe,
    get_segment_alignment_for_mega_moe,
    get_symm_buffer_for_mega_moe,
    get_token_alignment_for_mega_moe,
    nvfp4_mega_moe,
    nvfp4_mega_moe_bf16_input,
    route_sigmoid_topk,
    share_weights_for_mega_moe,
    transform_weights_for_mega_moe,
)
from .nvfp4 import (  # noqa: F401
    m_grouped_nvfp4_gemm_nt_contiguous,
    nvfp4_tensor_scale,
    pack_nvfp4_sf_mn_major,
    per_token_cast_to_nvfp4,
    per_token_cast_to_nvfp4_into,
)
from .runtime import (  # noqa: F401
    get_mk_alignment_for_contiguous_layout,
    get_num_sms,
    get_pdl,
    get_tc_util,
    get_theoretical_mk_alignment_for_contiguous_layout,
    init,
    set_block_size_multiple_of,
    set_ignore_compile_dims,
    set_mk_alignment_for_contiguous_layout,
    set_num_sms,
    set_pdl,
    set_tc_util,
)

__version__ = '0.1.0'
