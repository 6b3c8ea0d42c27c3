"""``import deep_gemm`` resolved to the B200 implementation in this repository.

The reference package of this name (deep_gemm/__init__.py:16-127) re-exports its compiled ``_C`` module; here every
name it exports for the Mega-MoE hot path is bound to ``deepgemm_b200`` (ctypes over the C ABI of libdgb200.so), so
the reference's own test drivers (``import deep_gemm``, ``from deep_gemm.utils import ...``,
``from deep_gemm.testing import ...``, ``from deep_gemm.utils.dist import ...``) run unchanged for that path.
Operators outside the path (einsum, MQA logits, hyperconnection, cuBLASLt wrappers, the Hopper and Triton kernels) do
not exist here: asking for them raises AttributeError, there is no fallback.
"""
import sys as _sys

import deepgemm_b200 as _impl
from deepgemm_b200 import *  # noqa: F401,F403
from deepgemm_b200 import mega, testing, utils  # noqa: F401
from deepgemm_b200.utils import *  # noqa: F401,F403

# submodules under the reference's dotted names
for _name, _module in (('utils', _impl.utils), ('utils.math', _impl.utils.math), ('utils.dist', _impl.utils.dist),
                       ('utils.layout', _impl.layout), ('testing', _impl.testing), ('testing.bench', _impl.testing.bench),
                       ('testing.numeric', _impl.testing.numeric), ('testing.utils', _impl.testing.utils),
                       ('mega', _impl.mega)):
    _sys.modules[f'{__name__}.{_name}'] = _module

# aliases the reference keeps for older callers (deep_gemm/__init__.py:84-86, deep_gemm/utils/layout.py:21-22)
fp8_m_grouped_gemm_nt_masked = _impl.m_grouped_fp8_gemm_nt_masked
bf16_m_grouped_gemm_nt_masked = _impl.m_grouped_bf16_gemm_nt_masked
get_m_alignment_for_contiguous_layout = _impl.get_mk_alignment_for_contiguous_layout
get_k_alignment_for_contiguous_layout = _impl.get_mk_alignment_for_contiguous_layout

__version__ = _impl.__version__
