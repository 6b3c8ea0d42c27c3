"""Process-global knobs with the reference's names (csrc/apis/runtime.hpp:12-48, csrc/apis/layout.hpp:142-150).

Kernels here are compiled ahead of time, so knobs that only steer the reference's JIT (compiled dims, block-size
multiples) are accepted and ignored; a knob that would change how a kernel runs and is not built (tensor-core
throttling) raises when set to anything but its default."""
from . import _lib

_state = {'tc_util': 100, 'pdl': True, 'mk_alignment': 128}


def set_num_sms(num_sms: int) -> None:
    _lib.check(_lib.lib().dgb200_set_num_sms(int(num_sms)))


def get_num_sms() -> int:
    return _lib.lib().dgb200_get_num_sms()


def set_tc_util(tc_util: int) -> None:
    """The reference throttles its MMA issue loop to ``tc_util`` percent (csrc/apis/runtime.hpp:21-27). The kernels
    here always issue at full rate: 100 is accepted, any other value is refused rather than silently ignored."""
    if not 0 <= tc_util <= 100:
        raise RuntimeError('tc_util must be in [0, 100]')
    if tc_util != 100:
        raise RuntimeError('tensor-core throttling is not built into these kernels: tc_util must stay 100')
    _state['tc_util'] = int(tc_util)


def get_tc_util() -> int:
    return _state['tc_util']


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch between the kernels of the single-rank layer and of the GEMM entry points
    (reference: set_pdl, csrc/apis/runtime.hpp:24-28). On by default; the reference's default is off."""
    _lib.check(_lib.lib().dgb200_set_tuning(b'pdl', 1 if enabled else 0))
    _state['pdl'] = bool(enabled)


def get_pdl() -> bool:
    return _state['pdl']


def set_ignore_compile_dims(ignore: bool) -> None:
    del ignore


def set_block_size_multiple_of(m: int = 1, n: int = 1) -> None:
    del m, n


def get_mk_alignment_for_contiguous_layout() -> int:
    """Row alignment of each group's segment in the contiguous layout (reference default 128,
    csrc/jit_kernels/heuristics/runtime.hpp:10)."""
    return _state['mk_alignment']


def set_mk_alignment_for_contiguous_layout(alignment: int) -> None:
    if alignment <= 0 or alignment % 4 != 0:
        raise RuntimeError('the contiguous-layout alignment must be a positive multiple of 4')
    _state['mk_alignment'] = int(alignment)


def get_theoretical_mk_alignment_for_contiguous_layout(expected_m=None) -> int:
    """The reference suggests 224..32 by expected rows per group (csrc/jit_kernels/heuristics/runtime.hpp:47-58);
    this kernel's M tile is 128 and it clips stores per group, so 128 is always the efficient choice."""
    del expected_m
    return 128


def init(library_root: str = '', cuda_home: str = '') -> None:
    """No-op: nothing is compiled at run time (reference: _C.init, deep_gemm/__init__.py:124-127)."""
    del library_root, cuda_home
