"""CPU checks of the C-ABI boundary: the library loads, exports exactly what include/dgb200.h declares, and its
host-only entry points validate their arguments the way the reference's DG_HOST_ASSERTs do. No kernel is launched."""
import ctypes
import os
import re

import pytest

from deepgemm_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    build.build()
    return _lib.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'dgb200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(dgb200_\w+)\s*\(', text)))


def test_header_symbols_are_exported(lib):
    declared = _declared_symbols()
    assert len(declared) >= 12
    for name in declared:
        assert hasattr(lib, name), f'{name} is declared in include/dgb200.h but not exported'


def test_binding_covers_header():
    assert sorted(_lib.exported_symbols()) == _declared_symbols()


def test_version_and_error_string(lib):
    assert lib.dgb200_version() >= 100
    assert isinstance(lib.dgb200_last_error(), bytes)


def test_buffer_layout_is_ordered_and_aligned(lib):
    words = (ctypes.c_int64 * 16)()
    rc = lib.dgb200_get_symm_buffer_layout_for_mega_moe(1, 256, 4096, 8, 7168, 2048, ctypes.cast(words, ctypes.c_void_p))
    assert rc == 0
    w = list(words)
    total, max_rows = w[0], w[9]
    offsets = [w[i] for i in (1, 2, 3, 4, 5, 6, 7, 8, 10, 11, 12, 13, 14, 15)]
    assert all(o % 1024 == 0 and 0 <= o < total for o in offsets)
    assert len(set(offsets)) == len(offsets)
    assert max_rows % 128 == 0 and max_rows >= 4096 * 8 + 256 * 16
    assert w[2] - w[1] >= 4096 * 7168            # x
    assert w[6] - w[5] >= max_rows * 7168        # l1_acts
    assert total < 4 * 2 ** 30


@pytest.mark.parametrize('args, fragment', [
    ((3, 256, 4096, 8, 7168, 2048), 'multiple of num_ranks'),
    ((9, 288, 4096, 8, 7168, 2048), 'num_ranks'),
    ((1, 256, 4096, 8, 7000, 2048), 'multiples of 128'),
    ((1, 256, 0, 8, 7168, 2048), 'max tokens'),
])
def test_buffer_layout_rejects_bad_shapes(lib, args, fragment):
    words = (ctypes.c_int64 * 16)()
    rc = lib.dgb200_get_symm_buffer_layout_for_mega_moe(*args, ctypes.cast(words, ctypes.c_void_p))
    assert rc == 1
    assert fragment in lib.dgb200_last_error().decode()


def test_gemm_rejects_bad_arguments_before_touching_cuda(lib):
    null = ctypes.c_void_p(0)
    # k not a multiple of 128
    rc = lib.dgb200_m_grouped_fp8_fp4_gemm_nt_contiguous(null, null, 128, null, null, 128, 128, ctypes.c_void_p(16), 128,
                                                         null, 128, 128, 100, 1, 128, 32, 1, 0, 0, 128, 0, null)
    assert rc == 1 and 'multiple of 128' in lib.dgb200_last_error().decode()
    # unknown layout kind
    rc = lib.dgb200_m_grouped_fp8_fp4_gemm_nt_contiguous(null, null, 128, null, null, 128, 128, ctypes.c_void_p(16), 128,
                                                         null, 128, 128, 128, 1, 128, 32, 1, 0, 7, 128, 0, null)
    assert rc == 1 and 'layout kind' in lib.dgb200_last_error().decode()
    # granularity
    rc = lib.dgb200_m_grouped_fp8_fp4_gemm_nt_masked(null, null, 128, 128, null, null, 128, 128, ctypes.c_void_p(16), 128,
                                                     null, 1, 128, 128, 128, 64, 64, 32, 1, 0, null)
    assert rc == 1 and 'gran_k_a' in lib.dgb200_last_error().decode()
    rc = lib.dgb200_route_sigmoid_topk(ctypes.c_void_p(16), 4, 2048, 8, ctypes.c_void_p(16), ctypes.c_void_p(16), null)
    assert rc == 1 and 'experts' in lib.dgb200_last_error().decode()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, '_lib', None)
    monkeypatch.setattr(_lib, 'LIB_PATH', str(tmp_path / 'libdgb200.so'))
    with pytest.raises(RuntimeError, match='no CPU or PyTorch fallback'):
        _lib.lib()
