"""ctypes binding of libdgb200.so (the C ABI declared in include/dgb200.h).

The reference binds its host layer with pybind11 (csrc/python_api.cpp:17-28); here the boundary is a plain
C ABI, so the same library can be bound from any host language. There is no CPU fallback: if the shared
object is missing or fails to load, importing an operator raises.
"""
import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, 'libdgb200.so')

_lib = None

_i32, _i64, _ptr = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p

# name -> argtypes; every function returns int except where noted below
_SIGNATURES = {
    'dgb200_version': [],
    'dgb200_set_num_sms': [ctypes.c_int],
    'dgb200_get_num_sms': [],
    'dgb200_set_tuning': [ctypes.c_char_p, _i32],
    'dgb200_device_status': [_ptr, _ptr],
    'dgb200_m_grouped_fp8_fp4_gemm_nt_contiguous': [
        _ptr, _ptr, _i64, _ptr, _ptr, _i64, _i64, _ptr, _i64, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_m_grouped_fp8_fp4_gemm_nn_contiguous': [
        _ptr, _ptr, _i64, _ptr, _ptr, _i64, _i64, _ptr, _i64, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_m_grouped_fp8_fp4_gemm_nt_masked': [
        _ptr, _ptr, _i64, _i64, _ptr, _ptr, _i64, _i64, _ptr, _i64, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_per_token_cast_to_fp8': [_ptr, _i64, _i32, _i32, _i32, _ptr, _i64, _ptr, _ptr, _i64, _i64, _ptr],
    'dgb200_per_token_cast_to_fp4': [_ptr, _i64, _i32, _i32, _i32, _ptr, _i64, _ptr, _ptr, _i64, _i64, _ptr],
    'dgb200_transform_sf_into_required_layout': [
        _ptr, _i64, _i64, _i64, _ptr, _i32, _i32, _i32, _i32, _ptr, _i32, _i32, _ptr],
    'dgb200_nvfp4_tensor_scale': [_ptr, _i64, _i32, _i32, _ptr, _ptr],
    'dgb200_per_token_cast_to_nvfp4': [_ptr, _i64, _i32, _i32, _ptr, _ptr, _i64, _ptr, _i64, _i64, _ptr],
    'dgb200_m_grouped_nvfp4_gemm_nt_contiguous': [
        _ptr, _ptr, _i64, _ptr, _ptr, _ptr, _i64, _i64, _ptr, _ptr, _i64, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_route_sigmoid_topk': [_ptr, _i32, _i32, _i32, _ptr, _ptr, _ptr],
    'dgb200_get_token_alignment_for_mega_moe': [],
    'dgb200_m_grouped_bf16_gemm_nt_contiguous': [_ptr, _i64, _ptr, _i64, _i32, _ptr, _i64, _ptr, _i32, _i32, _i32, _i32, _i32,
                                                 _i32, _i32, _i32, _ptr],
    'dgb200_m_grouped_bf16_gemm_nt_masked': [_ptr, _ptr, _ptr, _i64, _ptr, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_bf16_gemm_nt': [_ptr, _i64, _i32, _ptr, _i64, _i32, _ptr, _i64, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_k_grouped_bf16_gemm_tn_contiguous': [_ptr, _ptr, _ptr, _ptr, _ptr, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_per_channel_cast_to_fp8': [_ptr, _i32, _i32, _i32, _ptr, _ptr, _ptr],
    'dgb200_k_grouped_sf_workspace_bytes': [_i32, _i32, _i32, _i32],
    'dgb200_k_grouped_fp8_gemm_tn_contiguous': [_ptr, _ptr, _i32, _ptr, _ptr, _ptr, _ptr, _ptr, _i32, _i32, _i32, _i32, _i32, _i32,
                                                _i32, _ptr, _ptr],
    'dgb200_fp8_fp4_gemm_nt': [_ptr, _ptr, _i64, _ptr, _ptr, _i64, _ptr, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_get_segment_alignment_for_mega_moe': [],
    'dgb200_get_gate_up_interleave_for_mega_moe': [],
    'dgb200_get_weight_tile_rows_for_mega_moe': [],
    'dgb200_get_symm_buffer_layout_for_mega_moe': [_i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_get_symm_buffer_layout_for_nvfp4_mega_moe': [_i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_fp8_fp4_mega_moe_bf16_input': [
        _ptr, _ptr, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, ctypes.c_float, _i32, _ptr],
    'dgb200_get_symm_buffer_layout_for_mega_moe_ex': [_i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_fp8_fp4_mega_moe_ex': [_ptr, _ptr],
    'dgb200_nvfp4_mega_moe': [
        _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, ctypes.c_float, _i32, _ptr],
    'dgb200_nvfp4_mega_moe_bf16_input': [
        _ptr, _ptr, _i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, ctypes.c_float, _i32, _ptr],
    'dgb200_get_symm_buffer_layout_for_bf16_mega_moe': [_i32, _i32, _i32, _i32, _i32, _i32, _i32, _ptr],
    'dgb200_bf16_mega_moe': [_ptr, _ptr, _ptr, _ptr, _ptr, _i32, _ptr, _ptr, _ptr, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                             _i32, ctypes.c_float, _i32, _ptr],
    'dgb200_moe_dispatch_plan_noalloc': [_ptr, _i32, _i32, _i32, _i32, _ptr, _ptr, _ptr, _ptr],
    'dgb200_set_mega_moe_stage_events': [_ptr, _i32],
    'dgb200_ep_plan_with_guest_experts': [_ptr, _i32, _i32, _i32, _i32, _i32, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr],
    'dgb200_fp8_fp4_mega_moe': [
        _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
        _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, ctypes.c_float, _i32, _ptr],
}


class MegaMoeArgs(ctypes.Structure):
    """dgb200_mega_moe_args of include/dgb200.h, field for field."""
    _fields_ = [('struct_size', ctypes.c_size_t)] + \
        [(n, ctypes.c_void_p) for n in ('y', 'l1_w', 'l1_w_sf', 'l2_w', 'l2_w_sf', 'shared_l1_w', 'shared_l1_w_sf', 'shared_l2_w',
                                        'shared_l2_w_sf', 'x_bf16', 'logits', 'cumulative_local_expert_recv_stats', 'buffer',
                                        'peer_buffer_ptrs')] + \
        [('x_bf16_row_stride', ctypes.c_int64), ('shared_intermediate_hidden', ctypes.c_int32)] + \
        [(n, ctypes.c_int32) for n in ('rank', 'num_ranks', 'num_tokens', 'num_max_tokens_per_rank', 'num_experts', 'num_topk',
                                       'hidden', 'intermediate_hidden')] + \
        [('activation_clamp', ctypes.c_float), ('fast_math', ctypes.c_int32), ('num_guest_experts', ctypes.c_int32)] + \
        [(n, ctypes.c_void_p) for n in ('peer_l1_w', 'peer_l1_w_sf', 'peer_l2_w', 'peer_l2_w_sf')]


def exported_symbols():
    """Names of every entry point this binding expects the library to export."""
    return ['dgb200_last_error'] + sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Loads the library on first use. Raises if it has not been built (``python -m deepgemm_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f'{LIB_PATH} is missing: build it with `python -m deepgemm_b200.build` (needs nvcc). '
                'deepgemm_b200 has no CPU or PyTorch fallback.')
        handle = ctypes.CDLL(LIB_PATH)
        handle.dgb200_last_error.restype = ctypes.c_char_p
        handle.dgb200_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int64 if name == 'dgb200_k_grouped_sf_workspace_bytes' else ctypes.c_int
        _lib = handle
    return _lib


def check(rc: int) -> None:
    """Raises RuntimeError with the library's message, as the reference's DGException surfaces in Python
    (csrc/utils/exception.hpp:12-23)."""
    if rc != 0:
        raise RuntimeError(lib().dgb200_last_error().decode())


def current_stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def device_status(raise_on_error: bool = True):
    """Synchronises the current stream and returns the 8 status words; raises if a kernel reported a failure."""
    words = (ctypes.c_int32 * 8)()
    rc = lib().dgb200_device_status(ctypes.cast(words, ctypes.c_void_p), current_stream_ptr())
    if rc != 0 and raise_on_error:
        check(rc)
    return list(words)
