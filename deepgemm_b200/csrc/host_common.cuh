// Host-side helpers shared by the C-ABI entry points: error reporting, launch attributes, tensor-map encoding.
// Counterparts in the reference: csrc/utils/exception.hpp:12-107 (DG_HOST_ASSERT / CUDA check macros),
// csrc/jit/handle.hpp:174-219 (launch config), csrc/jit_kernels/impls/runtime_utils.hpp:113-150 (tensor maps).
#pragma once
#include <algorithm>

#include <cstdarg>
#include <cstdio>
#include <string>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/dgb200.h"

namespace dgb {

inline std::string& last_error_storage() {
    static thread_local std::string s;
    return s;
}

inline int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_storage() = buf;
    return code;
}

#define DGB_REQUIRE(cond, ...)                                   \
    do {                                                         \
        if (!(cond)) return ::dgb::fail(DGB200_EINVAL, __VA_ARGS__); \
    } while (0)

#define DGB_CUDA(call)                                                                                  \
    do {                                                                                                \
        cudaError_t e_ = (call);                                                                        \
        if (e_ != cudaSuccess)                                                                          \
            return ::dgb::fail(DGB200_ECUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

inline int& num_sms_setting() {
    static int v = 0;
    return v;
}

// SM count of the current device, narrowed by dgb200_set_num_sms.
// SMs the persistent GEMM kernels of the calling host thread leave free (the expert-parallel layer keeps a few for
// the kernels that move rows over NVLink while its GEMMs run).
inline int& reserved_sms() {
    thread_local int reserved = 0;
    return reserved;
}

inline int effective_num_sms(int* out) {
    int dev = 0, sms = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    DGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int want = num_sms_setting();
    const int usable = (want > 0 && want < sms) ? want : sms;
    *out = std::max(1, usable - std::max(0, reserved_sms()));
    return 0;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &f, 12000, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// 2-D row-major tensor [outer, inner] with a 128-byte-swizzled box; `inner`/`box_inner` are in elements of `dtype`.
inline int make_tensor_map_2d(CUtensorMap* out, CUtensorMapDataType dtype, const void* base, uint64_t inner,
                              uint64_t outer, uint64_t outer_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                              CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(DGB200_ECUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {outer_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DGB200_ECUDA,
                    "cuTensorMapEncodeTiled failed with CUresult %d (dtype %d, dims %llu x %llu, stride %llu, box %u x %u)",
                    static_cast<int>(r), static_cast<int>(dtype), static_cast<unsigned long long>(inner),
                    static_cast<unsigned long long>(outer), static_cast<unsigned long long>(outer_stride_bytes),
                    box_inner, box_outer);
    return 0;
}

}  // namespace dgb
