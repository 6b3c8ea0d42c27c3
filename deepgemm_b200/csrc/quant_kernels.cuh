// HBM-bound quantisation and scale-factor layout kernels.
//
//   cast_rows_kernel<kFp4>: BF16 rows -> E4M3 (or packed E2M1) + one UE8M0 scale per `gran_k` elements, scales written
//       either as FP32 [rows, K/gran] or directly as packed int32 in the MN-major layout the GEMM consumes.
//       CUDA counterpart of the reference's torch helpers per_token_cast_to_fp8 / per_token_cast_to_fp4
//       (deep_gemm/utils/math.py:26-49, 96-122), fused with the packing the reference does in a second kernel.
//   pack_sf_kernel: FP32 power-of-two scales -> packed UE8M0 int32, MN-major, MN stride padded to 4
//       (reference: transpose_and_pack_fp32_into_ue8m0 / pack_fp32_into_ue8m0,
//        deep_gemm/include/deep_gemm/impls/smxx_layout.cuh:56-246).
//
// Tile of one CTA in cast_rows_kernel: 32 rows x 512 columns; a warp owns 4 rows, a lane 16 consecutive elements
// (two 16-byte loads, one 16-byte FP8 store or one 8-byte FP4 store). Scale bytes are staged in shared memory so that
// the packed int32 output is written as 128-byte row-contiguous segments.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "gemm_kernel.cuh"  // k_group_extent
#include "ptx.cuh"

namespace dgb {

__device__ __forceinline__ uint32_t ue8m0_ceil_bits(float x) {
    // biased exponent of the smallest power of two >= x (x > 0), clamped to [1, 254]
    const uint32_t bits = __float_as_uint(x);
    uint32_t e = (bits >> 23) & 0xffu;
    if (bits & 0x7fffffu) ++e;
    return min(max(e, 1u), 254u);
}

struct CastParams {
    const __nv_bfloat16* x;
    long long x_row_stride;  // elements
    void* q;
    long long q_row_stride;  // bytes
    float* sf_f32;           // [rows, ceil(k / gran)] row-major, or null
    uint32_t* sf_packed;     // int (kp, row) at sf_packed[kp * sf_k_stride + row * sf_row_stride], or null
    long long sf_k_stride, sf_row_stride;  // (aligned rows, 1) = MN-major for the GEMM; (1, packed k) = token-major
    int rows, k, gran_k;
};

template <bool kFp4>
__global__ void __launch_bounds__(256) dgb200_cast_rows_kernel(const CastParams p) {
    __shared__ uint8_t sf_stage[32][16];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.x * 512, row0 = blockIdx.y * 32;
    const int col = col0 + lane * 16;
    const int lanes_per_block = p.gran_k / 16;  // 2 or 8
    const float divisor = kFp4 ? 6.0f : 448.0f;
    const int num_sf = (p.k + p.gran_k - 1) / p.gran_k;

    for (int i = threadIdx.x; i < 32 * 16; i += 256) (&sf_stage[0][0])[i] = 127;  // padding scales are 1.0
    __syncthreads();

#pragma unroll 1
    for (int rr = 0; rr < 4; ++rr) {
        const int row = row0 + warp * 4 + rr;
        if (row >= p.rows) break;
        float v[16];
        if (col < p.k) {  // k % 16 == 0 is checked on the host
            const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(row) * p.x_row_stride + col);
            const uint4 r0 = ld_global_nc_v4(src), r1 = ld_global_nc_v4(src + 1);
            const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
        for (int off = 1; off < lanes_per_block; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const uint32_t e = ue8m0_ceil_bits(fmaxf(amax, 1e-4f) / divisor);
        const float inv = 1.0f / __uint_as_float(e << 23);
        if (col < p.k) {
            if constexpr (kFp4) {
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    lo |= e2m1_code(v[i] * inv) << (4 * i);
                    hi |= e2m1_code(v[8 + i] * inv) << (4 * i);
                }
                *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.q) + static_cast<long long>(row) * p.q_row_stride + col / 2) =
                    make_uint2(lo, hi);
            } else {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __nv_fp8x4_e4m3 q4(make_float4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv));
                    o[i] = q4.__x;
                }
                st_global_v4(static_cast<uint8_t*>(p.q) + static_cast<long long>(row) * p.q_row_stride + col, o[0], o[1], o[2], o[3]);
            }
            if (lane % lanes_per_block == 0) {
                const int sf_idx = col / p.gran_k;
                if (p.sf_f32 != nullptr) p.sf_f32[static_cast<long long>(row) * num_sf + sf_idx] = __uint_as_float(e << 23);
                sf_stage[warp * 4 + rr][(col - col0) / p.gran_k] = static_cast<uint8_t>(e);
            }
        }
    }
    if (p.sf_packed == nullptr) return;
    __syncthreads();
    const int ints_per_tile = 512 / p.gran_k / 4;  // 4 (gran 32) or 1 (gran 128)
    const int num_packed = (num_sf + 3) / 4;
    for (int i = threadIdx.x; i < ints_per_tile * 32; i += 256) {
        const int kp_local = i >> 5, r = i & 31;
        const int kp = col0 / (p.gran_k * 4) + kp_local;
        if (row0 + r < p.rows && kp < num_packed)
            p.sf_packed[static_cast<long long>(kp) * p.sf_k_stride + static_cast<long long>(row0 + r) * p.sf_row_stride] =
                *reinterpret_cast<const uint32_t*>(&sf_stage[r][kp_local * 4]);
    }
}

struct PackSfParams {
    const float* sf;  // element (g, r, c) at sf[g * in_stride_g + r * in_stride_mn + c * in_stride_k]
    long long in_stride_g, in_stride_mn, in_stride_k;
    uint32_t* out;  // int (g, kp, row) at out[g * packed_k * aligned_mn + kp * aligned_mn + row]
    long long aligned_mn;
    int num_groups, mn, sf_k, gran_mn;
    const int* psum_layout;  // optional: rows in the gaps between groups pack as 0
    int num_psum_groups, psum_alignment;
};

__global__ void __launch_bounds__(256) dgb200_pack_sf_kernel(const PackSfParams p) {
    const int packed_k = (p.sf_k + 3) / 4;
    const long long total = static_cast<long long>(p.num_groups) * packed_k * p.mn;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
        const int row = static_cast<int>(i % p.mn);
        const long long rest = i / p.mn;
        const int kp = static_cast<int>(rest % packed_k), g = static_cast<int>(rest / packed_k);
        bool valid = true;
        if (p.psum_layout != nullptr) {
            valid = false;
            for (int q = 0; q < p.num_psum_groups && !valid; ++q) {
                const int prev = q == 0 ? 0 : __ldg(p.psum_layout + q - 1);
                const int start = (prev + p.psum_alignment - 1) / p.psum_alignment * p.psum_alignment;
                valid = row >= start && row < __ldg(p.psum_layout + q);
            }
        }
        uint32_t packed = 0;
        if (valid) {
            const float* src = p.sf + g * p.in_stride_g + static_cast<long long>(row / p.gran_mn) * p.in_stride_mn;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = kp * 4 + j;
                if (c < p.sf_k) {
                    const uint32_t bits = __float_as_uint(__ldg(src + c * p.in_stride_k));
                    if (bits & 0x807fffffu) report_error(kBadArgument, row, c);  // not a positive power of two
                    packed |= ((bits >> 23) & 0xffu) << (8 * j);
                }
            }
        }
        p.out[(static_cast<long long>(g) * packed_k + kp) * p.aligned_mn + row] = packed;
    }
}

}  // namespace dgb

namespace dgb {

// ------------------------------------------------------------------------------------------------------------------
// NVFP4 quantisation (no reference counterpart: the reference has no NVFP4 code; format and rounding rules are stated
// in oracle/nvfp4.py): value = e2m1 * ue4m3(block of 16) * fp32 per-tensor scale.
// ------------------------------------------------------------------------------------------------------------------

// out[0] (as int bits of a non-negative float) = max(out[0], amax of this CTA's elements); out must start at 0.
__global__ void __launch_bounds__(256)
dgb200_amax_kernel(const __nv_bfloat16* __restrict__ x, long long row_stride, int rows, int k, float* out) {
    float amax = 0.0f;
    const long long vec_per_row = k / 8;
    const long long total = static_cast<long long>(rows) * vec_per_row;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
        const long long r = i / vec_per_row, c = i - r * vec_per_row;
        const uint4 v = ld_global_nc_v4(reinterpret_cast<const uint4*>(x + r * row_stride) + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            amax = fmaxf(amax, fabsf(__uint_as_float(w[j] << 16)));
            amax = fmaxf(amax, fabsf(__uint_as_float(w[j] & 0xffff0000u)));
        }
    }
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(amax));
}

// amax -> per-tensor scale amax / (6 * 448), 1 for an all-zero tensor
__global__ void dgb200_finish_tensor_scale_kernel(float* out) {
    const float amax = out[0];
    out[0] = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
}

struct CastNvfp4Params {
    const __nv_bfloat16* x;
    long long x_row_stride;     // elements
    unsigned char* q;           // packed e2m1 [rows, k / 2]
    long long q_row_stride;     // bytes
    const float* tensor_scale;  // device scalar
    uint32_t* sf_packed;        // int (kq, row) at sf_packed[kq * sf_k_stride + row * sf_row_stride]; kq = K / 64 index,
    long long sf_k_stride, sf_row_stride;  // byte j of an int = the UE4M3 scale of K block (16 elements) 4 kq + j
    int rows, k;
};

// Same tiling as dgb200_cast_rows_kernel: 32 rows x 512 columns per CTA, a lane owns 16 consecutive elements, which is
// exactly one NVFP4 block.
__global__ void __launch_bounds__(256) dgb200_cast_rows_nvfp4_kernel(const CastNvfp4Params p) {
    __shared__ uint8_t sf_stage[32][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col0 = blockIdx.x * 512, row0 = blockIdx.y * 32;
    const int col = col0 + lane * 16;
    const float s_t = __ldg(p.tensor_scale);
    for (int i = threadIdx.x; i < 32 * 32; i += 256) (&sf_stage[0][0])[i] = 0;
    __syncthreads();
#pragma unroll 1
    for (int rr = 0; rr < 4; ++rr) {
        const int row = row0 + warp * 4 + rr;
        if (row >= p.rows) break;
        if (col >= p.k) continue;
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<long long>(row) * p.x_row_stride + col);
        const uint4 r0 = ld_global_nc_v4(src), r1 = ld_global_nc_v4(src + 1);
        const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        float v[16];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
        }
        const uint32_t sf_byte = e4m3_byte(amax / 6.0f / s_t);
        const float factor = e4m3_to_float(sf_byte) * s_t;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo |= (factor > 0.0f ? e2m1_code(v[i] / factor) : 0u) << (4 * i);
            hi |= (factor > 0.0f ? e2m1_code(v[8 + i] / factor) : 0u) << (4 * i);
        }
        *reinterpret_cast<uint2*>(p.q + static_cast<long long>(row) * p.q_row_stride + col / 2) = make_uint2(lo, hi);
        sf_stage[warp * 4 + rr][lane] = static_cast<uint8_t>(sf_byte);
    }
    __syncthreads();
    const int num_packed = (p.k / 16 + 3) / 4;
    for (int i = threadIdx.x; i < 8 * 32; i += 256) {
        const int kq_local = i >> 5, r = i & 31;
        const int kq = col0 / 64 + kq_local;
        if (row0 + r < p.rows && kq < num_packed)
            p.sf_packed[static_cast<long long>(kq) * p.sf_k_stride + static_cast<long long>(row0 + r) * p.sf_row_stride] =
                *reinterpret_cast<const uint32_t*>(&sf_stage[r][kq_local * 4]);
    }
}

// Operand quantiser of the K-grouped GEMM: x bf16 [k, mn] -> e4m3 [k, mn] + one FP32 power-of-two scale per gran_k K rows
// and channel [k / gran_k, mn]: sf = 2^ceil(log2(max(amax, 1e-4) / 448)), q = e4m3_rn(x / sf). One thread owns two
// neighbouring channels of one K block (warps read 128 contiguous bytes per row); the second pass over the block's rows
// comes from L2. Reference: per_channel_cast_to_fp8(use_ue8m0=True), deep_gemm/utils/math.py:52-59 (torch ops there).
__global__ void __launch_bounds__(256)
dgb200_cast_channels_kernel(const __nv_bfloat16* __restrict__ x, int k, int mn, int gran_k, unsigned char* __restrict__ q,
                            float* __restrict__ sf) {
    const int col = (blockIdx.x * 256 + threadIdx.x) * 2;
    const int row0 = blockIdx.y * gran_k;
    if (col >= mn) return;
    const int rows = min(gran_k, k - row0);
    float amax0 = 0.0f, amax1 = 0.0f;
    for (int r = 0; r < rows; ++r) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(x + static_cast<long long>(row0 + r) * mn + col);
        amax0 = fmaxf(amax0, fabsf(__uint_as_float(w << 16)));
        amax1 = fmaxf(amax1, fabsf(__uint_as_float(w & 0xffff0000u)));
    }
    const uint32_t e0 = ue8m0_ceil_bits(fmaxf(amax0, 1e-4f) / 448.0f), e1 = ue8m0_ceil_bits(fmaxf(amax1, 1e-4f) / 448.0f);
    const float sf0 = __uint_as_float(e0 << 23), sf1 = __uint_as_float(e1 << 23);
    const float inv0 = 1.0f / sf0, inv1 = 1.0f / sf1;
    *reinterpret_cast<float2*>(sf + static_cast<long long>(blockIdx.y) * mn + col) = make_float2(sf0, sf1);
    for (int r = 0; r < rows; ++r) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(x + static_cast<long long>(row0 + r) * mn + col);
        const __nv_fp8x2_e4m3 q2(make_float2(__uint_as_float(w << 16) * inv0, __uint_as_float(w & 0xffff0000u) * inv1));
        *reinterpret_cast<unsigned short*>(q + static_cast<long long>(row0 + r) * mn + col) = q2.__x;
    }
}

// Scale factors of a K-grouped operand: FP32 powers of two [sum of ceil(k_g / gran_k) rows, mn], the groups' rows
// concatenated (the reference's tests build them per group, tests/generators.py:413-435) -> packed UE8M0 ints, every
// group starting on an int boundary: with gran_k = 128 int (j, col) of a group holds the exponent bytes of its K blocks
// 4j .. 4j+3, with gran_k = 32 those of the four 32-row scales of K block j (zero past the group's end). One block row
// per group (blockIdx.y); each block finds its group's first rows with a serial scan over the layout (at most a few
// hundred groups). Reference: transform_k_grouped_sf_into_required_layout, csrc/apis/layout.hpp (called from
// csrc/apis/gemm.hpp:335-336).
__global__ void __launch_bounds__(256)
dgb200_pack_k_grouped_sf_kernel(const float* __restrict__ sf, int sf_rows, const int* __restrict__ ks, int psum, int alignment,
                                int gran_k, int mn, long long aligned_mn, uint32_t* __restrict__ out) {
    const int g = blockIdx.y;
    int row0 = 0, kp0 = 0, prev_end = 0, start = 0, len = 0;
    for (int i = 0; i <= g; ++i) {
        if (i > 0) {
            const int rows = (len + gran_k - 1) / gran_k;
            row0 += rows;
            kp0 += (rows + 3) / 4;
        }
        k_group_extent(ks, i, psum, alignment, prev_end, start, len);
    }
    const int num_rows = (len + gran_k - 1) / gran_k;
    const int num_kp = (num_rows + 3) / 4;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < static_cast<long long>(num_kp) * mn; i += gridDim.x * 256ll) {
        const int j = static_cast<int>(i / mn), col = static_cast<int>(i - static_cast<long long>(j) * mn);
        uint32_t packed = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int r = j * 4 + b;
            if (r < num_rows && row0 + r < sf_rows)
                packed |= ((__float_as_uint(sf[static_cast<long long>(row0 + r) * mn + col]) >> 23) & 0xffu) << (8 * b);
        }
        out[static_cast<long long>(kp0 + j) * aligned_mn + col] = packed;
    }
}

}  // namespace dgb
