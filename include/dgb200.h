/* C ABI of libdgb200.so: the B200 (sm_100a) replacement for the Mega-MoE hot path of DeepGEMM.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (passed as void*, i.e. a
 * cudaStream_t; NULL = the legacy default stream). Nothing here names a torch type. All functions return 0 on
 * success and a non-zero DGB200_E* code on failure; dgb200_last_error() then returns a human-readable message
 * for the calling host thread. Kernels are launched asynchronously on the given stream and never synchronise
 * the host. Device-side failures (a bounded wait that ran out) never trap: they are recorded in a per-device
 * status block that dgb200_device_status() reads back.
 *
 * Reference interfaces are cited as <file>:<line> inside the DeepGEMM source tree.
 */
#ifndef DGB200_H_
#define DGB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DGB200_OK 0
#define DGB200_EINVAL 1   /* an argument the reference would reject with DG_HOST_ASSERT */
#define DGB200_ECUDA 2    /* a CUDA runtime / driver call failed */
#define DGB200_EDEVICE 3  /* the device status block holds an error */

/* Layout of the rows of A / D across groups (reference: GemmType in
 * deep_gemm/include/deep_gemm/common/types.cuh:20-28). */
#define DGB200_LAYOUT_ROW_IDS 0 /* grouped_layout[m] = group of row m, -1 = padding */
#define DGB200_LAYOUT_PSUM 1    /* grouped_layout[g] = end row of group g (use_psum_layout=True) */

const char* dgb200_last_error(void);
int dgb200_version(void);

/* Number of SMs persistent kernels are launched on (0 = all). Reference: set_num_sms / get_num_sms,
 * csrc/apis/runtime.hpp:12-20. */
int dgb200_set_num_sms(int num_sms);
int dgb200_get_num_sms(void);

/* Synchronises `stream`, copies the 8-word device status block to `out_words` (may be NULL) and clears it.
 * Returns DGB200_EDEVICE when word 0 is non-zero. Words: {code, block, detail a, detail b, 0, 0, 0, 0}.
 * Replaces the reference's device-side printf + trap (deep_gemm/include/deep_gemm/comm/barrier.cuh:36-41,
 * deep_gemm/include/deep_gemm/common/exception.cuh:15-30). */
int dgb200_device_status(int32_t* out_words, void* stream);

/* D[m, :] = A[m, :] . B[group(m)]^T over an m-grouped contiguous layout.
 * Reference: m_grouped_fp8_fp4_gemm_nt_contiguous, csrc/apis/gemm.hpp:166-232 (host) and
 * csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:161-242 (launch).
 *   a    e4m3 [m, k], row stride k bytes.
 *   sfa  int32, 4 UE8M0 bytes per int (byte j = K block 4i+j), MN-major: int (kp, row) at sfa[kp*sfa_k_stride+row].
 *   b    b_is_fp4 ? packed e2m1 [num_groups, n, k/2] (even k index in the low nibble) : e4m3 [num_groups, n, k].
 *   sfb  int32 packed UE8M0, int (g, kp, ch) at sfb[g*sfb_group_stride + kp*sfb_k_stride + ch].
 *   d    d_is_fp32 ? float [m, n] : bf16 [m, n], row stride d_row_stride elements.
 *   grouped_layout  int32, see DGB200_LAYOUT_*; `alignment` is the contiguous-layout M alignment
 *                   (get_mk_alignment_for_contiguous_layout, csrc/apis/layout.hpp:142-150), a multiple of 4.
 *   gran_k_a / gran_k_b  K elements per scale: 32 or 128 (recipe_a[1], recipe_b[1]).
 *   store_padding  psum only: also write the rows between a group's end and its aligned end
 *                  (ensure_zero_padding=True, csrc/apis/gemm.hpp:166).
 * Requires k % 128 == 0, n % 128 == 0. */
int dgb200_m_grouped_fp8_fp4_gemm_nt_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, int32_t store_padding, void* stream);

/* Masked layout: a [G, max_m, k], d [G, max_m, n], only rows < masked_m[g] of each group are computed and
 * written (stores are clipped at masked_m[g]; the reference writes whole tiles, see
 * deep_gemm/include/deep_gemm/scheduler/gemm.cuh:189-216).
 * Reference: m_grouped_fp8_fp4_gemm_nt_masked, csrc/apis/gemm.hpp:250-297 and
 * csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:244-311.
 *   sfa int (g, kp, row) at sfa[g*sfa_group_stride + kp*sfa_k_stride + row]. `expected_m` only steers tiling. */
int dgb200_m_grouped_fp8_fp4_gemm_nt_masked(
    const void* a, const void* sfa, int64_t sfa_k_stride, int64_t sfa_group_stride,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* masked_m,
    int32_t num_groups, int32_t max_m, int32_t n, int32_t k, int32_t expected_m,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* DGB200_H_ */
