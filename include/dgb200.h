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

/* Process-wide tuning knobs of the GEMM kernels. Plays the role of the reference's heuristics overrides
 * (csrc/apis/runtime.hpp:21-41).
 *   "block_n"            0 = automatic, 128 or 256: width of an output tile of the tokens-on-M kernel.
 *   "swap_ab"            layer GEMMs: -1 = choose the tile orientation from the expected rows per expert (default:
 *                        swapped-operand kernel alone for decode-sized batches, experts split by size around 128
 *                        rows per expert, tokens-on-M kernel otherwise), 0 = tokens-on-M kernel only, 1 = everything
 *                        through the swapped-operand kernel including its fused SwiGLU epilogue, 2 = the size split
 *                        with every expert of up to 160 rows on the swapped side (1 and 2: testing, experiments).
 *   "fused_dispatch"     expert-parallel layer with guest experts: 0 (default) = the dispatch push is a kernel of its own;
 *                        1 or a phase count 2..4 = several expert phases, and the epilogue warps of the gate/up GEMM of
 *                        phase q also push the rows this rank routes to phase q + 1 (measured slower than the default:
 *                        the guest experts balance a rank's total rows, not its rows per phase).
 *   "fused_return"       expert-parallel layer with guest experts: 1 (default) = the down GEMM sends every output row to
 *                        the rank its token came from straight from its epilogue (GEMM and transfer in one kernel, tile by
 *                        tile); 0 = the GEMM writes its rows locally and a kernel of its own sends them afterwards.
 *   "pdl"                1 (default) = the kernels of the single-rank layer and of the GEMM entry points are launched
 *                        with programmatic stream serialization: a kernel may start while its predecessor in the
 *                        stream still runs and waits (griddepcontrol.wait) before it touches memory. 0 = plain
 *                        launches. Reference: set_pdl, csrc/apis/runtime.hpp:24-28.
 *   "ep_comm_sms"        expert-parallel layer: 0 (default) = every kernel on the caller's stream and on all SMs.
 *                        n > 0 (at most 64) = the kernels that move rows between ranks run on a second, library-owned
 *                        stream on n SMs that the GEMMs leave free, beside the GEMMs of other expert phases (measured
 *                        on B200: an SM moves about 5 GB/s over NVLink, so hiding the transfers costs more SMs than it
 *                        saves time at 4 and 8 ranks). Every rank must use the same value.
 *   "peer_wait_us"       expert-parallel layer: how long a rank waits for a flag another rank writes before it gives
 *                        up, records DGB200 status code 7 (peer timeout) and carries on (default 10 s; at least 1). */
int dgb200_set_tuning(const char* name, int32_t value);

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

/* The same GEMM with an MN-major b, the operand of the reference's m_grouped_fp8_fp4_gemm_nn_contiguous
 * (csrc/apis/gemm.hpp:234-248; on SM100 the NT form accepts an MN-major b as well, :181-183):
 *   b  b_is_fp4 ? packed e2m1 [num_groups, k, n / 2] (even n index in the low nibble) : e4m3 [num_groups, k, n],
 *      rows dense. Read through MN-major shared-memory descriptors; n must be a multiple of 32.
 * Every other argument as above (sfb stays int (g, kp, ch) at sfb[g*sfb_group_stride + kp*sfb_k_stride + ch]). */
int dgb200_m_grouped_fp8_fp4_gemm_nn_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, int32_t store_padding, void* stream);

/* Dense D = A . B^T (one group, no layout array); operands and scales as in the grouped form above. accumulate != 0
 * (float32 d only): D += A . B^T, the reference's accumulator input `c` after the caller has put c into d.
 * Reference: fp8_fp4_gemm_nt, csrc/apis/gemm.hpp:73-124. */
int dgb200_fp8_fp4_gemm_nt(const void* a, const void* sfa, int64_t sfa_k_stride, const void* b, const void* sfb,
                           int64_t sfb_k_stride, void* d, int64_t d_row_stride, int32_t m, int32_t n, int32_t k,
                           int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32, int32_t accumulate,
                           void* stream);

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

/* BF16 x BF16 forms of the three GEMMs above (tcgen05 kind::f16, FP32 accumulation, no scale factors): a and b are
 * BF16 K-major with row strides in elements (multiples of 8), d BF16 or FP32, layouts as above. Requires k % 64 == 0 and
 * n % 128 == 0. b_mn_major != 0 (contiguous and dense forms): b is [num_groups * k, n] with n contiguous, the operand
 * of the reference's "nn" forms (csrc/apis/gemm.hpp:440-446, :519-526), read through MN-major shared-memory descriptors;
 * b_row_stride is then the pitch of one K row. a_mn_major != 0 (dense form only): likewise a is [k, m] with m contiguous
 * (the "tn" / "tt" forms, csrc/apis/gemm.hpp:448-462), m % 8 == 0.
 * Reference: m_grouped_bf16_gemm_nt_contiguous csrc/apis/gemm.hpp:464-517, m_grouped_bf16_gemm_nt_masked :528-564,
 * bf16_gemm_nt :404-438 (accumulate as in dgb200_fp8_fp4_gemm_nt). */
int dgb200_m_grouped_bf16_gemm_nt_contiguous(const void* a, int64_t a_row_stride, const void* b, int64_t b_row_stride,
                                             int32_t b_mn_major, void* d, int64_t d_row_stride, const int32_t* grouped_layout, int32_t m, int32_t n,
                                             int32_t k, int32_t num_groups, int32_t d_is_fp32, int32_t layout_kind,
                                             int32_t alignment, int32_t store_padding, void* stream);
int dgb200_m_grouped_bf16_gemm_nt_masked(const void* a, const void* b, void* d, int64_t d_row_stride, const int32_t* masked_m,
                                         int32_t num_groups, int32_t max_m, int32_t n, int32_t k, int32_t expected_m,
                                         int32_t d_is_fp32, void* stream);
int dgb200_bf16_gemm_nt(const void* a, int64_t a_row_stride, int32_t a_mn_major, const void* b, int64_t b_row_stride,
                        int32_t b_mn_major, void* d, int64_t d_row_stride, int32_t m, int32_t n, int32_t k, int32_t d_is_fp32,
                        int32_t accumulate, void* stream);

/* Operand quantiser of the K-grouped GEMM: x bf16 [k, mn] contiguous -> q e4m3 [k, mn] and sf float [k / gran_k, mn], one
 * power-of-two scale per gran_k (32 or 128) K rows and channel; k % gran_k == 0, mn even.
 * Reference: per_channel_cast_to_fp8(use_ue8m0=True), deep_gemm/utils/math.py:52-59 (a torch helper there). */
int dgb200_per_channel_cast_to_fp8(const void* x, int32_t k, int32_t mn, int32_t gran_k, void* q, float* sf, void* stream);

/* K-grouped FP8 GEMM (the MoE weight gradient): for every group g, d[g] = c[g] + a[rows of g]^T . b[rows of g] with
 * a e4m3 [sum_k, m] and b e4m3 [sum_k, n] (both MN-major: the K rows of the groups one after the other), sfa float
 * [sf_rows, m] and sfb float [sf_rows, n] (one power-of-two scale per gran_k = 32 or 128 K rows of a group and channel,
 * ceil(k_g / gran_k) rows per group, groups concatenated), c and d float [num_groups, m, n] (may alias), ks int32 [num_groups] on the device:
 *   use_psum_layout = 0: ks[g] = K rows of group g, each a multiple of 128, groups packed back to back;
 *   use_psum_layout = 1: ks[g] = end K row of group g; group g starts at align(ks[g-1], k_alignment) (k_alignment a
 *                        multiple of 128) and the rows between a group's end and the next start are zero.
 * sum_k = rows of a and b (a multiple of 128). sf_workspace: dgb200_k_grouped_sf_workspace_bytes(...) bytes of device
 * scratch for the packed scales. m % 16 == 0, n % 128 == 0, num_groups <= 512. Same kernel as the m-grouped GEMMs with
 * MN-major shared-memory descriptors, per-group K extents and an accumulating FP32 epilogue.
 * Reference: k_grouped_fp8_gemm_tn_contiguous, csrc/apis/gemm.hpp:299-346 (recipes (1, 1, 128) and (1, 1, 32);
 * K alignments below 128 are not built). */
int64_t dgb200_k_grouped_sf_workspace_bytes(int32_t num_groups, int32_t m, int32_t n, int32_t sum_k);
int dgb200_k_grouped_fp8_gemm_tn_contiguous(const void* a, const float* sfa, int32_t sf_rows, const void* b, const float* sfb,
                                            const float* c, float* d, const int32_t* ks, int32_t use_psum_layout,
                                            int32_t k_alignment, int32_t gran_k, int32_t num_groups, int32_t m, int32_t n,
                                            int32_t sum_k, void* sf_workspace, void* stream);

/* BF16 form of the K-grouped GEMM: a bf16 [sum_k, m], b bf16 [sum_k, n] (MN-major), K extents / alignment multiples of
 * 64, m % 8 == 0, n % 128 == 0; c, d, ks and the two layouts as above; no scale factors, no workspace.
 * Reference: k_grouped_bf16_gemm_tn_contiguous, csrc/apis/gemm.hpp:566-608. */
int dgb200_k_grouped_bf16_gemm_tn_contiguous(const void* a, const void* b, const float* c, float* d, const int32_t* ks,
                                             int32_t use_psum_layout, int32_t k_alignment, int32_t num_groups, int32_t m,
                                             int32_t n, int32_t sum_k, void* stream);

/* BF16 rows -> E4M3 + one UE8M0 scale per gran_k (32 or 128) elements: sf = 2^ceil(log2(max(amax, 1e-4) / 448)),
 * q = e4m3_rn(x / sf). Reference: per_token_cast_to_fp8(use_ue8m0=True), deep_gemm/utils/math.py:26-49 (a torch
 * helper there; one fused kernel here).
 *   x  bf16 [rows, k], row stride x_row_stride elements; k % 16 == 0.   q  e4m3 [rows, k], row stride in bytes.
 *   sf_f32     optional float [rows, ceil(k / gran_k)] row-major.
 *   sf_packed  optional int32, 4 scales per int (missing K blocks pack as 2^0); int (kp, row) is written at
 *              sf_packed[kp * sf_k_stride + row * sf_row_stride]: (align(rows, 4), 1) gives the MN-major layout of
 *              dgb200_transform_sf_into_required_layout, (1, packed k) the token-major one of
 *              per_token_cast_to_fp8(use_packed_ue8m0=True). */
int dgb200_per_token_cast_to_fp8(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, int32_t gran_k, void* q,
                                 int64_t q_row_stride, float* sf_f32, void* sf_packed, int64_t sf_k_stride,
                                 int64_t sf_row_stride, void* stream);

/* BF16 rows -> packed E2M1 (two codes per byte, even K index in the low nibble) + UE8M0 scales:
 * sf = 2^ceil(log2(max(amax, 1e-4) / 6)); thresholds .25 .75 1.25 1.75 2.5 3.5 5 with ties rounding down.
 * Reference: per_token_cast_to_fp4(use_ue8m0=True), deep_gemm/utils/math.py:84-122.  q int8 [rows, k / 2]. */
int dgb200_per_token_cast_to_fp4(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, int32_t gran_k, void* q,
                                 int64_t q_row_stride, float* sf_f32, void* sf_packed, int64_t sf_k_stride,
                                 int64_t sf_row_stride, void* stream);

/* FP32 power-of-two scales -> packed UE8M0 int32, MN-major, MN stride align(mn, 4):
 * out[g * packed_k * align(mn, 4) + kp * align(mn, 4) + row], byte j of an int = K block 4 kp + j.
 * Reference: transform_sf_into_required_layout, csrc/apis/layout.hpp:14-61 ->
 * get_mn_major_tma_aligned_packed_ue8m0_tensor, csrc/jit_kernels/impls/smxx_layout.hpp:180-253.
 *   sf element (g, r, c) at sf[g * stride_g + r * stride_mn + c * stride_k]; row r of the output reads input row
 *   r / gran_mn. psum_layout (optional, device int32 [num_psum_groups]): rows that fall in the gap between one
 *   group's end and the next group's aligned start pack as 0 instead of being read. A scale that is not a positive
 *   power of two sets the device status (the reference traps). */
int dgb200_transform_sf_into_required_layout(const float* sf, int64_t stride_g, int64_t stride_mn, int64_t stride_k,
                                             void* out, int32_t num_groups, int32_t mn, int32_t sf_k, int32_t gran_mn,
                                             const int32_t* psum_layout, int32_t num_psum_groups,
                                             int32_t psum_alignment, void* stream);

/* ---- NVFP4 variant (packed E2M1, one UE4M3 scale per 16 elements, one FP32 scale per tensor). The reference has no
 * NVFP4 code; these entry points have no counterpart there. Format and rounding: oracle/nvfp4.py.
 * Packed scale layout: int32, byte j of int (kq, row) = scale of the 16-element K block 4 kq + j. */

/* out_scale[0] = amax(x) / (6 * 448) (1.0 for an all-zero tensor): the per-tensor scale of the quantiser below. */
int dgb200_nvfp4_tensor_scale(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, float* out_scale, void* stream);

/* BF16 rows -> packed E2M1 [rows, k/2] + UE4M3 block scales: sf = e4m3_rn(amax16 / 6 / tensor_scale), saturating at 448;
 * codes of x / (float(sf) * tensor_scale) with the E2M1 thresholds of dgb200_per_token_cast_to_fp4. k % 64 == 0.
 * sf_packed strides as in dgb200_per_token_cast_to_fp8 ((align(rows, 4), 1) = MN-major for the GEMM). */
int dgb200_per_token_cast_to_nvfp4(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, const float* tensor_scale,
                                   void* q, int64_t q_row_stride, void* sf_packed, int64_t sf_k_stride,
                                   int64_t sf_row_stride, void* stream);

/* D[m, :] = a_scale[0] * b_scales[group(m)] * (A[m, :] . B[group(m)]^T with block scales), FP4 x FP4
 * (tcgen05 kind::mxf4nvf4, scale_vec::4X). a packed e2m1 [m, k/2]; b packed e2m1 [G, n, k/2]; sfa / sfb packed UE4M3
 * int32 MN-major ([k/64][align(m,4)] and [G][k/64][align(n,4)]); a_scale, b_scales device floats. k % 256 == 0. */
int dgb200_m_grouped_nvfp4_gemm_nt_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride, const float* a_scale,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride, const float* b_scales,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, void* stream);

/* Router used by the benchmark layer: top-k of the logits (descending, ties to the lower expert index), weights =
 * sigmoid(logit) renormalised to sum to one. No reference counterpart (its tests call torch.topk,
 * tests/test_mega_moe.py:124-125).  logits float [tokens, experts]; topk_idx int64, topk_weights float [tokens, topk]. */
int dgb200_route_sigmoid_topk(const float* logits, int32_t tokens, int32_t experts, int32_t topk, int64_t* topk_idx,
                              float* topk_weights, void* stream);

/* Token-count granularity of the mega-MoE buffer. Reference: get_token_alignment_for_mega_moe, csrc/apis/mega.hpp:19-21. */
int dgb200_get_token_alignment_for_mega_moe(void);

/* Rows every expert's segment is padded to in the expert-sorted buffers (dest_row / expert_start / expert_end follow
 * it). No reference counterpart: the reference sizes its pools by block_m tiles (csrc/apis/mega.hpp:34-80). */
int dgb200_get_segment_alignment_for_mega_moe(void);

/* Rows of one gate/up interleave block of the FP8 x MXFP4 layer's L1 weights: the rows of l1_w (and of its scale
 * factors) must be ordered [gate 0..g-1 | up 0..g-1 | gate g..2g-1 | ...] with g = this value (16 for the fused
 * expert-MLP kernel, 128 for the separate gate/up and down kernels; fixed for the life of the process).
 * Reference: _interleave_weights (granularity 8), deep_gemm/mega/__init__.py:97-111. */
int dgb200_get_gate_up_interleave_for_mega_moe(void);

/* Rows of one weight tile of the FP8 x MXFP4 layer, or 0 for plain row-major weights. With r > 0 the packed E2M1 bytes
 * of l1_w and l2_w must be stored as contiguous tiles of r rows x 128 K elements (r x 64 bytes), in the order (expert,
 * r-row block, K block): byte (e, n, kb, c) of the row-major [E_local, N, K / 2] tensor (kb = K block of 64 bytes,
 * c < 64) moves to offset (((e * N / r + n / r) * (K / 128) + kb) * r + n % r) * 64 + c. The fused expert-MLP kernel
 * reads a tile as one TMA box and asks for it ahead of time with one bulk L2 prefetch. No reference counterpart. */
int dgb200_get_weight_tile_rows_for_mega_moe(void);

/* Byte layout of the per-rank mega-MoE buffer. Reference: get_symm_buffer_size_for_mega_moe, csrc/apis/mega.hpp:34-155.
 * out[16] = {total bytes, x, x_sf, topk_idx, topk_weights, l1_acts, l1_sf, l2_acts, l2_sf, max_rows (rows, not bytes),
 *            dest_row, src_of_row, expert_start, expert_end, l2_out, row_weight}; all but out[0], out[9] are byte
 * offsets. The caller writes x (e4m3 [T, hidden]), x_sf (int32 [T, hidden / 128], per-32 UE8M0, token-major),
 * topk_idx (int64 [T, topk], -1 = masked) and topk_weights (float [T, topk]) before each call; the rest is private. */
int dgb200_get_symm_buffer_layout_for_mega_moe(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                               int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                               int64_t* out);

/* The MoE layer: dispatch -> L1 (gate/up GEMM + SwiGLU + FP8 requant) -> L2 (down GEMM) -> weighted top-k combine.
 * Reference: fp8_fp4_mega_moe, csrc/apis/mega.hpp:157-286 (host) and
 * deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:55-1458 (kernel).
 *   y        bf16 [num_tokens, hidden], written.
 *   l1_w     packed e2m1 [E_local, 2 * inter, hidden / 2], rows gate/up-interleaved in blocks of
 *            dgb200_get_gate_up_interleave_for_mega_moe() rows, bytes tiled as dgb200_get_weight_tile_rows_for_mega_moe() says;
 *   l1_w_sf  packed UE8M0 int32 (per-32), MN-major [E_local][hidden / 128][2 * inter], same row order, then every
 *            aligned group of 128 rows stored in tcgen05.cp order: row r of a group at position 4 (r % 32) + r / 32.
 *   l2_w     packed e2m1 [E_local, hidden, inter / 2]; l2_w_sf int32 [E_local][inter / 128][hidden], rows in the
 *            same 128-group order.
 *   cumulative_local_expert_recv_stats  optional int32 [E_local], incremented by the rows each expert received.
 *   buffer / peer_buffer_ptrs  this rank's buffer and the host array of all ranks' buffer addresses.
 *   activation_clamp <= 0 disables the clamp. */
int dgb200_fp8_fp4_mega_moe(void* y, const void* l1_w, const void* l1_w_sf, const void* l2_w, const void* l2_w_sf,
                            int32_t* cumulative_local_expert_recv_stats, void* buffer, const uint64_t* peer_buffer_ptrs,
                            int32_t rank, int32_t num_ranks, int32_t num_tokens, int32_t num_max_tokens_per_rank,
                            int32_t num_experts, int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                            float activation_clamp, int32_t fast_math, void* stream);

/* The same layer with the two steps the reference leaves to its caller (README.md:72: quantise x with
 * per_token_cast_to_fp8 into the buffer; tests/test_mega_moe.py:124-125: route with torch.topk) fused into its
 * prologue: x is BF16 [num_tokens, hidden] (row stride in elements) and is quantised (E4M3, UE8M0 per 32) while it is
 * dispatched, so the buffer's x / x_sf views are not used; with `logits` (float [num_tokens, num_experts], may be
 * NULL) the sigmoid / top-k / renormalise router fills topk_idx and topk_weights first. Results are bit-identical to
 * dgb200_per_token_cast_to_fp8 (gran 32) + dgb200_route_sigmoid_topk + dgb200_fp8_fp4_mega_moe. */
int dgb200_fp8_fp4_mega_moe_bf16_input(void* y, const void* x, int64_t x_row_stride, const float* logits, const void* l1_w,
                                       const void* l1_w_sf, const void* l2_w, const void* l2_w_sf,
                                       int32_t* cumulative_local_expert_recv_stats, void* buffer,
                                       const uint64_t* peer_buffer_ptrs, int32_t rank, int32_t num_ranks, int32_t num_tokens,
                                       int32_t num_max_tokens_per_rank, int32_t num_experts, int32_t num_topk, int32_t hidden,
                                       int32_t intermediate_hidden, float activation_clamp, int32_t fast_math, void* stream);

/* Every option of the FP8 x MXFP4 layer in one call: the arguments of dgb200_fp8_fp4_mega_moe, the fused prologue of
 * dgb200_fp8_fp4_mega_moe_bf16_input (x_bf16 / logits, NULL = not used), and shared experts.
 * Shared experts (reference: shared_l1_weights / shared_l2_weights of fp8_fp4_mega_moe, csrc/apis/mega.hpp:161-232, and
 * the SharedLinear1/2 tasks of the fused kernel, ...mega_moe.cuh:769-778,1275-1278): a dense FP8 x FP8 MLP applied to
 * every token of this rank, its BF16 output row added to the token's combine after the top-k slots.
 *   shared_l1_w e4m3 [2 * shared_inter, hidden] (rows gate/up-interleaved by 128), shared_l1_w_sf packed UE8M0 int32
 *   (per-32), MN-major [hidden / 128][2 * shared_inter], 128-row groups in tcgen05.cp order; shared_l2_w e4m3
 *   [hidden, shared_inter], shared_l2_w_sf [shared_inter / 128][hidden]. shared_intermediate_hidden = 0: none.
 * The buffer must have been sized with dgb200_get_symm_buffer_layout_for_mega_moe_ex and the same shared size; the
 * token capacity must then be a multiple of 128. struct_size = sizeof(dgb200_mega_moe_args). */
typedef struct dgb200_mega_moe_args {
    size_t struct_size;
    void* y;
    const void* l1_w;
    const void* l1_w_sf;
    const void* l2_w;
    const void* l2_w_sf;
    const void* shared_l1_w;
    const void* shared_l1_w_sf;
    const void* shared_l2_w;
    const void* shared_l2_w_sf;
    const void* x_bf16;
    const float* logits;
    int32_t* cumulative_local_expert_recv_stats;
    void* buffer;
    const uint64_t* peer_buffer_ptrs;
    int64_t x_bf16_row_stride;
    int32_t shared_intermediate_hidden;
    int32_t rank, num_ranks, num_tokens, num_max_tokens_per_rank, num_experts, num_topk, hidden, intermediate_hidden;
    float activation_clamp;
    int32_t fast_math;
    /* Hot-expert row spill, expert-parallel runs only (num_guest_experts = 0: every expert's rows stay on its owner).
     * With skewed routing the rank that owns the popular experts receives several times the mean number of rows and
     * all ranks wait for it. With num_guest_experts = G > 0 (at most 8) every rank derives, from the exchanged
     * per-expert counts, the same plan that moves the rows some source ranks route to a hot expert onto a less loaded
     * rank; that rank computes them in one of its G guest slots with a copy of the expert's weights, which it fetches
     * from the owner during the call. A row's arithmetic does not depend on the rank that computes it; outputs can
     * differ from a run without the spill only where the layer picks another tile orientation for an expert whose row
     * count changed, i.e. in the last bits of FP32 sums. Requirements: l1_w, l1_w_sf,
     * l2_w, l2_w_sf of EVERY rank hold E_local + G experts (the guest slots, after the rank's own experts, are scratch
     * of the library) and are mapped into every process; peer_l1_w[r] ... peer_l2_w_sf[r] are the addresses of rank
     * r's four tensors in this process (host arrays of num_ranks entries; entry `rank` must equal l1_w ... l2_w_sf).
     * Every rank must pass the same G. No reference counterpart (the reference keeps an expert's rows on its owner). */
    int32_t num_guest_experts;
    const uint64_t* peer_l1_w;
    const uint64_t* peer_l1_w_sf;
    const uint64_t* peer_l2_w;
    const uint64_t* peer_l2_w_sf;
} dgb200_mega_moe_args;
int dgb200_fp8_fp4_mega_moe_ex(const dgb200_mega_moe_args* args, void* stream);

/* dgb200_get_symm_buffer_layout_for_mega_moe with room for shared experts: out[26] = the 16 words above, then the byte
 * offsets of the shared experts' private regions (x scales in GEMM order, activations, their scales, output rows) and,
 * last, of the cross-rank flag words (int32 [13][8]: rows 0..8 = flag rows, slot s = the epoch rank s last signalled:
 * row 0 counts published, rows 1..4 dispatch phases, rows 5..8 output phases; rows 9..12 = this rank's own counts of
 * signals sent and waits completed per flag row), then five more private regions of the expert-parallel plan:
 * my_base, my_dest, my_slot (int32 [num_experts] each: first row, computing rank and expert slot there of this
 * rank's entries per expert; my_dest / my_slot are written only with guest experts), guest_expert (int32 [8]: the
 * experts this rank hosts, -1 = unused) and rank_rows (int32 [2][num_ranks]: every rank's rows before and after the
 * spill). expert_start / expert_end hold E_local entries, plus 8 guest slots when num_ranks > 1. The whole buffer must be zeroed once after it is allocated, on every
 * rank and before any rank's first call (the flag words are never reset afterwards; everything else is rewritten by
 * each call before it is read). */
int dgb200_get_symm_buffer_layout_for_mega_moe_ex(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                                  int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                                  int32_t shared_intermediate_hidden, int64_t* out);

/* BF16 x BF16 form of the layer. Buffer layout: same out[16] fields as dgb200_get_symm_buffer_layout_for_mega_moe; the
 * caller writes x (bf16 [T, hidden]); the scale-factor regions are empty. Stages as in dgb200_fp8_fp4_mega_moe with BF16
 * rows throughout: l1_w bf16 [E_local, 2 * inter, hidden] (gate/up interleaved by 128), l2_w bf16 [E_local, hidden, inter];
 * the gate/up GEMM's epilogue writes silu(gate) * up * topk_weight as BF16. hidden and inter must be multiples of 128.
 * Shared experts (shared_intermediate_hidden > 0): shared_l1_w bf16 [2 * shared_inter, hidden] (interleaved likewise),
 * shared_l2_w bf16 [hidden, shared_inter], a dense MLP over this rank's tokens with routing weight 1 whose rows are one
 * more combine slot; the token capacity must then be a multiple of 128. out[26] as in
 * dgb200_get_symm_buffer_layout_for_mega_moe_ex.
 * Reference: bf16_mega_moe, csrc/apis/mega.hpp:288-400 and deep_gemm/include/deep_gemm/impls/sm100_bf16_mega_moe.cuh:52. */
int dgb200_get_symm_buffer_layout_for_bf16_mega_moe(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                                    int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                                    int32_t shared_intermediate_hidden, int64_t* out);
int dgb200_bf16_mega_moe(void* y, const void* l1_w, const void* l2_w, const void* shared_l1_w, const void* shared_l2_w,
                         int32_t shared_intermediate_hidden, int32_t* cumulative_local_expert_recv_stats, void* buffer,
                         const uint64_t* peer_buffer_ptrs, int32_t rank, int32_t num_ranks, int32_t num_tokens,
                         int32_t num_max_tokens_per_rank, int32_t num_experts, int32_t num_topk, int32_t hidden,
                         int32_t intermediate_hidden, float activation_clamp, int32_t fast_math, void* stream);

/* NVFP4 x NVFP4 form of the layer (no reference counterpart; the reference's layer is FP8 x MXFP4 only).
 * Buffer layout: same out[16] fields as dgb200_get_symm_buffer_layout_for_mega_moe; the caller writes
 * x (packed e2m1 [T, hidden / 2]) and x_sf (int32 [T, hidden / 64], four UE4M3 bytes per int, token-major).
 * hidden and intermediate_hidden must be multiples of 256. */
int dgb200_get_symm_buffer_layout_for_nvfp4_mega_moe(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                                     int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                                     int64_t* out);

/* Same stages and argument meaning as dgb200_fp8_fp4_mega_moe with NVFP4 tensors:
 *   l1_w packed e2m1 [E_local, 2 * inter, hidden / 2] (gate/up interleaved by 128), l1_w_sf packed UE4M3 int32
 *   MN-major [E_local][hidden / 64][2 * inter], l1_w_scales float [E_local]; l2_w [E_local, hidden, inter / 2],
 *   l2_w_sf [E_local][inter / 64][hidden], l2_w_scales float [E_local]; scale rows in the 128-group order above.
 *   x_scale   device float: per-tensor scale the caller quantised x with; must hold the same value on every rank
 *             (a calibrated input scale), because an expert's rows come from all ranks.
 *   act_scale device float: calibrated per-tensor scale of the post-SwiGLU activations; the L1 epilogue quantises
 *             against it (block scales saturate at 448) and the L2 GEMM multiplies by it. */
int dgb200_nvfp4_mega_moe(void* y, const void* l1_w, const void* l1_w_sf, const float* l1_w_scales, const void* l2_w,
                          const void* l2_w_sf, const float* l2_w_scales, const float* x_scale, const float* act_scale,
                          int32_t* cumulative_local_expert_recv_stats, void* buffer, const uint64_t* peer_buffer_ptrs,
                          int32_t rank, int32_t num_ranks, int32_t num_tokens, int32_t num_max_tokens_per_rank,
                          int32_t num_experts, int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                          float activation_clamp, int32_t fast_math, void* stream);

/* The expert-parallel dispatch plan with guest experts (hot-expert row spill, see dgb200_mega_moe_args) as rank `rank`
 * derives it inside the layer call, as a call of its own: for schedulers that want to know where rows will be computed
 * before they launch the layer, and for tests. No reference counterpart. All pointers are device memory.
 *   all_counts    int32 [num_ranks, num_experts]: entries that source rank s routes to expert e
 *   my_base, my_dest, my_slot  int32 [num_experts]: first row, computing rank and expert slot there of rank `rank`'s
 *                 entries for each expert (slots 0 .. E_local - 1 = the computing rank's own experts, then guest slots)
 *   slot_start, slot_end  int32 [E_local + num_guest_experts]: the row segments of rank `rank`'s own slots, each
 *                 starting at a multiple of `alignment`; inside a slot rows are ordered by (source rank, entry)
 *   guest_expert  int32 [num_guest_experts]: the experts rank `rank` hosts, -1 = unused
 *   rank_rows     int32 [2 * num_ranks + 1]: every rank's rows as routed, every rank's rows as computed, and rank
 *                 `rank`'s padded row total
 * num_ranks <= 8, num_guest_experts <= 8, E_local + num_guest_experts <= 255, num_ranks * num_experts <= 5120. */
int dgb200_ep_plan_with_guest_experts(const int32_t* all_counts, int32_t num_ranks, int32_t num_experts, int32_t rank,
                                      int32_t alignment, int32_t num_guest_experts, int32_t* my_base, int32_t* my_dest,
                                      int32_t* my_slot, int32_t* slot_start, int32_t* slot_end, int32_t* guest_expert,
                                      int32_t* rank_rows, void* stream);

/* dgb200_nvfp4_mega_moe on a single rank with its prologue fused in (no reference counterpart): x is BF16 [num_tokens,
 * hidden] (row stride in elements) and is quantised to NVFP4 against x_scale while it is dispatched, so the buffer's
 * x / x_sf views are not used; with `logits` (float [num_tokens, num_experts], may be NULL) the sigmoid / top-k /
 * renormalise router fills topk_idx and topk_weights first. Results are bit-identical to dgb200_per_token_cast_to_nvfp4 +
 * dgb200_route_sigmoid_topk + dgb200_nvfp4_mega_moe. The buffer is the one of
 * dgb200_get_symm_buffer_layout_for_nvfp4_mega_moe with num_ranks = 1. */
int dgb200_nvfp4_mega_moe_bf16_input(void* y, const void* x, int64_t x_row_stride, const float* logits, const void* l1_w,
                                     const void* l1_w_sf, const float* l1_w_scales, const void* l2_w, const void* l2_w_sf,
                                     const float* l2_w_scales, const float* x_scale, const float* act_scale,
                                     int32_t* cumulative_local_expert_recv_stats, void* buffer, int32_t num_tokens,
                                     int32_t num_max_tokens_per_rank, int32_t num_experts, int32_t num_topk, int32_t hidden,
                                     int32_t intermediate_hidden, float activation_clamp, int32_t fast_math, void* stream);

/* Dispatch plan for callers that cannot allocate device memory. It has no counterpart in the reference.
 * Some hosts of this library run it from places where cudaMalloc is off limits: inside a region whose memory is
 * owned by another allocator with a fixed pool, in a callback that must not synchronise the device, or in a service
 * that forbids allocation after start-up. For them this entry point computes the layer's dispatch permutation
 * (the stable sort of the (token, k) entries by expert that dgb200_fp8_fp4_mega_moe builds inside its buffer) using
 * a scratch array that is part of the library image instead of a caller buffer. It calls no cudaMalloc / cudaFree and
 * no allocating library routine; inputs and outputs are the caller's.
 *   topk_idx      int64 [num_tokens, num_topk], -1 = masked slot
 *   dest_row      int32 [num_tokens * num_topk]   row of each entry in expert-sorted order, -1 for masked slots
 *   expert_start  int32 [num_experts]             first row of each expert (multiples of `alignment`)
 *   expert_end    int32 [num_experts]             one past the last row of each expert
 * Limits: num_tokens * num_topk <= 65536 and num_experts <= 512 (about 129 KB of device memory per GPU, held from
 * library load to process exit); larger problems are rejected with DGB200_EINVAL.
 * The first call on a device looks up the scratch array's device address (cudaGetSymbolAddress): make that first
 * call outside any stream capture. All calls on a device share the one scratch array: it keeps whatever the last
 * call left (every word a call reads it has written first, so nothing needs clearing), and two calls that overlap
 * on the GPU (different streams, no ordering) race on it. */
int dgb200_moe_dispatch_plan_noalloc(const int64_t* topk_idx, int32_t num_tokens, int32_t num_topk, int32_t num_experts,
                                     int32_t alignment, int32_t* dest_row, int32_t* expert_start, int32_t* expert_end,
                                     void* stream);

/* Measurement hook: the NEXT dgb200_fp8_fp4_mega_moe call of this host thread records events[i] (cudaEvent_t
 * handles) on its stream at stage boundary i: 0 entry, 1 after the dispatch plan, 2 after the gather, 3 after L1,
 * 4 after L2, 5 after the combine. The setting is consumed by that call. No reference counterpart (the reference
 * times its kernel from outside with kineto, deep_gemm/testing/bench.py:79-146). */
int dgb200_set_mega_moe_stage_events(void* const* events, int32_t count);

#ifdef __cplusplus
}
#endif

#endif /* DGB200_H_ */
