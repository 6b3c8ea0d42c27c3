// Persistent, warp-specialised m-grouped GEMM for sm_100a:
//   D[m, :] = A[m, :] . B[group(m)]^T,  A = E4M3 activations, B = packed E2M1 (MXFP4) or E4M3 weights,
//   UE8M0 block scales applied inside tcgen05.mma (kind::mxf8f6f4.block_scale), FP32 accumulation in TMEM.
//
// Replaces, for the m-grouped contiguous / psum / masked layouts, the reference kernel
// deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_gemm_1d1d.cuh:33-534 together with its scheduler
// (deep_gemm/include/deep_gemm/scheduler/gemm.cuh:39-325) and epilogue
// (deep_gemm/include/deep_gemm/epilogue/sm100_store_cd_swap_ab.cuh:23-142).
//
// Design differences from the reference (it is not a translation):
//   * Tokens sit on the UMMA M side (TMEM lanes), weight channels on the N side (TMEM columns). One epilogue
//     thread therefore owns one token row: stores are row-contiguous 16-byte vectors straight from registers,
//     and the SwiGLU / amax / requant epilogue needs no shuffles or shared-memory exchange.
//   * Scale factors arrive through their own tensor maps, 512 B per 128 rows per packed scale int; when the caller
//     stores them in tcgen05.cp row order (the MoE layer does) they go from shared to tensor memory untouched.
//   * Stores are clipped to the valid rows of a group, so a masked group never writes into its neighbour.
//   * Every wait is bounded; a timeout unwinds the CTA and is reported through the status block.
//
// Other forms of the same kernel (template parameters):
//   * kKindNvfp4: packed E2M1 x packed E2M1 with UE4M3 scales per 16 and FP32 tensor scales (kind::mxf4nvf4).
//   * kKindBf16: BF16 x BF16 without scales (kind::f16), the reference's BF16 GEMM family
//     (deep_gemm/include/deep_gemm/impls/sm100_bf16_gemm.cuh) and the BF16 layer's GEMMs.
//   * kEpiF32Acc: the K-grouped GEMM d[g] = c[g] + A_g^T B_g with MN-major operands (FP8 with per-channel scales, or
//     BF16); replaces the reference's K-grouped use of its 1d1d kernels (scheduler/gemm.cuh:238-261).
//
// Warp roles (384 threads): warp 0 loads A tiles and their scale factors, warp 3 the weight tiles and theirs, warp 1
// issues the MMAs, warp 2 allocates TMEM and (only for scale factors in plain row order) transposes them for tcgen05.cp,
// warps 4-11 are the epilogue (TMEM lane quarter = warp index % 4, two warps per quarter splitting the columns).
// The control warpgroup hands registers to the epilogue warpgroups with setmaxnreg.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace dgb {

enum GroupMode : int {
    kModeRowIds = 0,  // layout[m] = group of row m, -1 on padding rows (segments aligned to `alignment`)
    kModePsum = 1,    // layout[g] = end row of group g; group g starts at align(layout[g-1], alignment)
    kModeMasked = 2,  // A/D are [G, max_m, *]; layout[g] = valid rows of group g
    kModeDense = 3,   // one group covering rows [0, m); no layout array
    kModeKGrouped = 4,  // groups along K: A [sum_k, m], B [sum_k, n] (MN-major), D [G, m, n]; layout[g] = K rows of group g
};

enum EpilogueKind : int {
    kEpiBF16 = 0,    // D bf16
    kEpiF32 = 1,     // D fp32 (raw accumulators; bring-up and tests)
    kEpiSwiGLU = 2,  // gate/up -> silu(gate)*up*row_weight -> per-32 UE8M0 FP8 requant
    kEpiSwiGLUNvfp4 = 3,  // gate/up -> silu(gate)*up*row_weight -> NVFP4 (per-16 UE4M3 scales, given per-tensor scale)
    kEpiSwiGLUBf16 = 4,   // gate/up -> silu(gate)*up*row_weight -> BF16 rows (the BF16 layer)
    kEpiF32Acc = 5,       // D fp32 = C + accumulator; selects the K-grouped form of the kernel (kModeKGrouped)
    kEpiSwiGLUPush = 6,   // kEpiSwiGLU whose epilogue warps also push dispatch rows of the next expert phase (GemmParams::push):
                          // an instantiation of its own, so that the plain kernel's register allocation stays as it is
};

enum MmaKind : int {
    kKindFp8Fp4 = 0,  // kind::mxf8f6f4: E4M3 activations x E2M1 (unpacked in smem) or E4M3 weights, UE8M0 scales, K block 128
    kKindNvfp4 = 1,   // kind::mxf4nvf4 scale_vec::4X: packed E2M1 x packed E2M1, UE4M3 scale per 16, K block 256
    kKindBf16 = 2,    // kind::f16: BF16 x BF16, no scale factors, K block 64 (the scale-factor loads, copies and
                      // TMEM columns of the other kinds stay unused)
};

constexpr int kMaxRanks = 8;

// Rows the gate/up GEMM's epilogue warps push to other ranks between tiles (see GemmParams::push). Lives in device memory.
struct PushWork {
    const int* list;             // entries (token * topk + k) of the next phase, in any order
    const int* count;            // their number
    const unsigned char* x;      // this rank's quantised rows [tokens, row_bytes]
    const unsigned* x_sf;        // their packed scale ints [tokens, sf_per_row]
    const float* topk_weights;   // [tokens * topk]
    const long long* topk_idx;   // [tokens * topk]
    const int* dest_row;         // row of each entry on the rank that computes it
    const int* my_dest;          // computing rank per expert (spill plan), or null: expert / experts_per_rank
    int experts_per_rank, topk, row_bytes, sf_per_row, my_rank, entries_per_rank;
    unsigned long long acts_base[kMaxRanks], sf_base[kMaxRanks], weight_base[kMaxRanks], src_base[kMaxRanks];  // per rank
};

struct GemmParams {
    // Scale factors are read through tensor maps over int32 [groups * packed_k, aligned MN] (packed UE8M0, MN-major):
    // int (group, kp, row) sits at outer coordinate group * packed_k + kp, inner coordinate row.
    int sfa_group_rows;  // packed K ints per group of A's scale factors (0 when A is not grouped)
    int sfb_packed_k;    // packed K ints per group of B's scale factors
    void* d;
    long long d_row_stride;  // elements
    const int* layout;
    int mode, m, n, k, num_groups, alignment;
    int gran_a, gran_b;      // 32 or 128
    unsigned b_tx_bytes;     // bytes the B tile's TMA reports to the mbarrier
    unsigned b_fmt;          // kFmtE2M1_F8F6F4 or kFmtE4M3
    int store_padding;       // psum only: also write the rows between a group's end and its aligned end
    int rows_lo, rows_hi;    // psum / masked layouts: only groups whose valid rows lie in [rows_lo, rows_hi] (rows_skip = 0)
    int rows_skip;           // ... or outside it (rows_skip = 1) are computed; {0, 0, 0} = every group. Lets two kernels
                             // with different tile orientations split the groups of one GEMM by size.
    int group_begin, group_end;  // psum / masked layouts: only groups in [group_begin, group_end) are computed; {0, 0} = all.
                                 // The expert-parallel layer runs its experts phase by phase.
    // SwiGLU epilogue only
    unsigned char* act_q;        // e4m3 [rows, n/2]
    int tma_store;               // epilogue stores through shared memory + TMA (BLOCK_N = 256, FP8 x FP4 kind): 0 never,
                                 // 1 for tiles whose 128 rows are all valid, 2 always (rows past a group's end may be overwritten)
    int sf_transposed;           // scale factors of A and B already lie in the tcgen05.cp row order (sf_row_in_cp_order)
    int act_sf_transposed;       // the SwiGLU epilogues write act_sf in that order too
    unsigned char* act_sf;       // packed UE8M0 bytes, MN-major ints: ((j/128)*act_sf_k_stride + row)*4 + (j/32)%4
    long long act_q_row_stride;  // bytes
    long long act_sf_k_stride;   // ints
    const float* row_weight;     // per destination row, may be null (weight 1)
    float clamp;                 // <= 0: no clamp
    int fast_math;               // SwiGLU: approximate exp / reciprocal (the reference's default) or IEEE expf and division
    // NVFP4 only: FP32 per-tensor scales. The accumulator is multiplied by a_scale[0] * b_scales[group]; the SwiGLU
    // epilogue requantises with the given (calibrated) out_scale[0].
    const float* a_scale;
    const float* b_scales;
    const float* out_scale;
    const float* c;  // kEpiF32Acc: unused by the kernel (the host puts c into d before the launch)
    int a_mn_major;  // BF16 kind, dense mode only: A is [k, m] with m contiguous (the reference's "tn" / "tt" forms)
    int b_mn_major;  // BF16 and FP8 x FP4 kinds: B is [groups * k, n] with n contiguous (the reference's "nn" forms; packed FP4
                     // then holds two consecutive N elements per byte) instead of [groups * n, k]
    int accumulate;  // kEpiF32 only: d += accumulator instead of d = accumulator (the dense GEMMs' input c, already in d)
    int kg_psum;     // kModeKGrouped: layout[g] is the end K row of group g (groups start at multiples of `alignment`,
                     // the gap rows are zero) instead of its K extent
    // kEpiBF16, BLOCK_N = 256, expert-parallel down GEMM only: the epilogue does not write d but sends every output row
    // straight to the rank its token came from (GEMM and return transfer in one kernel, tile by tile):
    // ret_src[row] = source rank * ret_entries_per_rank + entry (written by the dispatch push), the row goes to
    // ret_base[source rank] + entry * n * 2 bytes. Null = write d.
    const int* ret_src;
    int ret_entries_per_rank;
    unsigned long long ret_base[kMaxRanks];  // each rank's buffer of returned rows as mapped into this process
    // kEpiSwiGLU, expert-parallel gate/up GEMM only: between its tiles every epilogue warp also pushes some of the rows this
    // rank routes to the NEXT expert phase into the buffers of the ranks that compute them (the dispatch of phase q + 1
    // rides on the GEMM of phase q, whose epilogue warps are idle most of a tile). Null: nothing to push. A pointer to device
    // memory, not a member: the descriptor is large and kernel parameters are copied at every launch of every variant.
    const PushWork* push;
};

// K rows [start, start + len) of group `g` of a K-grouped operand; `prev_end` carries the running end between calls
// made for g = 0, 1, ... in order.
__device__ __forceinline__ void k_group_extent(const int* layout, int g, int psum, int alignment, int& prev_end, int& start,
                                               int& len) {
    const int v = layout[g];
    if (psum) {
        start = (prev_end + alignment - 1) / alignment * alignment;
        len = max(v - start, 0);
        prev_end = v;
    } else {
        start = prev_end;
        len = v;
        prev_end += v;
    }
}

struct Tile {
    int row_start;     // first row in the flattened A / D
    int sf_row_start;  // first row inside the group's SF block (masked) or global row (others)
    int rows_store;    // rows of this tile to write
    int group;
    int n_block;
    // K-grouped form only: first K row of the group in A / B, its K blocks, first packed scale row of the group
    int k_row_start, num_kb, sf_kp0;
};

constexpr int kMaxCachedGroups = 512;   // group extents of up to this many groups are staged in shared memory

// Per-group schedule staged in shared memory by the kernel prologue (psum and masked layouts, up to
// kMaxCachedGroups groups): the layout words, each group's first row and the running tile count. Every warp role
// walks the tile sequence on its own, and the MMA issuer does so on the critical path between two tiles while the
// epilogue warps compete for the same issue slots, so finding the next tile must take a handful of instructions.
struct GroupTable {
    const int* lay;        // psum ends / masked counts
    const int* start;      // first row of the group
    const int* tiles_end;  // tiles of groups 0..g inclusive
    bool cached;           // false: walk the global layout array with the arithmetic below (more groups than the table holds)
};

__device__ __forceinline__ bool group_in_range(const GemmParams& p, int group) {
    return (p.group_begin == 0 && p.group_end == 0) || (group >= p.group_begin && group < p.group_end);
}

__device__ __forceinline__ bool group_selected(const GemmParams& p, int rows) {
    if (p.rows_lo == 0 && p.rows_hi == 0) return true;
    const bool inside = rows >= p.rows_lo && rows <= p.rows_hi;
    return p.rows_skip ? !inside : inside;
}

template <int BLOCK_N, bool kKGrouped = false>
struct TileScheduler {
    const GemmParams& p;
    const GroupTable tab;
    int num_n_blocks;
    int tile;  // next global tile index of this CTA
    int g, tiles_before_g;

    __device__ TileScheduler(const GemmParams& params, const GroupTable& table)
        : p(params), tab(table), num_n_blocks(params.n / BLOCK_N), tile(static_cast<int>(blockIdx.x)), g(0),
          tiles_before_g(0) {}

    // First row, valid rows and rows to store of one group, from the layout words.
    __device__ __forceinline__ static void group_extent(const GemmParams& p, const int* lay, int group, int& start, int& rows,
                                                        int& rows_store) {
        if (p.mode == kModeMasked) {
            start = group * p.m;
            rows = min(lay[group], p.m);
            rows_store = rows;
        } else {
            const int prev_end = group == 0 ? 0 : lay[group - 1];
            start = (prev_end + p.alignment - 1) / p.alignment * p.alignment;
            const int end = lay[group];
            rows = max(end - start, 0);
            const int aligned_end = min((end + p.alignment - 1) / p.alignment * p.alignment, p.m);
            rows_store = p.store_padding ? max(aligned_end - start, 0) : rows;
        }
    }

    __device__ __forceinline__ void fill(Tile& t, int group, int start, int rows_store, int local) {
        int mb = 0;
        while (local >= num_n_blocks) { local -= num_n_blocks; ++mb; }  // groups are a few M blocks tall
        t.n_block = local;
        t.row_start = start + mb * 128;
        t.sf_row_start = p.mode == kModeMasked ? mb * 128 : t.row_start;
        t.rows_store = min(128, rows_store - mb * 128);
        t.group = group;
        tile += static_cast<int>(gridDim.x);
    }

    // Returns false when this CTA has no more tiles. A tile with group < 0 must be skipped by every role.
    __device__ bool next(Tile& t) {
        if constexpr (kKGrouped) {
            // every group has the same (m blocks x n blocks) output tiles; the table holds (K blocks, first K row,
            // first packed scale row) per group
            const int per_group = (p.m + 127) / 128 * num_n_blocks;
            if (tile >= p.num_groups * per_group) return false;
            const int group = tile / per_group;
            const int local = tile - group * per_group;
            const int mb = local / num_n_blocks;
            t.n_block = local - mb * num_n_blocks;
            t.row_start = t.sf_row_start = mb * 128;
            t.rows_store = min(128, p.m - mb * 128);
            t.group = group;
            t.num_kb = tab.lay[group];
            t.k_row_start = tab.start[group];
            t.sf_kp0 = tab.tiles_end[group];
            tile += static_cast<int>(gridDim.x);
            return true;
        }
        if (p.mode == kModeRowIds || p.mode == kModeDense) {
            const int num_m_blocks = (p.m + 127) / 128;
            if (tile >= num_m_blocks * num_n_blocks) return false;
            const int mb = tile / num_n_blocks;
            t.n_block = tile - mb * num_n_blocks;
            t.row_start = t.sf_row_start = mb * 128;
            t.rows_store = min(128, p.m - t.row_start);
            t.group = p.mode == kModeDense ? 0 : __ldg(p.layout + t.row_start);
            tile += static_cast<int>(gridDim.x);
            return true;
        }
        if (tab.cached) {
            while (g < p.num_groups && tile >= tab.tiles_end[g]) ++g;
            if (g >= p.num_groups) return false;
            const int start = tab.start[g];
            int rows_store;
            if (p.mode == kModeMasked) {
                rows_store = min(tab.lay[g], p.m);
            } else if (p.store_padding) {
                rows_store = max(min((tab.lay[g] + p.alignment - 1) / p.alignment * p.alignment, p.m) - start, 0);
            } else {
                rows_store = max(tab.lay[g] - start, 0);
            }
            fill(t, g, start, rows_store, tile - (g == 0 ? 0 : tab.tiles_end[g - 1]));
            return true;
        }
        while (g < p.num_groups) {
            int start, rows, rows_store;
            group_extent(p, tab.lay, g, start, rows, rows_store);
            const int tiles_g = (group_selected(p, rows) && group_in_range(p, g)) ? (max(rows, rows_store) + 127) / 128 * num_n_blocks : 0;
            if (tile < tiles_before_g + tiles_g) {
                fill(t, g, start, rows_store, tile - tiles_before_g);
                return true;
            }
            tiles_before_g += tiles_g;
            ++g;
        }
        return false;
    }
};

template <int BLOCK_N, int kStages, int kKind = kKindFp8Fp4, bool kAlwaysStaged = false>
struct GemmSmem {
    static constexpr int kSfIntsPerRow = kKind == kKindNvfp4 ? 4 : 1;  // packed scale ints per row per K block
    static constexpr int kABytes = 128 * 128;
    static constexpr int kBBytes = BLOCK_N * 128;
    static constexpr int kSfaBytes = 128 * 4 * kSfIntsPerRow;
    static constexpr int kSfbBytes = BLOCK_N * 4 * kSfIntsPerRow;
    static constexpr int kOffA = 0;
    static constexpr int kOffB = kOffA + kStages * kABytes;
    static constexpr int kOffSfa = kOffB + kStages * kBBytes;
    static constexpr int kOffSfb = kOffSfa + kStages * kSfaBytes;
    static constexpr int kOffBar = kOffSfb + kStages * kSfbBytes;
    static constexpr int kNumBars = 3 * kStages + 4;
    static constexpr int kOffMisc = kOffBar + kNumBars * 8;
    static constexpr int kOffGroups = kOffMisc + 16;
    // Epilogue staging for TMA stores: 32 rows x 64 bytes per epilogue warp, in the 64-byte swizzle (512-byte atoms).
    // The NVFP4 kind only has room for it next to its larger scale-factor stages with 3 pipeline stages.
    static constexpr int kStageBytesPerWarp =
        (kAlwaysStaged || (BLOCK_N == 256 && (kKind != kKindNvfp4 || kStages <= 3))) ? 2048 : 0;
    static constexpr int kOffStage = (kOffGroups + 3 * kMaxCachedGroups * 4 + 511) / 512 * 512;
    static constexpr int kTotal = kOffStage + 8 * kStageBytesPerWarp;
    static constexpr int kDynamicBytes = kTotal + 1024;  // slack to align the base to 1024 B
};

// Smallest power of two >= amax/448, as (sf, 1/sf, biased exponent byte). Mirrors the reference's in-kernel
// requant rule (deep_gemm/include/deep_gemm/common/math.cuh:83-99): exponent is bumped when the mantissa of
// amax/448 is non-zero; no lower clamp other than the UE8M0 range.
__device__ __forceinline__ void ue8m0_scale_for_amax(float amax, float& sf_inv, uint32_t& sf_byte) {
    const float s = amax * (1.0f / 448.0f);
    const uint32_t bits = __float_as_uint(s);
    uint32_t e = (bits >> 23) & 0xffu;
    if (bits & 0x7fffffu) ++e;
    e = min(max(e, 1u), 254u);
    sf_byte = e;
    sf_inv = __uint_as_float((254u - e) << 23);  // 2^(127-e)
}

constexpr int kGemmThreads = 384;       // warps 0-3: loaders / MMA / transposer; warps 4-11: epilogue
constexpr int kRegsControlWarps = 96;   // after setmaxnreg: the control warpgroup gives registers away ...
constexpr int kRegsEpilogueWarps = 200; // ... to the two epilogue warpgroups, which hold a drained accumulator

template <int BLOCK_N, int kStages, int kEpilogue, int kKind = kKindFp8Fp4>
__global__ void __launch_bounds__(kGemmThreads, 1)
dgb200_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
                           const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ GemmParams p) {
    constexpr bool kPushes = kEpilogue == kEpiSwiGLUPush;
    constexpr int EPI = kPushes ? static_cast<int>(kEpiSwiGLU) : kEpilogue;
    using L = GemmSmem<BLOCK_N, kStages, kKind, EPI == kEpiF32Acc>;
    static_assert(BLOCK_N == 128 || BLOCK_N == 256, "BLOCK_N must be 128 or 256");
    static_assert(L::kDynamicBytes <= 232448, "shared memory budget");
    constexpr int kSfInts = L::kSfIntsPerRow;          // scale ints per row per K block = tcgen05.cp blocks per 128 rows
    constexpr int kSfBlocksA = kSfInts;                // 512-byte blocks of A scales per stage
    constexpr int kSfBlocksB = kSfInts * BLOCK_N / 128;
    constexpr int kBlockK = kKind == kKindNvfp4 ? 256 : (kKind == kKindBf16 ? 64 : 128);  // K elements per stage (128 bytes per row either way)
    constexpr int kTmaXPerKb = kKind == kKindBf16 ? 64 : 128;  // tensor-map elements along K per stage (bytes, 4-bit or 16-bit elements)
    constexpr bool kScaled = kKind != kKindBf16;
    constexpr uint32_t kAccumCols = BLOCK_N;
    constexpr uint32_t kNumAccum = BLOCK_N == 128 ? 2 : 1;
    // Scale factors get their own TMEM columns per pipeline stage: with a single region every tcgen05.cp would have
    // to wait for the previous K block's MMAs to finish reading it, which serialises copy and MMA.
    constexpr uint32_t kSfColsPerStage = 4 * (kSfBlocksA + kSfBlocksB);
    constexpr uint32_t kSfCol0 = kAccumCols * kNumAccum;
    constexpr uint32_t kTmemCols = 512;
    static_assert(kSfCol0 + kStages * kSfColsPerStage <= kTmemCols, "TMEM budget");
    // NVFP4 needs 12 tcgen05.cp per K block (4 scale ints per row); issued next to the 4 MMAs they make the MMA warp's
    // instruction stream, not the tensor pipe, the bound. With scale factors in tcgen05.cp order warp 2 has no
    // transposing to do and issues the copies instead, one stage ahead of the MMAs.
    constexpr bool kCpByHelper = kKind == kKindNvfp4;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + kStages;
    uint64_t* sf_ready_bar = bars + 2 * kStages;
    uint64_t* tmem_full_bar = bars + 3 * kStages;
    uint64_t* tmem_empty_bar = bars + 3 * kStages + 2;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kOffMisc + 4);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(full_bar + i, 2);       // the A-side loader and the B-side loader
            mbar_init(empty_bar + i, 1);      // tcgen05.commit of the MMA issuer
            mbar_init(sf_ready_bar + i, 1);   // one lane of the transposer warp, after a warp barrier
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tmem_full_bar + i, 1);
            mbar_init(tmem_empty_bar + i, 8);  // lane 0 of each epilogue warp
        }
        fence_mbar_init();
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        prefetch_tensormap(&tm_sfa);
        prefetch_tensormap(&tm_sfb);
        if (p.tma_store) prefetch_tensormap(&tm_out);
    }
    pdl_prologue();  // everything above touches only this CTA's shared memory and the kernel's own parameters
    // Stage the per-group schedule (see GroupTable): every thread fills its groups, warp 0 turns the per-group tile
    // counts into running totals.
    int* group_cache = reinterpret_cast<int*>(smem + L::kOffGroups);
    int* group_start = group_cache + kMaxCachedGroups;
    int* group_tiles_end = group_start + kMaxCachedGroups;
    constexpr bool kKG = EPI == kEpiF32Acc;  // K-grouped form: MN-major operands, per-group K extents, D = C + acc
    const bool cache_groups = ((p.mode == kModePsum || p.mode == kModeMasked) && p.num_groups <= kMaxCachedGroups) || kKG;
    if constexpr (kKG) {
        // (K blocks, first K row, first packed scale row) per group: a serial scan by one thread (at most
        // kMaxCachedGroups groups, checked by the host)
        if (threadIdx.x == 0) {
            int prev_end = 0, kp = 0;
            for (int i = 0; i < p.num_groups; ++i) {
                int start, len;
                k_group_extent(p.layout, i, p.kg_psum, p.alignment, prev_end, start, len);
                // Plain layout: the groups abut, so an extent that is not a whole number of K blocks would make the
                // last block read the next group's rows, and extents that overrun the operands would read past them.
                // Such a group is reported and left out (d keeps c). In the psum layout a partial last block reads
                // the zero rows of the gap, which is what that layout is for.
                if (len < 0 || start + len > p.k || (!p.kg_psum && len % kBlockK != 0)) {
                    report_error(kBadArgument, i, len);
                    len = 0;
                }
                const int blocks = (len + kBlockK - 1) / kBlockK;
                group_cache[i] = blocks;
                group_start[i] = start;
                group_tiles_end[i] = kp;
                kp += p.gran_a == 32 ? blocks : (blocks + 3) / 4;  // packed scale rows: one per K block, or per 4 K blocks
            }
        }
    } else if (cache_groups) {
        for (int i = threadIdx.x; i < p.num_groups; i += kGemmThreads) {
            int start, rows, rows_store;
            TileScheduler<BLOCK_N, EPI == kEpiF32Acc>::group_extent(p, p.layout, i, start, rows, rows_store);
            group_cache[i] = __ldg(p.layout + i);
            group_start[i] = start;
            group_tiles_end[i] = (group_selected(p, rows) && group_in_range(p, i)) ? (max(rows, rows_store) + 127) / 128 * (p.n / BLOCK_N) : 0;
        }
        __syncthreads();
        if (warp == 0) {
            const int chunk = (p.num_groups + 31) / 32;
            const int lo = min(static_cast<int>(lane) * chunk, p.num_groups), hi = min(lo + chunk, p.num_groups);
            int sum = 0;
            for (int i = lo; i < hi; ++i) sum += group_tiles_end[i];
            int incl = sum;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, off);
                if (static_cast<int>(lane) >= off) incl += v;
            }
            int run = incl - sum;
            for (int i = lo; i < hi; ++i) {
                run += group_tiles_end[i];
                group_tiles_end[i] = run;
            }
        }
    }
    const GroupTable group_layout{cache_groups ? group_cache : p.layout, group_start, group_tiles_end, cache_groups};
    if (warp == 2) tmem_alloc(tmem_ptr_smem, kTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;

    const int num_kb = p.k / kBlockK;
    const int a_per = (kKind == kKindNvfp4 || p.gran_a == 32) ? 1 : 4;  // K blocks covered by one packed SF int
    const int b_per = (kKind == kKindNvfp4 || p.gran_b == 32) ? 1 : 4;

    // Register re-balancing: each setmaxnreg dominates the code of its warpgroups, so that the compiler allocates
    // the epilogue (which holds half an accumulator row in registers) under the raised limit.
    if (warp < 4) {
    setmaxnreg_dec<kRegsControlWarps>();
    if (warp == 0) {
        // ---------------------------------------------------------------- loader: A tile + its scale factors
        // TMA instructions cost on the order of 100 cycles each in the issuing thread, so the loads of one stage are
        // split over two threads (this one and warp 3); both arrive on the stage's full barrier with their own bytes.
        // The whole warp walks the schedule with warp-uniform values and one elected lane issues: TMA and tcgen05
        // instructions take their descriptors from uniform registers, which a single-lane (divergent) loop would
        // have to refill through slow register-to-uniform moves for every instruction.
        {
            TileScheduler<BLOCK_N, EPI == kEpiF32Acc> sched(p, group_layout);
            Tile t;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            while (ok && sched.next(t)) {
                if (t.group < 0) continue;
                const int sfa_y = kKG ? t.sf_kp0 : t.group * p.sfa_group_rows;
                const int tile_kb = kKG ? t.num_kb : num_kb;
                for (int kb = 0; kb < tile_kb; ++kb) {
                    ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, kTimeoutEmpty, kb);
                    if (!ok) break;
                    const bool load_sfa = kScaled && kb % a_per == 0;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(full_bar + stage, L::kABytes + (load_sfa ? L::kSfaBytes : 0));
                        if constexpr (kKG) {
                            // MN-major A: one box per 128 bytes of M (128 E4M3 or 64 BF16 channels) x kBlockK K rows
                            constexpr int kBoxes = kKind == kKindBf16 ? 2 : 1;
#pragma unroll
                            for (int h = 0; h < kBoxes; ++h)
                                tma_load_2d(smem + L::kOffA + stage * L::kABytes + h * (L::kABytes / kBoxes), &tm_a,
                                            full_bar + stage, t.row_start + h * (128 / kBoxes), t.k_row_start + kb * kBlockK);
                        } else if (kKind == kKindBf16 && p.a_mn_major) {
#pragma unroll
                            for (int h = 0; h < 2; ++h)
                                tma_load_2d(smem + L::kOffA + stage * L::kABytes + h * 8192, &tm_a, full_bar + stage,
                                            t.row_start + h * 64, kb * 64);
                        } else
                            tma_load_2d(smem + L::kOffA + stage * L::kABytes, &tm_a, full_bar + stage, kb * kTmaXPerKb,
                                        t.row_start);
                        if (load_sfa)
                            tma_load_2d(smem + L::kOffSfa + stage * L::kSfaBytes, &tm_sfa, full_bar + stage,
                                        t.sf_row_start, sfa_y + kb * kSfInts / a_per);
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 3) {
        // ---------------------------------------------------------------- loader: B (weight) tile + its scale factors
        {
            TileScheduler<BLOCK_N, EPI == kEpiF32Acc> sched(p, group_layout);
            Tile t;
            uint32_t stage = 0, phase = 0;
            bool ok = true;

            const bool leader = elect_one();

            while (ok && sched.next(t)) {
                if (t.group < 0) continue;
                const int b_row = t.group * p.n + t.n_block * BLOCK_N;
                const int sfb_y = kKG ? t.sf_kp0 : t.group * p.sfb_packed_k;
                const int tile_kb = kKG ? t.num_kb : num_kb;
                for (int kb = 0; kb < tile_kb; ++kb) {
                    ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, kTimeoutEmpty, kb);
                    if (!ok) break;
                    const bool load_sfb = kScaled && kb % b_per == 0;
                    if (leader) {
                        mbar_arrive_expect_tx(full_bar + stage, p.b_tx_bytes + (load_sfb ? L::kSfbBytes : 0));
                        if constexpr (kKG) {
                            // one box per 128 bytes of N (a swizzle span: 128 E4M3 or 64 BF16 channels) x kBlockK K rows
                            constexpr int kChan = kKind == kKindBf16 ? 64 : 128;
#pragma unroll
                            for (int h = 0; h < BLOCK_N / kChan; ++h)
                                tma_load_2d(smem + L::kOffB + stage * L::kBBytes + h * (128 * kBlockK), &tm_b, full_bar + stage,
                                            t.n_block * BLOCK_N + h * kChan, t.k_row_start + kb * kBlockK);
                        } else if (kKind == kKindBf16 && p.b_mn_major) {
                            // MN-major weights: boxes of 64 channels x 64 K rows, as in the K-grouped form
#pragma unroll
                            for (int h = 0; h < BLOCK_N / 64; ++h)
                                tma_load_2d(smem + L::kOffB + stage * L::kBBytes + h * 8192, &tm_b, full_bar + stage,
                                            t.n_block * BLOCK_N + h * 64, t.group * p.k + kb * 64);
                        } else if (kKind == kKindFp8Fp4 && p.b_mn_major) {
                            // MN-major 8-bit (or 4-bit in byte containers) weights: boxes of 128 channels x 128 K rows
#pragma unroll
                            for (int h = 0; h < BLOCK_N / 128; ++h)
                                tma_load_2d(smem + L::kOffB + stage * L::kBBytes + h * 16384, &tm_b, full_bar + stage,
                                            t.n_block * BLOCK_N + h * 128, t.group * p.k + kb * 128);
                        } else
                            tma_load_2d(smem + L::kOffB + stage * L::kBBytes, &tm_b, full_bar + stage, kb * kTmaXPerKb, b_row);
                        if (load_sfb)
                            tma_load_2d(smem + L::kOffSfb + stage * L::kSfbBytes, &tm_sfb, full_bar + stage,
                                        t.n_block * BLOCK_N, sfb_y + kb * kSfInts / b_per);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // Warp-uniform loop, one elected lane issues (see the loader above).
        {
        TileScheduler<BLOCK_N, EPI == kEpiF32Acc> sched(p, group_layout);
        Tile t;
        uint32_t stage = 0, phase = 0, iter = 0;
        const uint32_t idesc = kKG
            ? ((kKind == kKindBf16 ? make_idesc_bf16_f32(128, BLOCK_N)
                                   : make_idesc_block_scaled(kFmtE4M3, kFmtE4M3, 128, BLOCK_N, kScaleUE8M0)) |
               (1u << 15) | (1u << 16))  // both operands MN-major
            : kKind == kKindBf16
            ? (make_idesc_bf16_f32(128, BLOCK_N) | (p.a_mn_major ? (1u << 15) : 0u) | (p.b_mn_major ? (1u << 16) : 0u))
            : kKind == kKindNvfp4 ? make_idesc_block_scaled(kFmtE2M1_MXF4, kFmtE2M1_MXF4, 128, BLOCK_N, kScaleUE4M3)
                                  : (make_idesc_block_scaled(kFmtE4M3, p.b_fmt, 128, BLOCK_N, kScaleUE8M0) |
                                     (p.b_mn_major ? (1u << 16) : 0u));
        const uint32_t a_base = smem_u32(smem + L::kOffA), b_base = smem_u32(smem + L::kOffB);
        const uint32_t sfa_smem = smem_u32(smem + L::kOffSfa), sfb_smem = smem_u32(smem + L::kOffSfb);
        uint32_t tmem_sfa = 0, tmem_sfb = 0;  // TMEM columns holding the scale factors of the current K block
        const bool leader = elect_one();      // the same lane issues every tcgen05 instruction of this CTA
        bool ok = true;
        while (ok && sched.next(t)) {
            if (t.group < 0) continue;
            const uint32_t as = iter % kNumAccum, aphase = (iter / kNumAccum) & 1;
            ++iter;
            ok = mbar_wait(tmem_empty_bar + as, aphase ^ 1, abort_flag, kTimeoutTmemEmpty, static_cast<int>(iter));
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t tmem_acc = tmem_base + as * kAccumCols;
            const int tile_kb = kKG ? t.num_kb : num_kb;
            if (kKG && tile_kb == 0 && leader) tcgen05_commit(tmem_full_bar + as);  // empty group: D = C, nothing to wait for
            for (int kb = 0; kb < tile_kb; ++kb) {
                // scale factors stored in tcgen05.cp order need no transposer pass: the loads' barrier is enough
                ok = mbar_wait(((!kScaled || (p.sf_transposed && !kCpByHelper)) ? full_bar : sf_ready_bar) + stage, phase, abort_flag,
                               kTimeoutSfReady, kb);
                if (!ok) break;
                if (kCpByHelper && p.sf_transposed) tcgen05_fence_after();  // the helper warp's tcgen05.cp precede our MMAs
                // No tcgen05 fence here: the data this wait covers was written to shared memory through the async proxy
                // (TMA, or the transposer's stores followed by its proxy fence), not by tcgen05 operations.
                if (leader) {
                    // One tcgen05.cp moves the scales of 128 rows for one MMA (one packed int per row) into 4 TMEM columns.
                    const uint32_t sf_cols = tmem_base + kSfCol0 + stage * kSfColsPerStage;
                    const bool cp_here = kScaled && !(kCpByHelper && p.sf_transposed);
                    if (kb % a_per == 0) {
                        tmem_sfa = sf_cols;
                        if (cp_here) {
#pragma unroll
                            for (int b = 0; b < kSfBlocksA; ++b)
                                tcgen05_cp_32x128b_warpx4(tmem_sfa + b * 4, make_sf_desc(sfa_smem + stage * L::kSfaBytes + b * 512));
                        }
                    }
                    if (kb % b_per == 0) {
                        tmem_sfb = sf_cols + 4 * kSfBlocksA;
                        if (cp_here) {
#pragma unroll
                            for (int b = 0; b < kSfBlocksB; ++b)
                                tcgen05_cp_32x128b_warpx4(tmem_sfb + b * 4, make_sf_desc(sfb_smem + stage * L::kSfbBytes + b * 512));
                        }
                    }
                    // MN-major tiles: consecutive 128-byte chunks along M / N are one TMA box (128 bytes x kBlockK rows) apart
                    const bool a_mn = kKG || (kKind == kKindBf16 && p.a_mn_major);
                    const uint64_t adesc = a_mn ? make_mnmajor_sw128_desc(a_base + stage * L::kABytes, 128 * kBlockK)
                                                : make_kmajor_sw128_desc(a_base + stage * L::kABytes);
                    const bool b_mn = kKG || ((kKind == kKindBf16 || kKind == kKindFp8Fp4) && p.b_mn_major);
                    const uint64_t bdesc = b_mn ? make_mnmajor_sw128_desc(b_base + stage * L::kBBytes, 128 * kBlockK)
                                                : make_kmajor_sw128_desc(b_base + stage * L::kBBytes);
                    // K-major: +32 bytes along K inside the swizzle span per MMA; MN-major: the K rows of one MMA (32 E4M3 or
                    // 16 BF16) are 4 or 2 groups of 8 rows = 1024 B each
                    constexpr uint32_t kDescStep = kKG ? (kKind == kKindBf16 ? 128 : 256) : 2;
                    const uint32_t a_step = (kKind == kKindBf16 && a_mn) ? 128u : kDescStep;
                    const uint32_t b_step = (kKind == kKindBf16 && b_mn) ? 128u : ((kKind == kKindFp8Fp4 && b_mn) ? 256u : kDescStep);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4) {
                        // +32 bytes along K inside the 128-byte swizzle span = +2 in the (addr >> 4) field
                        if constexpr (kKind == kKindBf16) {
                            // K = 16 BF16 elements (32 bytes) per MMA
                            tcgen05_mma_f16(tmem_acc, adesc + k4 * a_step, bdesc + k4 * b_step, idesc, (kb | k4) != 0 ? 1u : 0u);
                        } else if constexpr (kKind == kKindNvfp4) {
                            // K = 64 per MMA; its 4 scales per row are the 4 bytes of packed int k4 of the stage
                            tcgen05_mma_mxf4nvf4_4x(tmem_acc, adesc + k4 * 2, bdesc + k4 * 2, idesc, tmem_sfa + k4 * 4,
                                                    tmem_sfb + k4 * (BLOCK_N / 32), (kb | k4) != 0 ? 1u : 0u);
                        } else {
                            const uint32_t sfa_id = p.gran_a == 32 ? k4 : static_cast<uint32_t>(kb % 4);
                            const uint32_t sfb_id = p.gran_b == 32 ? k4 : static_cast<uint32_t>(kb % 4);
                            tcgen05_mma_mxf8f6f4(tmem_acc, adesc + k4 * a_step, bdesc + k4 * b_step,
                                                 idesc_with_sf_ids(idesc, sfa_id, sfb_id), tmem_sfa, tmem_sfb,
                                                 (kb | k4) != 0 ? 1u : 0u);
                        }
                    }
                    tcgen05_commit(empty_bar + stage);
                    if (kb == tile_kb - 1) tcgen05_commit(tmem_full_bar + as);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- scale-factor transposer
        // tcgen05.cp 32x128b wants, per 128 rows, 32 rows x 4 words with word j of row r = source row r + 32 j.
        TileScheduler<BLOCK_N, EPI == kEpiF32Acc> sched(p, group_layout);
        Tile t;
        uint32_t stage = 0, phase = 0;
        bool ok = kScaled && p.sf_transposed == 0;  // nothing to do when the scale factors arrive in tcgen05.cp order
        while (ok && sched.next(t)) {
            if (t.group < 0) continue;
            const int tile_kb = kKG ? t.num_kb : num_kb;
            for (int kb = 0; kb < tile_kb; ++kb) {
                ok = mbar_wait(full_bar + stage, phase, abort_flag, kTimeoutFull, kb);
                if (!ok) break;
                // All reads first, one warp barrier, then all writes: this warp serves every K block in turn, so its
                // service time bounds the whole pipeline.
                const bool do_a = kb % a_per == 0, do_b = kb % b_per == 0;
                uint32_t* sa = reinterpret_cast<uint32_t*>(smem + L::kOffSfa + stage * L::kSfaBytes);
                uint32_t* sb = reinterpret_cast<uint32_t*>(smem + L::kOffSfb + stage * L::kSfbBytes);
                uint32_t va[kSfBlocksA][4], vb[kSfBlocksB][4];
                if (do_a) {
#pragma unroll
                    for (int b = 0; b < kSfBlocksA; ++b)
#pragma unroll
                        for (int j = 0; j < 4; ++j) va[b][j] = sa[b * 128 + j * 32 + lane];
                }
                if (do_b) {
#pragma unroll
                    for (int b = 0; b < kSfBlocksB; ++b)
#pragma unroll
                        for (int j = 0; j < 4; ++j) vb[b][j] = sb[b * 128 + j * 32 + lane];
                }
                __syncwarp();
                if (do_a) {
#pragma unroll
                    for (int b = 0; b < kSfBlocksA; ++b)
                        *reinterpret_cast<uint4*>(sa + b * 128 + lane * 4) = make_uint4(va[b][0], va[b][1], va[b][2], va[b][3]);
                }
                if (do_b) {
#pragma unroll
                    for (int b = 0; b < kSfBlocksB; ++b)
                        *reinterpret_cast<uint4*>(sb + b * 128 + lane * 4) = make_uint4(vb[b][0], vb[b][1], vb[b][2], vb[b][3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(sf_ready_bar + stage);
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
        if (kCpByHelper && p.sf_transposed != 0) {
            TileScheduler<BLOCK_N, EPI == kEpiF32Acc> cp_sched(p, group_layout);
            const uint32_t sfa_smem = smem_u32(smem + L::kOffSfa), sfb_smem = smem_u32(smem + L::kOffSfb);
            const bool leader = elect_one();
            stage = 0;
            phase = 0;
            ok = true;
            while (ok && cp_sched.next(t)) {
                if (t.group < 0) continue;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(full_bar + stage, phase, abort_flag, kTimeoutFull, kb);
                    if (!ok) break;
                    if (leader) {
                        const uint32_t sf_cols = tmem_base + kSfCol0 + stage * kSfColsPerStage;
#pragma unroll
                        for (int b = 0; b < kSfBlocksA; ++b)
                            tcgen05_cp_32x128b_warpx4(sf_cols + b * 4, make_sf_desc(sfa_smem + stage * L::kSfaBytes + b * 512));
#pragma unroll
                        for (int b = 0; b < kSfBlocksB; ++b)
                            tcgen05_cp_32x128b_warpx4(sf_cols + 4 * kSfBlocksA + b * 4,
                                                      make_sf_desc(sfb_smem + stage * L::kSfbBytes + b * 512));
                        tcgen05_commit(sf_ready_bar + stage);  // arrives once the copies above have completed
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    }
    } else {
        setmaxnreg_inc<kRegsEpilogueWarps>();
        // ---------------------------------------------------------------- epilogue (8 warps)
        // Warp w may read TMEM lanes [32 (w % 4), +32): two warps share a lane quarter and split the columns.
        // Each thread first drains its half row of the accumulator into registers and releases the accumulator, so
        // the MMA issuer can start the next tile while the arithmetic and the stores below run.
        constexpr int kCols = BLOCK_N / 2;  // accumulator columns per thread
        TileScheduler<BLOCK_N, EPI == kEpiF32Acc> sched(p, group_layout);
        Tile t;
        uint32_t iter = 0;
        const uint32_t q = warp & 3, half = (warp - 4) >> 2;
        const int r = static_cast<int>(q * 32 + lane);
        bool ok = true;
        // rows of the next expert phase this warp pushes between its tiles: entries cursor, cursor + all epilogue warps, ...
        int push_cursor = static_cast<int>(blockIdx.x * 8 + (warp - 4)), push_count = 0;
        if constexpr (kPushes) {
            if (p.push != nullptr) push_count = __ldg(p.push->count);
        }
        auto push_rows = [&](int max_rows) {
            if constexpr (kPushes) {
                const PushWork& w = *p.push;
                for (int n = 0; n < max_rows && push_cursor < push_count; ++n, push_cursor += static_cast<int>(gridDim.x) * 8) {
                    const int entry = __ldg(w.list + push_cursor);
                    const int token = entry / w.topk;
                    const int expert = static_cast<int>(__ldg(w.topk_idx + entry));
                    const int owner = w.my_dest != nullptr ? __ldg(w.my_dest + expert) : expert / w.experts_per_rank;
                    const long long dest = __ldg(w.dest_row + entry);
                    const uint4* from = reinterpret_cast<const uint4*>(w.x + static_cast<long long>(token) * w.row_bytes);
                    uint4* to = reinterpret_cast<uint4*>(w.acts_base[owner] + dest * w.row_bytes);
                    const int vecs = w.row_bytes / 16;
                    for (int c0 = static_cast<int>(lane); c0 < vecs; c0 += 32 * 7) {
                        uint4 v[7];
#pragma unroll
                        for (int j = 0; j < 7; ++j)
                            if (c0 + 32 * j < vecs) v[j] = ld_global_nc_v4(from + c0 + 32 * j);
#pragma unroll
                        for (int j = 0; j < 7; ++j)
                            if (c0 + 32 * j < vecs) st_global_v4(to + c0 + 32 * j, v[j].x, v[j].y, v[j].z, v[j].w);
                    }
                    unsigned* sf_to = reinterpret_cast<unsigned*>(w.sf_base[owner]) + dest * w.sf_per_row;
                    for (int c = static_cast<int>(lane); c < w.sf_per_row; c += 32)
                        sf_to[c] = __ldg(w.x_sf + static_cast<long long>(token) * w.sf_per_row + c);
                    if (lane == 0) {
                        reinterpret_cast<float*>(w.weight_base[owner])[dest] = __ldg(w.topk_weights + entry);
                        reinterpret_cast<int*>(w.src_base[owner])[dest] = w.my_rank * w.entries_per_rank + entry;
                    }
                }
            }
        };
        while (ok && sched.next(t)) {
            if (t.group < 0) continue;
            const uint32_t as = iter % kNumAccum, aphase = (iter / kNumAccum) & 1;
            ++iter;
            ok = mbar_wait<32>(tmem_full_bar + as, aphase, abort_flag, kTimeoutTmemFull, static_cast<int>(iter));
            if (!ok) break;
            tcgen05_fence_after();
            const bool warp_has_rows = static_cast<int>(q * 32) < t.rows_store;
            uint32_t acc[kCols];
            if (warp_has_rows) {
                if constexpr (EPI == kEpiSwiGLU || EPI == kEpiSwiGLUNvfp4 || EPI == kEpiSwiGLUBf16) {
                    // tile columns are [gate BLOCK_N / 2 | up BLOCK_N / 2]: this thread takes its half of the gate columns
                    // and the matching up columns
                    const uint32_t tmem_row = tmem_base + as * kAccumCols + ((q * 32u) << 16) + half * (kCols / 2);
#pragma unroll
                    for (int c = 0; c < kCols / 64; ++c) {
                        tmem_ld_32x32b_x32(tmem_row + c * 32, acc + c * 32);
                        tmem_ld_32x32b_x32(tmem_row + BLOCK_N / 2 + c * 32, acc + kCols / 2 + c * 32);
                    }
                } else {
                    const uint32_t tmem_row = tmem_base + as * kAccumCols + ((q * 32u) << 16) + half * kCols;
#pragma unroll
                    for (int c = 0; c < kCols / 32; ++c) tmem_ld_32x32b_x32(tmem_row + c * 32, acc + c * 32);
                }
                tmem_ld_wait();
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty_bar + as);
            // Row-per-thread stores put 32 different cache lines into every store instruction, and the burst of a whole
            // tile keeps the load/store pipe busy long enough to stall the control warps' shared-memory accesses.
            // Staging the warp's 32 x 64-byte slab in shared memory and handing it to TMA costs 4 store wavefronts
            // per 16-byte column instead of 32.
            const bool via_tma = L::kStageBytesPerWarp != 0 && (p.tma_store == 2 || (p.tma_store == 1 && t.rows_store == 128));
            uint8_t* stage_buf = smem + L::kOffStage + (warp - 4) * L::kStageBytesPerWarp;
            // 16-byte chunk c of this thread's 64-byte row in the 64-byte swizzle pattern of the tensor map
            auto stage_chunk = [&](int c) { return reinterpret_cast<uint4*>(stage_buf + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)); };

            const bool store = r < t.rows_store;
            const long long row = static_cast<long long>(t.row_start) + r;
            const long long sf_row = p.act_sf_transposed ? sf_row_in_cp_order(row) : row;  // used by the SwiGLU epilogues
            if constexpr (kKind == kKindNvfp4) {
                if (warp_has_rows) {
                    // fold the two FP32 per-tensor scales into the accumulator
                    const float alpha = __ldg(p.a_scale) * __ldg(p.b_scales + t.group);
#pragma unroll
                    for (int i = 0; i < kCols; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
                }
            }
            if constexpr (L::kStageBytesPerWarp != 0 && EPI == kEpiBF16) {
                if (p.ret_src != nullptr) {
                    // Fused return: this warp's 32 rows x 128 columns (256 bytes of BF16 per row) go to 32 different places
                    // in other ranks' memory. A thread holds a whole row segment in registers, but 32 threads storing 16
                    // bytes each into 32 rows make the worst pattern for NVLink, so the warp turns its slab through the
                    // 2 KB staging buffer eight rows at a time: the eight owners write their 256 bytes (XOR-swizzled
                    // chunks), then every store instruction of the warp writes two complete 256-byte segments.
                    if (warp_has_rows) {
                        unsigned long long my_dst = 0;
                        if (store) {
                            const int src = __ldg(p.ret_src + row);
                            const int src_rank = src / p.ret_entries_per_rank;
                            // a row whose push never arrived (a rank that timed out) carries a stale source id: never
                            // index past the table or store through a null base
                            if (src >= 0 && src_rank < kMaxRanks && p.ret_base[src_rank] != 0)
                                my_dst = p.ret_base[src_rank] +
                                     (static_cast<unsigned long long>(src - src_rank * p.ret_entries_per_rank) * p.n +
                                      static_cast<unsigned long long>(t.n_block * BLOCK_N + static_cast<int>(half) * kCols)) * 2ull;
                        }
#pragma unroll 1
                        for (int pass = 0; pass < 4; ++pass) {
                            __syncwarp();
                            if (static_cast<int>(lane >> 3) == pass) {
                                uint8_t* mine = stage_buf + (lane & 7) * 256;
#pragma unroll
                                for (int c = 0; c < kCols / 8; ++c)
                                    *reinterpret_cast<uint4*>(mine + ((c ^ static_cast<int>(lane & 7)) << 4)) = make_uint4(
                                        pack_bf16x2(__uint_as_float(acc[c * 8 + 0]), __uint_as_float(acc[c * 8 + 1])),
                                        pack_bf16x2(__uint_as_float(acc[c * 8 + 2]), __uint_as_float(acc[c * 8 + 3])),
                                        pack_bf16x2(__uint_as_float(acc[c * 8 + 4]), __uint_as_float(acc[c * 8 + 5])),
                                        pack_bf16x2(__uint_as_float(acc[c * 8 + 6]), __uint_as_float(acc[c * 8 + 7])));
                            }
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int slab_row = static_cast<int>(lane >> 4) + 2 * j;  // 0..7: two rows per instruction
                                const int chunk = static_cast<int>(lane & 15);
                                const uint4 v = *reinterpret_cast<const uint4*>(stage_buf + slab_row * 256 + ((chunk ^ slab_row) << 4));
                                const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, pass * 8 + slab_row);
                                if (dst != 0) st_global_v4(reinterpret_cast<void*>(dst + chunk * 16), v.x, v.y, v.z, v.w);
                            }
                        }
                    }
                } else if (via_tma && warp_has_rows) {
                    // 32 columns (64 bytes of BF16 per row) per TMA store; rows past rows_store hold whatever the MMA
                    // produced from the tile's padding rows and land in padding rows of D
                    const int x0 = t.n_block * BLOCK_N + static_cast<int>(half) * kCols;
#pragma unroll
                    for (int c = 0; c < kCols / 32; ++c) {
                        if (lane == 0) bulk_wait_group_read_all();  // the previous slab has left the staging buffer
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *stage_chunk(i) = make_uint4(
                                pack_bf16x2(__uint_as_float(acc[c * 32 + i * 8 + 0]), __uint_as_float(acc[c * 32 + i * 8 + 1])),
                                pack_bf16x2(__uint_as_float(acc[c * 32 + i * 8 + 2]), __uint_as_float(acc[c * 32 + i * 8 + 3])),
                                pack_bf16x2(__uint_as_float(acc[c * 32 + i * 8 + 4]), __uint_as_float(acc[c * 32 + i * 8 + 5])),
                                pack_bf16x2(__uint_as_float(acc[c * 32 + i * 8 + 6]), __uint_as_float(acc[c * 32 + i * 8 + 7])));
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tm_out, stage_buf, x0 + c * 32, t.row_start + static_cast<int>(q) * 32);
                            bulk_commit_group();
                        }
                    }
                }
            }
            if constexpr (L::kStageBytesPerWarp != 0 && EPI == kEpiSwiGLU) {
                if (via_tma && warp_has_rows) {
                    if (lane == 0) bulk_wait_group_read_all();  // the previous tile's slab has left the staging buffer
                    __syncwarp();
                }
            }
            if constexpr (EPI == kEpiF32Acc) {
                // D += accumulator through TMA reductions (FP32 add in the memory system; d already holds c): the warp's
                // 32 rows x 16 columns per slab, coalesced, and no read of c through the load/store pipe. Row-per-thread
                // loads and stores of FP32 tiles cost more than the MMAs of a tile with a short K extent.
                if (via_tma && warp_has_rows && t.num_kb != 0) {
                    const int x0 = t.n_block * BLOCK_N + static_cast<int>(half) * kCols;
                    const int y0 = t.group * p.m + t.row_start + static_cast<int>(q) * 32;
#pragma unroll
                    for (int c = 0; c < kCols / 16; ++c) {
                        if (lane == 0) bulk_wait_group_read_all();  // the previous slab has left the staging buffer
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *stage_chunk(i) = make_uint4(acc[c * 16 + i * 4 + 0], acc[c * 16 + i * 4 + 1], acc[c * 16 + i * 4 + 2],
                                                         acc[c * 16 + i * 4 + 3]);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_reduce_add_2d(&tm_out, stage_buf, x0 + c * 16, y0);
                            bulk_commit_group();
                        }
                    }
                }
            }
            if constexpr (EPI == kEpiSwiGLUBf16) {
                // Same column order and arithmetic as the FP8 form below, the outputs stay BF16 (reference:
                // deep_gemm/include/deep_gemm/impls/sm100_bf16_mega_moe.cuh:927-955). One 32-output group is one
                // 32 x 64-byte slab of the warp: staged in shared memory and stored by TMA like the BF16 epilogue's, or
                // written row by row where the tile's tail rows must stay untouched.
                if (warp_has_rows) {
                    const float w = (p.row_weight != nullptr && (store || via_tma)) ? __ldg(p.row_weight + row) : 1.0f;
#pragma unroll
                    for (int c = 0; c < kCols / 64; ++c) {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float o[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                float gv = bf16_round(__uint_as_float(acc[c * 32 + i * 2 + h]));
                                float uv = bf16_round(__uint_as_float(acc[kCols / 2 + c * 32 + i * 2 + h]));
                                if (p.clamp > 0.0f) {
                                    gv = fminf(gv, p.clamp);
                                    uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                                }
                                const float silu = p.fast_math ? gv * rcp_approx(1.0f + __expf(-gv))
                                                               : gv / (1.0f + expf(-gv));
                                o[h] = silu * uv * w;
                            }
                            packed[i] = pack_bf16x2(o[0], o[1]);
                        }
                        const int j = t.n_block * (BLOCK_N / 2) + static_cast<int>(half) * (kCols / 2) + c * 32;
                        if (via_tma) {
                            if (lane == 0) bulk_wait_group_read_all();  // the previous slab has left the staging buffer
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                *stage_chunk(i) = make_uint4(packed[i * 4], packed[i * 4 + 1], packed[i * 4 + 2], packed[i * 4 + 3]);
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) {
                                tma_store_2d(&tm_out, stage_buf, j, t.row_start + static_cast<int>(q) * 32);
                                bulk_commit_group();
                            }
                        } else if (store) {
                            unsigned char* dst = p.act_q + row * p.act_q_row_stride + j * 2;
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                st_global_v4(dst + i * 16, packed[i * 4], packed[i * 4 + 1], packed[i * 4 + 2], packed[i * 4 + 3]);
                        }
                    }
                }
            }
            if (store) {
                if constexpr (EPI == kEpiBF16 || EPI == kEpiF32) {
                    const long long col0 = static_cast<long long>(t.n_block) * BLOCK_N + half * kCols;
                    if constexpr (EPI == kEpiF32) {
                        float* dst = reinterpret_cast<float*>(p.d) + row * p.d_row_stride + col0;
                        if (p.accumulate) {
#pragma unroll
                            for (int i = 0; i < kCols / 4; ++i) {
                                const float4 old = *reinterpret_cast<const float4*>(dst + i * 4);
                                st_global_v4(dst + i * 4, __float_as_uint(old.x + __uint_as_float(acc[i * 4 + 0])),
                                             __float_as_uint(old.y + __uint_as_float(acc[i * 4 + 1])),
                                             __float_as_uint(old.z + __uint_as_float(acc[i * 4 + 2])),
                                             __float_as_uint(old.w + __uint_as_float(acc[i * 4 + 3])));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < kCols / 4; ++i)
                                st_global_v4(dst + i * 4, acc[i * 4 + 0], acc[i * 4 + 1], acc[i * 4 + 2], acc[i * 4 + 3]);
                        }
                    } else if (!via_tma && p.ret_src == nullptr) {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.d) + row * p.d_row_stride + col0;
#pragma unroll
                        for (int i = 0; i < kCols / 8; ++i)
                            st_global_v4(dst + i * 8,
                                         pack_bf16x2(__uint_as_float(acc[i * 8 + 0]), __uint_as_float(acc[i * 8 + 1])),
                                         pack_bf16x2(__uint_as_float(acc[i * 8 + 2]), __uint_as_float(acc[i * 8 + 3])),
                                         pack_bf16x2(__uint_as_float(acc[i * 8 + 4]), __uint_as_float(acc[i * 8 + 5])),
                                         pack_bf16x2(__uint_as_float(acc[i * 8 + 6]), __uint_as_float(acc[i * 8 + 7])));
                    }
                } else if constexpr (EPI == kEpiF32Acc) {
                    // tiles with fewer than 128 rows (the tail of m): d += accumulator row by row (d already holds c; an
                    // empty group adds nothing: its accumulator was never written)
                    if (!via_tma && t.num_kb != 0) {
                        const long long off = (static_cast<long long>(t.group) * p.m + row) * p.d_row_stride +
                                              static_cast<long long>(t.n_block) * BLOCK_N + half * kCols;
                        float* dst = reinterpret_cast<float*>(p.d) + off;
#pragma unroll
                        for (int i = 0; i < kCols / 4; ++i) {
                            const float4 cv = *reinterpret_cast<const float4*>(dst + i * 4);
                            st_global_v4(dst + i * 4, __float_as_uint(cv.x + __uint_as_float(acc[i * 4 + 0])),
                                         __float_as_uint(cv.y + __uint_as_float(acc[i * 4 + 1])),
                                         __float_as_uint(cv.z + __uint_as_float(acc[i * 4 + 2])),
                                         __float_as_uint(cv.w + __uint_as_float(acc[i * 4 + 3])));
                        }
                    }
                } else if constexpr (EPI == kEpiSwiGLUNvfp4) {
                    // Same column order as below; the 32 outputs of a gate/up pair are requantised to NVFP4: two
                    // UE4M3 block scales (16 outputs each) against the calibrated per-tensor scale out_scale[0].
                    const float w = p.row_weight != nullptr ? __ldg(p.row_weight + row) : 1.0f;
                    const float s_out = __ldg(p.out_scale);
#pragma unroll
                    for (int c = 0; c < kCols / 64; ++c) {
                        float o[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float gv = bf16_round(__uint_as_float(acc[c * 32 + i]));
                            float uv = bf16_round(__uint_as_float(acc[kCols / 2 + c * 32 + i]));
                            if (p.clamp > 0.0f) {
                                gv = fminf(gv, p.clamp);
                                uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                            }
                            const float silu = p.fast_math ? gv * rcp_approx(1.0f + __expf(-gv))
                                                           : gv / (1.0f + expf(-gv));
                            o[i] = silu * uv * w;
                        }
                        const int j = t.n_block * (BLOCK_N / 2) + static_cast<int>(half) * (kCols / 2) + c * 32;
                        uint32_t packed[4];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float amax = 0.0f;
#pragma unroll
                            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(o[h * 16 + i]));
                            const uint32_t sf_byte = e4m3_byte(amax / 6.0f / s_out);
                            const float factor = e4m3_to_float(sf_byte) * s_out;
                            // one reciprocal and the hardware E2M1 conversion instead of 16 divisions and threshold
                            // ladders: this epilogue otherwise costs more than the tile's MMAs
                            const float rcp = factor > 0.0f ? 1.0f / factor : 0.0f;
                            float scaled[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) scaled[i] = o[h * 16 + i] * rcp;
                            packed[h * 2] = pack_e2m1x8_rn(scaled);
                            packed[h * 2 + 1] = pack_e2m1x8_rn(scaled + 8);
                            const int jb = j + h * 16;
                            p.act_sf[(static_cast<long long>(jb / 64) * p.act_sf_k_stride + sf_row) * 4 + ((jb / 16) & 3)] =
                                static_cast<unsigned char>(sf_byte);
                        }
                        st_global_v4(p.act_q + row * p.act_q_row_stride + j / 2, packed[0], packed[1], packed[2], packed[3]);
                    }
                } else if constexpr (EPI == kEpiSwiGLUBf16) {
                    // handled above, warp-uniformly (its staged stores need the whole warp)
                } else {
                    // acc[0, kCols / 2) are gate channels, acc[kCols / 2, kCols) the matching up channels (see the drain
                    // above); one 32-wide output group = one UE8M0 scale.
                    const float w = p.row_weight != nullptr ? __ldg(p.row_weight + row) : 1.0f;
#pragma unroll
                    for (int c = 0; c < kCols / 64; ++c) {
                        float o[32];
                        float amax = 0.0f;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            float gv = bf16_round(__uint_as_float(acc[c * 32 + i]));
                            float uv = bf16_round(__uint_as_float(acc[kCols / 2 + c * 32 + i]));
                            if (p.clamp > 0.0f) {
                                gv = fminf(gv, p.clamp);
                                uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                            }
                            const float silu = p.fast_math ? gv * rcp_approx(1.0f + __expf(-gv))
                                                           : gv / (1.0f + expf(-gv));
                            o[i] = silu * uv * w;
                            amax = fmaxf(amax, fabsf(o[i]));
                        }
                        float sf_inv;
                        uint32_t sf_byte;
                        ue8m0_scale_for_amax(amax, sf_inv, sf_byte);
                        const int j = t.n_block * (BLOCK_N / 2) + static_cast<int>(half) * (kCols / 2) + c * 32;
                        uint32_t packed[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const __nv_fp8x4_e4m3 q4(make_float4(o[i * 4 + 0] * sf_inv, o[i * 4 + 1] * sf_inv,
                                                                 o[i * 4 + 2] * sf_inv, o[i * 4 + 3] * sf_inv));
                            packed[i] = q4.__x;
                        }
                        if (via_tma) {
                            *stage_chunk(2 * c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            *stage_chunk(2 * c + 1) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        } else {
                            unsigned char* dst = p.act_q + row * p.act_q_row_stride + j;
                            st_global_v4(dst, packed[0], packed[1], packed[2], packed[3]);
                            st_global_v4(dst + 16, packed[4], packed[5], packed[6], packed[7]);
                        }
                        p.act_sf[(static_cast<long long>(j / 128) * p.act_sf_k_stride + sf_row) * 4 + ((j / 32) & 3)] =
                            static_cast<unsigned char>(sf_byte);
                    }
                }
            }
            if constexpr (L::kStageBytesPerWarp != 0 && EPI == kEpiSwiGLU) {
                if (via_tma && warp_has_rows) {
                    // one 32 x 64-byte slab of FP8 activations per warp and tile (rows past rows_store keep stale bytes
                    // and land in padding rows)
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_out, stage_buf, t.n_block * (BLOCK_N / 2) + static_cast<int>(half) * (kCols / 2),
                                     t.row_start + static_cast<int>(q) * 32);
                        bulk_commit_group();
                    }
                }
            }
            if constexpr (kPushes) push_rows(2);  // a couple of rows of the next phase's dispatch per tile
        }
        if constexpr (kPushes) push_rows(0x7fffffff);  // whatever is left of this warp's share
        if (L::kStageBytesPerWarp != 0 && lane == 0) bulk_wait_group_all();  // stores still in flight read this CTA's shared memory
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag != 0) {
        // Let copies and MMAs that were already issued land before shared and tensor memory are released.
        __nanosleep(100000);
        __syncthreads();
    }
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace dgb
