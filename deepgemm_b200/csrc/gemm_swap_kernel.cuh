// Swapped-operand grouped GEMM for the MoE layer: weight channels on the UMMA M side, tokens on the N side.
//
// The kernel in gemm_kernel.cuh puts 128 token rows on M, so an expert with 129..160 rows costs a second full pass over
// its weights for a handful of rows (a third of all tiles at 128 +- 11 rows per expert). Here one tile is
// 256 weight rows (two accumulators of 128 TMEM lanes each) x all tokens of the expert (UMMA N = tokens rounded up to
// 16, at most kSwapMaxTok): every expert with up to kSwapMaxTok rows is one pass, and the MMA time follows the token
// count. Experts with more rows are cut into 128-row token tiles. This is the orientation the reference's fused kernel
// uses (swap-AB, deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:754,984; BLOCK_M = tokens by expected
// rows per expert, csrc/jit_kernels/heuristics/mega_moe.hpp:81-102), rebuilt on this library's pipeline.
//
//   D^T[256 channels, tokens] = W[256, K] . X[tokens, K]^T     FP8 (E4M3) tokens x MXFP4 (E2M1) weights, UE8M0 per 32
//
// Layer path only: psum layout with 128-row expert segments, scale factors of both operands in tcgen05.cp row order,
// gate/up rows interleaved by 128 (accumulator 0 = 128 gate channels, accumulator 1 = the matching up channels).
// An epilogue thread owns one channel (TMEM lane) and walks the tokens (TMEM columns):
//   SwiGLU: bf16(gate), bf16(up) -> clamp -> silu(gate) * up * weight[token] -> amax over the warp's 32 channels (one
//           UE8M0 scale group) -> e4m3; a warp writes the 32 bytes of one token's scale group at a time.
//   BF16:   a warp writes 64 contiguous bytes of one token's output row at a time.
// Roles, barriers, bounded waits and the status block are those of gemm_kernel.cuh.
#pragma once

#include "gemm_kernel.cuh"

namespace dgb {

constexpr int kSwapMaxTok = 160;  // tokens per tile = largest UMMA N used (multiple of 16)
constexpr int kSwapStages = 4;

struct SwapSmem {
    static constexpr int kWBytes = 256 * 128;          // 256 weight rows x 128 K bytes (packed FP4 expanded by TMA)
    static constexpr int kXBytes = kSwapMaxTok * 128;  // token rows x 128 K bytes
    static constexpr int kSfwBytes = 2 * 512;          // one packed scale int per weight row
    static constexpr int kSfxBytes = 2 * 512;          // one packed scale int per token row (256-row box, 160 used)
    static constexpr int kOffW = 0;
    static constexpr int kOffX = kOffW + kSwapStages * kWBytes;
    static constexpr int kOffSfw = kOffX + kSwapStages * kXBytes;
    static constexpr int kOffSfx = kOffSfw + kSwapStages * kSfwBytes;
    static constexpr int kOffBar = kOffSfx + kSwapStages * kSfxBytes;
    static constexpr int kNumBars = 2 * kSwapStages + 2;
    static constexpr int kOffMisc = kOffBar + kNumBars * 8;
    static constexpr int kOffGroups = kOffMisc + 16;
    static constexpr int kTotal = kOffGroups + 3 * kMaxCachedGroups * 4;
    static constexpr int kDynamicBytes = kTotal + 1024;
    static_assert(kXBytes % 1024 == 0, "token tiles must keep the 1024-byte alignment of the 128-byte swizzle");
};

struct SwapTile {
    int group;      // expert
    int w_block;    // 256-row block of the expert's weight matrix
    int row_start;  // first token row of the tile in the expert-sorted buffers (a multiple of 128)
    int tokens;     // valid token rows of the tile (1 .. kSwapMaxTok)
};

// Token tiles of a group: one tile while the group fits kSwapMaxTok rows, else 128-row tiles (so that every tile starts
// on a 128-row boundary of the scale-factor layout).
__host__ __device__ inline int swap_token_tiles(int rows) { return rows <= 0 ? 0 : (rows <= kSwapMaxTok ? 1 : (rows + 127) / 128); }

// Walks the tiles of this CTA: groups in order, token tiles outer, weight blocks inner (an expert's weights are read
// once per token tile, its tokens stay in L2). Uses the per-group table the prologue staged in shared memory.
struct SwapScheduler {
    const int* lay;        // psum ends
    const int* start;      // first row of each group
    const int* tiles_end;  // running tile count
    int num_groups, num_w_blocks;
    int tile, g;

    __device__ SwapScheduler(const int* lay_, const int* start_, const int* tiles_end_, int num_groups_, int num_w_blocks_)
        : lay(lay_), start(start_), tiles_end(tiles_end_), num_groups(num_groups_), num_w_blocks(num_w_blocks_),
          tile(static_cast<int>(blockIdx.x)), g(0) {}

    __device__ bool next(SwapTile& t) {
        while (g < num_groups && tile >= tiles_end[g]) ++g;
        if (g >= num_groups) return false;
        int local = tile - (g == 0 ? 0 : tiles_end[g - 1]);
        const int rows = lay[g] - start[g];
        int tt = 0;
        while (local >= num_w_blocks) { local -= num_w_blocks; ++tt; }
        t.group = g;
        t.w_block = local;
        t.row_start = start[g] + tt * 128;
        t.tokens = rows <= kSwapMaxTok ? rows : min(128, rows - tt * 128);
        tile += static_cast<int>(gridDim.x);
        return true;
    }
};

// tm_x: tokens [rows, K] bytes, box 128 x kSwapMaxTok; tm_w: weights (16U4_ALIGN16B) box 128 x 256;
// tm_sfx / tm_sfw: packed scale ints, box 256 x 1. p: the GemmParams of the layer call (psum layout, alignment 128).
template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
dgb200_swap_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                        const __grid_constant__ CUtensorMap tm_sfx, const __grid_constant__ CUtensorMap tm_sfw,
                        const __grid_constant__ GemmParams p) {
    using L = SwapSmem;
    constexpr int kStages = kSwapStages;
    constexpr uint32_t kAcc1Col = kSwapMaxTok;           // accumulator 0: columns [0, 160), accumulator 1: [160, 320)
    constexpr uint32_t kSfCol0 = 2 * kSwapMaxTok;
    constexpr uint32_t kSfColsPerStage = 16;             // weights 2 x 4, tokens 2 x 4
    constexpr uint32_t kTmemCols = 512;
    static_assert(kSfCol0 + kStages * kSfColsPerStage <= kTmemCols, "TMEM budget");
    static_assert(EPI == kEpiSwiGLU || EPI == kEpiBF16, "epilogues of the layer path");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + kStages;
    uint64_t* tmem_full_bar = bars + 2 * kStages;
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 1;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kOffMisc + 4);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const int num_w_blocks = p.n / 256;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(full_bar + i, 2);   // token loader and weight loader
            mbar_init(empty_bar + i, 1);  // tcgen05.commit of the MMA issuer
        }
        mbar_init(tmem_full_bar, 1);
        mbar_init(tmem_empty_bar, 8);     // lane 0 of each epilogue warp
        fence_mbar_init();
        prefetch_tensormap(&tm_x);
        prefetch_tensormap(&tm_w);
        prefetch_tensormap(&tm_sfx);
        prefetch_tensormap(&tm_sfw);
    }
    // per-group table: layout word, first row, running tile count (host guarantees num_groups <= kMaxCachedGroups)
    int* group_lay = reinterpret_cast<int*>(smem + L::kOffGroups);
    int* group_start = group_lay + kMaxCachedGroups;
    int* group_tiles_end = group_start + kMaxCachedGroups;
    for (int i = threadIdx.x; i < p.num_groups; i += kGemmThreads) {
        const int prev_end = i == 0 ? 0 : __ldg(p.layout + i - 1);
        const int start = (prev_end + 127) / 128 * 128;
        const int end = __ldg(p.layout + i);
        group_lay[i] = end;
        group_start[i] = start;
        group_tiles_end[i] = (group_selected(p, end - start) && group_in_range(p, i)) ? swap_token_tiles(end - start) * num_w_blocks : 0;
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
    if (warp == 2) tmem_alloc(tmem_ptr_smem, kTmemCols);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    const int num_kb = p.k / 128;

    if (warp < 4) {
    setmaxnreg_dec<kRegsControlWarps>();
    if (warp == 0) {
        // ---------------------------------------------------------------- loader: token rows + their scale ints
        SwapScheduler sched(group_lay, group_start, group_tiles_end, p.num_groups, num_w_blocks);
        SwapTile t;
        uint32_t stage = 0, phase = 0;
        const bool leader = elect_one();
        bool ok = true;
        while (ok && sched.next(t)) {
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, kTimeoutEmpty, kb);
                if (!ok) break;
                if (leader) {
                    mbar_arrive_expect_tx(full_bar + stage, L::kXBytes + L::kSfxBytes);
                    tma_load_2d(smem + L::kOffX + stage * L::kXBytes, &tm_x, full_bar + stage, kb * 128, t.row_start);
                    tma_load_2d(smem + L::kOffSfx + stage * L::kSfxBytes, &tm_sfx, full_bar + stage, t.row_start, kb);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 3) {
        // ---------------------------------------------------------------- loader: weight rows + their scale ints
        SwapScheduler sched(group_lay, group_start, group_tiles_end, p.num_groups, num_w_blocks);
        SwapTile t;
        uint32_t stage = 0, phase = 0;
        const bool leader = elect_one();
        bool ok = true;
        while (ok && sched.next(t)) {
            const int w_row = t.group * p.n + t.w_block * 256;
            const int sfw_y = t.group * p.sfb_packed_k;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, kTimeoutEmpty, kb);
                if (!ok) break;
                if (leader) {
                    mbar_arrive_expect_tx(full_bar + stage, p.b_tx_bytes + L::kSfwBytes);
                    tma_load_2d(smem + L::kOffW + stage * L::kWBytes, &tm_w, full_bar + stage, kb * 128, w_row);
                    tma_load_2d(smem + L::kOffSfw + stage * L::kSfwBytes, &tm_sfw, full_bar + stage, t.w_block * 256, sfw_y + kb);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        SwapScheduler sched(group_lay, group_start, group_tiles_end, p.num_groups, num_w_blocks);
        SwapTile t;
        uint32_t stage = 0, phase = 0, iter = 0;
        const uint32_t w_base = smem_u32(smem + L::kOffW), x_base = smem_u32(smem + L::kOffX);
        const uint32_t sfw_smem = smem_u32(smem + L::kOffSfw), sfx_smem = smem_u32(smem + L::kOffSfx);
        const bool leader = elect_one();
        bool ok = true;
        while (ok && sched.next(t)) {
            ok = mbar_wait(tmem_empty_bar, (iter & 1) ^ 1, abort_flag, kTimeoutTmemEmpty, static_cast<int>(iter));
            ++iter;
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t n_tok = static_cast<uint32_t>((t.tokens + 15) & ~15);
            // weights are the A operand (E2M1 in byte containers or E4M3), tokens the B operand (E4M3)
            const uint32_t idesc = make_idesc_block_scaled(p.b_fmt, kFmtE4M3, 128, n_tok, kScaleUE8M0);
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(full_bar + stage, phase, abort_flag, kTimeoutFull, kb);
                if (!ok) break;
                if (leader) {
                    const uint32_t sf_cols = tmem_base + kSfCol0 + stage * kSfColsPerStage;
                    const uint32_t tmem_sfw = sf_cols, tmem_sfx = sf_cols + 8;
                    tcgen05_cp_32x128b_warpx4(tmem_sfw, make_sf_desc(sfw_smem + stage * L::kSfwBytes));
                    tcgen05_cp_32x128b_warpx4(tmem_sfw + 4, make_sf_desc(sfw_smem + stage * L::kSfwBytes + 512));
                    tcgen05_cp_32x128b_warpx4(tmem_sfx, make_sf_desc(sfx_smem + stage * L::kSfxBytes));
                    if (n_tok > 128) tcgen05_cp_32x128b_warpx4(tmem_sfx + 4, make_sf_desc(sfx_smem + stage * L::kSfxBytes + 512));
                    const uint64_t wdesc = make_kmajor_sw128_desc(w_base + stage * L::kWBytes);
                    const uint64_t xdesc = make_kmajor_sw128_desc(x_base + stage * L::kXBytes);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4) {
                        const uint32_t id = idesc_with_sf_ids(idesc, k4, k4);
                        const uint32_t acc = (kb | k4) != 0 ? 1u : 0u;
                        // rows 0..127 of the weight tile -> accumulator 0, rows 128..255 (16 KB further) -> accumulator 1
                        tcgen05_mma_mxf8f6f4(tmem_base, wdesc + k4 * 2, xdesc + k4 * 2, id, tmem_sfw, tmem_sfx, acc);
                        tcgen05_mma_mxf8f6f4(tmem_base + kAcc1Col, wdesc + (16384 >> 4) + k4 * 2, xdesc + k4 * 2, id, tmem_sfw + 4,
                                             tmem_sfx, acc);
                    }
                    tcgen05_commit(empty_bar + stage);
                    if (kb == num_kb - 1) tcgen05_commit(tmem_full_bar);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    }
    } else {
        setmaxnreg_inc<kRegsEpilogueWarps>();
        // ---------------------------------------------------------------- epilogue (8 warps)
        // Warp w reads TMEM lanes [32 (w % 4), +32) = 32 channels of each accumulator; the two warps of a lane quarter
        // split the token columns in halves. Everything is drained to registers first so that the MMA issuer can start
        // the next tile.
        constexpr int kHalf = kSwapMaxTok / 2;  // token columns per thread and accumulator
        SwapScheduler sched(group_lay, group_start, group_tiles_end, p.num_groups, num_w_blocks);
        SwapTile t;
        uint32_t iter = 0;
        const uint32_t q = warp & 3, half = (warp - 4) >> 2;
        const int channel = static_cast<int>(q * 32 + lane);  // within the 128-channel block of each accumulator
        bool ok = true;
        while (ok && sched.next(t)) {
            ok = mbar_wait<32>(tmem_full_bar, iter & 1, abort_flag, kTimeoutTmemFull, static_cast<int>(iter));
            ++iter;
            if (!ok) break;
            tcgen05_fence_after();
            const int col0 = static_cast<int>(half) * kHalf;
            const int my_tokens = min(max(t.tokens - col0, 0), kHalf);  // warp-uniform
            uint32_t a0[kHalf], a1[kHalf];
            const uint32_t lane_base = tmem_base + ((q * 32u) << 16) + static_cast<uint32_t>(col0);
#pragma unroll
            for (int c = 0; c < kHalf / 16; ++c) {
                if (c * 16 < my_tokens) {
                    tmem_ld_32x32b_x16(lane_base + c * 16, a0 + c * 16);
                    tmem_ld_32x32b_x16(lane_base + kAcc1Col + c * 16, a1 + c * 16);
                }
            }
            tmem_ld_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty_bar);

            if constexpr (EPI == kEpiSwiGLU) {
                // accumulator 0 = gate channels, accumulator 1 = up channels of output channels j .. j + 127
                const int j = t.w_block * 128 + channel;
                const long long row0 = static_cast<long long>(t.row_start) + col0;
                unsigned char* q_ptr = p.act_q + row0 * p.act_q_row_stride + j;
                const long long sf_k = static_cast<long long>(j >> 7) * p.act_sf_k_stride;
                // routing weights of this half's tokens: lane l holds tokens l, l + 32, l + 64 (no loads inside the token loop)
                float w_reg[(kHalf + 31) / 32];
#pragma unroll
                for (int c = 0; c < (kHalf + 31) / 32; ++c) {
                    const int i = c * 32 + static_cast<int>(lane);
                    w_reg[c] = (p.row_weight != nullptr && i < my_tokens) ? __ldg(p.row_weight + row0 + i) : 1.0f;
                }
#pragma unroll
                for (int i = 0; i < kHalf; ++i) {
                    if (i < my_tokens) {
                        const float w = __shfl_sync(0xffffffffu, w_reg[i / 32], i % 32);
                        float gv = bf16_round(__uint_as_float(a0[i]));
                        float uv = bf16_round(__uint_as_float(a1[i]));
                        if (p.clamp > 0.0f) {
                            gv = fminf(gv, p.clamp);
                            uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                        }
                        const float silu = p.fast_math ? gv * rcp_approx(1.0f + __expf(-gv)) : gv / (1.0f + expf(-gv));
                        const float o = silu * uv * w;
                        // the warp's 32 channels are one scale group: non-negative floats order like their bit patterns
                        const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(o))));
                        float sf_inv;
                        uint32_t sf_byte;
                        ue8m0_scale_for_amax(amax, sf_inv, sf_byte);
                        q_ptr[static_cast<long long>(i) * p.act_q_row_stride] =
                            __nv_cvt_float_to_fp8(o * sf_inv, __NV_SATFINITE, __NV_E4M3);
                        if (lane == 0)
                            p.act_sf[(sf_k + sf_row_in_cp_order(row0 + i)) * 4 + q] = static_cast<unsigned char>(sf_byte);
                    }
                }
            } else {
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.d) + t.w_block * 256 + channel;
#pragma unroll
                for (int i = 0; i < kHalf; ++i) {
                    if (i < my_tokens) {
                        const long long row = static_cast<long long>(t.row_start) + col0 + i;
                        out[row * p.d_row_stride] = __float2bfloat16_rn(__uint_as_float(a0[i]));
                        out[row * p.d_row_stride + 128] = __float2bfloat16_rn(__uint_as_float(a1[i]));
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag != 0) {
        __nanosleep(100000);  // let copies and MMAs that were already issued land before memory is released
        __syncthreads();
    }
    if (warp == 2) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace dgb
