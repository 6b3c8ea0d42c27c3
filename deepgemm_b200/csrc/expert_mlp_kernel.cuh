// Both grouped GEMMs of the FP8 x MXFP4 MoE layer in ONE persistent kernel on CTA pairs:
//   gate/up:  A2[rows, I]   = requant_fp8( silu(X W1g^T) * (X W1u^T) * routing weight )     (task phase 0)
//   down:     OUT[rows, H]  = bf16( A2 W2^T )                                                (task phase 1)
//
// Replaces, for that layer, the reference's fused kernel body and scheduler: the 2-CTA swap-AB main loop
// (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:669-919), its SwiGLU / BF16 epilogues (:987-1305) and the
// MegaMoEScheduler that interleaves gate/up and down tasks behind dependency counters
// (deep_gemm/include/deep_gemm/scheduler/mega_moe.cuh:152-415), with the tile choice of
// csrc/jit_kernels/heuristics/mega_moe.hpp:81-112 (cluster of two, tokens on UMMA N sized to the expert).
//
// Orientation ("swap AB"): weight rows sit on the UMMA M side, an expert's tokens on the N side.
//   * kPair: a cluster of two CTAs issues tcgen05.mma.cta_group::2 with M = 256: each CTA holds 128 weight rows and
//     accumulates them in its own tensor memory (128 lanes x N columns); the N token rows are split half / half between
//     the two CTAs' shared memory and read by both tensor cores. Each CTA loads its own halves with ordinary per-CTA TMA
//     loads that complete on the leader CTA's mbarrier; nothing is multicast. One thread of the leader issues the scale
//     copies, MMAs and commits for the pair.
//   * !kPair: the same code on single CTAs (cta_group::1, M = 128), for bring-up and as a fallback.
//   UMMA N = the tile's token count rounded up to 16 (at most kMlpMaxTok), so the MMA time follows the expert's size:
//   an expert of up to kMlpMaxTok rows is ONE pass over its weights, larger ones are cut into 128-row token tiles.
//
// Schedule: token tiles are numbered expert by expert. Tasks = (phase, token tile, weight block); they are dealt to the
// clusters round-robin from one sequence that every warp role derives by itself:
//   gate/up(tile group 0), gate/up(group 1), down(group 0), gate/up(group 2), down(group 1), ... , down(last group)
// A down task reads the activations every gate/up task of the same token tile wrote: each finished gate/up task adds to
// tile_done[tile] (release), the down task's token loader waits for the full count (acquire, bounded). The one-group lag
// means the count is normally complete long before it is needed, and a tile's activations are still in L2.
// Deadlock freedom: a task only depends on tasks earlier in the sequence, clusters take their tasks in sequence order and
// all clusters are co-resident (grid <= SM count, one CTA per SM).
//
// Accumulators are double-buffered in tensor memory (2 x kMlpMaxTok columns), so the epilogue of one task overlaps the
// MMAs of the next; it walks its accumulator in chunks of 16 token columns:
//   gate/up: weight rows are gate/up-interleaved by 16, so a warp's 32 lanes hold 16 gate and the 16 matching up rows;
//            lanes exchange halves with one shuffle per value, every lane then owns (one output channel, 8 tokens):
//            bf16 rounding -> clamp -> silu(gate) * up * weight -> amax over the 32 channels of a scale group (16 lanes
//            here + the neighbouring warp's 16 through shared memory) -> UE8M0 -> E4M3; for a fixed token the lanes hold
//            consecutive channels, so each store instruction writes contiguous bytes of the token's activation row; the
//            scale bytes go straight to the tcgen05.cp-ordered scale buffer.
//   down:    bf16 rounding; a store instruction writes 64 contiguous bytes of one token's output row.
// Every wait on an mbarrier or a flag is bounded; a timeout is reported through the status block and unwinds the CTA.
#pragma once

#include "gemm_kernel.cuh"

namespace dgb {

constexpr int kMlpMaxTok = 160;  // token rows of one tile = largest UMMA N used (a multiple of 32)
constexpr int kMlpThreads = 384;
constexpr int kMlpChunk = 16;    // token columns the epilogue handles at a time
constexpr int kMlpGateUpInterleave = 16;
constexpr int kMlpMaxExperts = 384;  // experts per rank whose tables fit next to the operand ring in shared memory

struct MlpPhase {
    int n;                // weight rows of the GEMM (2 x intermediate for gate/up, hidden for down)
    int k;                // reduction length
    unsigned w_tx_bytes;  // bytes one 128-row weight box credits to the mbarrier (packed FP4: 8192, E4M3: 16384)
    unsigned w_fmt;       // kFmtE2M1_F8F6F4 or kFmtE4M3
};

struct MlpParams {
    const int* expert_end;  // psum layout: end row of each expert; expert e starts at align(end[e - 1], 128)
    int num_experts;
    int phase_mask;         // bit 0: gate/up tasks, bit 1: down tasks
    int tiles_per_group;    // token tiles per schedule group
    MlpPhase ph[2];
    // gate/up epilogue: e4m3 activations [rows, I] and their scales; down epilogue: bf16 rows [rows, H]
    unsigned char* act_q;
    long long act_q_row_stride;  // bytes
    __nv_bfloat16* out;
    long long out_row_stride;    // elements
    unsigned char* act_sf;       // packed UE8M0 bytes of the activations: ((j / 128) * act_sf_k_stride + cp_row) * 4 + (j / 32) % 4
    long long act_sf_k_stride;   // ints
    const float* row_weight;     // per row of the expert-sorted buffers, may be null (weight 1)
    float clamp;                 // <= 0: no clamp
    int fast_math;
    unsigned* tile_done;         // one counter per token tile, zero when the kernel starts
};

constexpr int kMlpXMaps = kMlpMaxTok / 16;
struct MlpMaps {  // first index = phase
    CUtensorMap x[2][kMlpXMaps];  // token rows [rows, K] bytes: map i has a box of 128 B x 16 (i + 1) rows (128-byte swizzle)
    CUtensorMap w[2];             // weights as a tall tensor of tile rows [tiles x 128, 128 K elements], box 128 x 256 (two tiles)
    CUtensorMap sfx[2], sfw[2];   // packed scale ints, box 128 x 2 (two K blocks)
};

constexpr int kMlpKbPerStage = 2;  // K blocks (of 128) per pipeline stage

template <bool kPair>
struct MlpSmem {
    static constexpr int kCtas = kPair ? 2 : 1;
    static constexpr int kXRows = kMlpMaxTok / kCtas;
    static constexpr int kStages = kPair ? 4 : 2;  // stages of two K blocks (the single-CTA form holds twice the token rows per stage)
    static constexpr int kWBytes = 128 * 128;      // one weight tile: 128 rows x 128 K elements, one byte per element
    static constexpr int kXBytes = kXRows * 128;   // token rows of one K block
    static constexpr int kWStageBytes = kMlpKbPerStage * kWBytes;
    static constexpr int kXStageBytes = kMlpKbPerStage * kXBytes;
    static constexpr int kSfwStageBytes = kMlpKbPerStage * 512;       // [K block][128 ints]
    static constexpr int kSfxStageBytes = 2 * kMlpKbPerStage * 512;   // [box of 128 rows][K block][128 ints]
    static constexpr int kOffW = 0;
    static constexpr int kOffX = kOffW + kStages * kWStageBytes;
    static constexpr int kOffSfw = kOffX + kStages * kXStageBytes;
    static constexpr int kOffSfx = kOffSfw + kStages * kSfwStageBytes;
    static constexpr int kOffXch = kOffSfx + kStages * kSfxStageBytes;  // amax exchange between neighbouring warps: [2 warpgroups][2][2 pairs][2 warps][16]
    static constexpr int kOffTables = kOffXch + 1024;                   // expert end rows, running token-tile counts
    static constexpr int kOffBar = kOffTables + 2 * kMlpMaxExperts * 4;
    static constexpr int kNumBars = 2 * kStages + 4;
    static constexpr int kOffMisc = kOffBar + kNumBars * 8;
    static constexpr int kTotal = kOffMisc + 16;
    static_assert(kXBytes % 1024 == 0 && kOffX % 1024 == 0, "operand stages must keep the 1024-byte alignment of the 128-byte swizzle");
    static_assert(kTotal <= 232448, "shared memory budget");
};

__host__ __device__ inline int mlp_token_tiles(int rows) { return rows <= 0 ? 0 : (rows <= kMlpMaxTok ? 1 : (rows + 127) / 128); }

struct MlpTask {
    int phase, expert, tile, w_block;  // w_block counts blocks of 128 x (CTAs per cluster) weight rows
    int row_start, tokens;
};

// The task sequence of this cluster (see the header comment). `ends` and `tiles_end` are the shared-memory tables.
struct MlpScheduler {
    const int* ends;
    const int* tiles_end;
    int num_experts, total_tiles, gt, num_groups, mask, nb0, nb1;
    int task, stride;
    int q, num_segments, seg_start, seg_len, seg_phase, seg_group;
    int e_ptr0, e_ptr1;

    __device__ MlpScheduler(const MlpParams& p, const int* ends_, const int* tiles_end_, int ctas, int cluster, int num_clusters)
        : ends(ends_), tiles_end(tiles_end_), num_experts(p.num_experts), gt(p.tiles_per_group), mask(p.phase_mask),
          task(cluster), stride(num_clusters), q(-1), seg_start(0), seg_len(0), seg_phase(0), seg_group(0) {
        total_tiles = p.num_experts > 0 ? tiles_end_[p.num_experts - 1] : 0;
        num_groups = (total_tiles + gt - 1) / gt;
        nb0 = p.ph[0].n / (128 * ctas);
        nb1 = p.ph[1].n / (128 * ctas);
        num_segments = mask == 3 ? 2 * num_groups : num_groups;
        e_ptr0 = e_ptr1 = 0;
    }

    __device__ __forceinline__ void load_segment() {
        if (mask == 3) {
            if (q == 0) { seg_phase = 0; seg_group = 0; }
            else if (q == num_segments - 1) { seg_phase = 1; seg_group = num_groups - 1; }
            else if (q & 1) { seg_phase = 0; seg_group = (q + 1) >> 1; }
            else { seg_phase = 1; seg_group = (q >> 1) - 1; }
        } else {
            seg_phase = mask == 2 ? 1 : 0;
            seg_group = q;
        }
        seg_len = min(gt, total_tiles - seg_group * gt) * (seg_phase ? nb1 : nb0);
    }

    __device__ bool next(MlpTask& t) {
        while (q < 0 || task >= seg_start + seg_len) {
            seg_start += seg_len;
            if (++q >= num_segments) return false;
            load_segment();
        }
        const int local = task - seg_start;
        const int nb = seg_phase ? nb1 : nb0;
        const int tl = local / nb;
        t.phase = seg_phase;
        t.w_block = local - tl * nb;
        t.tile = seg_group * gt + tl;
        int e = seg_phase ? e_ptr1 : e_ptr0;
        while (t.tile >= tiles_end[e]) ++e;
        if (seg_phase) e_ptr1 = e; else e_ptr0 = e;
        t.expert = e;
        const int tt = t.tile - (e == 0 ? 0 : tiles_end[e - 1]);
        const int start = e == 0 ? 0 : (ends[e - 1] + 127) / 128 * 128;
        const int rows = ends[e] - start;
        t.row_start = start + tt * 128;
        t.tokens = rows <= kMlpMaxTok ? rows : min(128, rows - tt * 128);
        task += stride;
        return true;
    }
};

// One lane polls until `counter[tile]` has reached `want` (every other lane then acquires it once itself): the bounded wait
// of a down task's loaders for the gate/up tasks of its token tile. Returns false when the CTA has to unwind.
__device__ __forceinline__ bool wait_tile_done(const MlpParams& p, int tile, unsigned want, volatile uint32_t* abort_flag, uint32_t lane) {
    uint32_t done = 1;
    if (lane == 0) {
        const long long t0 = clock64();
        uint32_t spins = 0;
        while (ld_acquire_gpu(p.tile_done + tile) < want) {
            __nanosleep(40);
            if (((++spins) & 0xffu) == 0) {
                if (*abort_flag != 0) { done = 0; break; }
                if (clock64() - t0 > kWaitBudgetCycles) {
                    *abort_flag = static_cast<uint32_t>(kTimeoutGrid);
                    report_error(kTimeoutGrid, tile, static_cast<int>(ld_acquire_gpu(p.tile_done + tile)));
                    done = 0;
                    break;
                }
            }
        }
    }
    if (__shfl_sync(0xffffffffu, done, 0) == 0) return false;
    (void)ld_acquire_gpu(p.tile_done + tile);  // the lane that issues the loads acquires the counter itself ...
    fence_proxy_async_all();                   // ... and the loads go through the async proxy
    return true;
}


template <bool kPair>
__global__ void __launch_bounds__(kMlpThreads, 1)
dgb200_expert_mlp_kernel(const __grid_constant__ MlpMaps maps, const __grid_constant__ MlpParams p) {
    using L = MlpSmem<kPair>;
    constexpr int kCtas = L::kCtas;
    constexpr int kStages = L::kStages;
    constexpr uint32_t kAccCols = kMlpMaxTok;
    constexpr uint32_t kSfCol0 = 2 * kAccCols;
    constexpr uint32_t kSfColsPerKb = 12;  // weights 4, tokens 2 x 4
    constexpr uint32_t kTmemCols = 512;
    static_assert(kSfCol0 + kStages * kMlpKbPerStage * kSfColsPerKb <= kTmemCols, "TMEM budget");

    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + kStages;
    uint64_t* tmem_full_bar = bars + 2 * kStages;
    uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + L::kOffMisc);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + L::kOffMisc + 4);
    int* ends = reinterpret_cast<int*>(smem + L::kOffTables);
    int* tiles_end = ends + kMlpMaxExperts;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = kPair ? cluster_cta_rank() : 0u;
    const bool leader_cta = cta_rank == 0;
    const int cluster = static_cast<int>(blockIdx.x) / kCtas;
    const int num_clusters = static_cast<int>(gridDim.x) / kCtas;

    if (threadIdx.x == 0) {
        *abort_flag = (smem_u32(smem) & 1023u) != 0 ? static_cast<uint32_t>(kBadArgument) : 0u;  // swizzled tiles need this
        if (*abort_flag != 0) report_error(kBadArgument, 1024, static_cast<int>(smem_u32(smem) & 1023u));
        for (int i = 0; i < kStages; ++i) {
            mbar_init(full_bar + i, 3 * kCtas);  // token, weight and scale loaders of every CTA of the cluster
            mbar_init(empty_bar + i, 1);         // tcgen05.commit of the MMA issuer
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(tmem_full_bar + i, 1);
            mbar_init(tmem_empty_bar + i, 8 * kCtas);  // lane 0 of every epilogue warp of the cluster
        }
        fence_mbar_init();
#pragma unroll
        for (int ph = 0; ph < 2; ++ph) {
            prefetch_tensormap(&maps.w[ph]);
            prefetch_tensormap(&maps.sfx[ph]);
            prefetch_tensormap(&maps.sfw[ph]);
        }
    }
    // expert tables: end rows and token-tile counts, then running tile counts (host guarantees num_experts <= kMlpMaxExperts)
    for (int i = threadIdx.x; i < p.num_experts; i += kMlpThreads) {
        const int prev_end = i == 0 ? 0 : __ldg(p.expert_end + i - 1);
        const int end = __ldg(p.expert_end + i);
        ends[i] = end;
        tiles_end[i] = mlp_token_tiles(end - (prev_end + 127) / 128 * 128);
    }
    __syncthreads();
    if (warp == 0) {
        const int chunk = (p.num_experts + 31) / 32;
        const int lo = min(static_cast<int>(lane) * chunk, p.num_experts), hi = min(lo + chunk, p.num_experts);
        int sum = 0;
        for (int i = lo; i < hi; ++i) sum += tiles_end[i];
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (static_cast<int>(lane) >= off) incl += v;
        }
        int run = incl - sum;
        for (int i = lo; i < hi; ++i) {
            run += tiles_end[i];
            tiles_end[i] = run;
        }
    }
    // Tensor memory: both CTAs of a pair allocate together (the same warp in each), after a cluster barrier that makes
    // sure both are running and see each other's initialised barriers.
    if constexpr (kPair) cluster_sync_all();
    if (warp == 2) {
        if constexpr (kPair) tmem_alloc_pair(tmem_ptr_smem, kTmemCols);
        else tmem_alloc(tmem_ptr_smem, kTmemCols);
    }
    tcgen05_fence_before();
    __syncthreads();
    if constexpr (kPair) cluster_sync_all();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    const uint32_t signals_per_tile_task = 8u * kCtas;  // every epilogue warp of the cluster signals once per gate/up task

    if (warp < 4) {
        setmaxnreg_dec<kRegsControlWarps>();
        // A pipeline stage holds kMlpKbPerStage (2) K blocks of both operands. The three loader warps split its copies so
        // that no thread issues more than a few TMA instructions per stage: an instruction costs its issuing thread on the
        // order of a hundred cycles, and a K block of a pair tile is only about 256 cycles of tensor time.
        //   warp 0: token rows of the stage's first K block
        //   warp 3: the weight tiles of both K blocks (one box: consecutive tiles are contiguous) + token rows of the second
        //   warp 2: packed scale ints of both operands and both K blocks
        if (warp == 0 || warp == 2 || warp == 3) {
            MlpScheduler sched(p, ends, tiles_end, kCtas, cluster, num_clusters);
            MlpTask t;
            uint32_t stage = 0, phase = 0;
            const bool elected = elect_one();
            bool ok = *abort_flag == 0;
            while (ok && sched.next(t)) {
                const MlpPhase& ph = p.ph[t.phase];
                const int num_kb = ph.k / 128;
                const int num_ks = (num_kb + kMlpKbPerStage - 1) / kMlpKbPerStage;
                const int n_tok = (t.tokens + 15) & ~15;
                const int n_half = n_tok / kCtas;
                const int n_cover = (n_half + 15) & ~15;  // rows of the token box: one tensor map per multiple of 16
                const int x_row0 = t.row_start + static_cast<int>(cta_rank) * n_half;
                const CUtensorMap* x_map = &maps.x[t.phase][n_cover / 16 - 1];
                const int w_block = t.w_block * kCtas + static_cast<int>(cta_rank);  // this CTA's 128-row block
                const int w_row = (t.expert * (ph.n / 128) + w_block) * num_kb * 128;  // first row of the block's first tile
                const int sfw_y = t.expert * num_kb;
                const int sfx_boxes = n_tok > 128 ? 2 : 1;
                if (t.phase == 1 && p.phase_mask == 3 && true) {
                    // the activations (and their scales) of this token tile are complete once every gate/up task of the
                    // tile has signalled
                    ok = wait_tile_done(p, t.tile, static_cast<unsigned>(p.ph[0].n / (128 * kCtas)) * signals_per_tile_task, abort_flag, lane);
                    if (!ok) break;
                }
                for (int ks = 0; ks < num_ks; ++ks) {
                    ok = mbar_wait(empty_bar + stage, phase ^ 1, abort_flag, kTimeoutEmpty, ks);
                    if (!ok) break;
                    if (elected) {
                        const int kb = ks * kMlpKbPerStage;
                        const bool second = kb + 1 < num_kb;
                        uint8_t* xs = smem + L::kOffX + stage * L::kXStageBytes;
                        uint32_t tx;
                        if (warp == 0) tx = static_cast<uint32_t>(n_cover * 128);
                        else if (warp == 3) tx = 2u * ph.w_tx_bytes + (second ? static_cast<uint32_t>(n_cover * 128) : 0u);
                        else tx = static_cast<uint32_t>(1024 + sfx_boxes * 1024);
                        tx *= static_cast<uint32_t>(kCtas);
                        if constexpr (kPair) {
                            const uint32_t bar = map_to_cta(smem_u32(full_bar + stage), 0);
                            if (leader_cta) mbar_arrive_expect_tx(full_bar + stage, tx);
                            else mbar_arrive_cluster(bar);
                            if (warp == 0) {
                                tma_load_2d_pair(xs, x_map, bar, kb * 128, x_row0);
                            } else if (warp == 3) {
                                tma_load_2d_pair(smem + L::kOffW + stage * L::kWStageBytes, &maps.w[t.phase], bar, 0, w_row + kb * 128);
                                if (second) tma_load_2d_pair(xs + L::kXBytes, x_map, bar, (kb + 1) * 128, x_row0);
                            } else {
                                tma_load_2d_pair(smem + L::kOffSfw + stage * L::kSfwStageBytes, &maps.sfw[t.phase], bar, w_block * 128, sfw_y + kb);
                                for (int b = 0; b < sfx_boxes; ++b)
                                    tma_load_2d_pair(smem + L::kOffSfx + stage * L::kSfxStageBytes + b * 1024, &maps.sfx[t.phase], bar, t.row_start + b * 128, kb);
                            }
                        } else {
                            mbar_arrive_expect_tx(full_bar + stage, tx);
                            if (warp == 0) {
                                tma_load_2d(xs, x_map, full_bar + stage, kb * 128, x_row0);
                            } else if (warp == 3) {
                                tma_load_2d(smem + L::kOffW + stage * L::kWStageBytes, &maps.w[t.phase], full_bar + stage, 0, w_row + kb * 128);
                                if (second) tma_load_2d(xs + L::kXBytes, x_map, full_bar + stage, (kb + 1) * 128, x_row0);
                            } else {
                                tma_load_2d(smem + L::kOffSfw + stage * L::kSfwStageBytes, &maps.sfw[t.phase], full_bar + stage, w_block * 128, sfw_y + kb);
                                for (int b = 0; b < sfx_boxes; ++b)
                                    tma_load_2d(smem + L::kOffSfx + stage * L::kSfxStageBytes + b * 1024, &maps.sfx[t.phase], full_bar + stage, t.row_start + b * 128, kb);
                            }
                        }
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        } else if (warp == 1 && leader_cta) {
            // ---------------------------------------------------------------- MMA issuer (leader CTA only)
            MlpScheduler sched(p, ends, tiles_end, kCtas, cluster, num_clusters);
            MlpTask t;
            uint32_t stage = 0, phase = 0, iter = 0;
            const uint32_t w_base = smem_u32(smem + L::kOffW), x_base = smem_u32(smem + L::kOffX);
            const uint32_t sfw_smem = smem_u32(smem + L::kOffSfw), sfx_smem = smem_u32(smem + L::kOffSfx);
            const bool elected = elect_one();
            bool ok = *abort_flag == 0;
            while (ok && sched.next(t)) {
                const uint32_t as = iter & 1, aphase = (iter >> 1) & 1;
                ++iter;
                ok = mbar_wait(tmem_empty_bar + as, aphase ^ 1, abort_flag, kTimeoutTmemEmpty, static_cast<int>(iter));
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t n_tok = static_cast<uint32_t>((t.tokens + 15) & ~15);
                // weights are the A operand (E2M1 in byte containers, or E4M3), tokens the B operand (E4M3)
                const uint32_t idesc = make_idesc_block_scaled(p.ph[t.phase].w_fmt, kFmtE4M3, 128 * kCtas, n_tok, kScaleUE8M0);
                const uint32_t tmem_acc = tmem_base + as * kAccCols;
                const int num_kb = p.ph[t.phase].k / 128;
                const int num_ks = (num_kb + kMlpKbPerStage - 1) / kMlpKbPerStage;
                for (int ks = 0; ks < num_ks; ++ks) {
                    ok = mbar_wait(full_bar + stage, phase, abort_flag, kTimeoutFull, ks);
                    if (!ok) break;
                    if (elected) {
#pragma unroll
                        for (int kk = 0; kk < kMlpKbPerStage; ++kk) {
                            const int kb = ks * kMlpKbPerStage + kk;
                            if (kb >= num_kb) break;  // an odd K block count: the stage's second half holds nothing to multiply
                            const uint32_t sf_cols = tmem_base + kSfCol0 + (stage * kMlpKbPerStage + kk) * kSfColsPerKb;
                            const uint32_t tmem_sfw = sf_cols, tmem_sfx = sf_cols + 4;
                            const uint64_t sfw_desc = make_sf_desc(sfw_smem + stage * L::kSfwStageBytes + kk * 512);
                            const uint64_t sfx_desc = make_sf_desc(sfx_smem + stage * L::kSfxStageBytes + kk * 512);
                            const uint64_t wdesc = make_kmajor_sw128_desc(w_base + stage * L::kWStageBytes + kk * L::kWBytes);
                            const uint64_t xdesc = make_kmajor_sw128_desc(x_base + stage * L::kXStageBytes + kk * L::kXBytes);
                            if constexpr (kPair) {
                                tcgen05_cp_32x128b_warpx4_pair(tmem_sfw, sfw_desc);
                                tcgen05_cp_32x128b_warpx4_pair(tmem_sfx, sfx_desc);
                                if (n_tok > 128) tcgen05_cp_32x128b_warpx4_pair(tmem_sfx + 4, sfx_desc + (1024 >> 4));
#pragma unroll
                                for (uint32_t k4 = 0; k4 < 4; ++k4)
                                    tcgen05_mma_mxf8f6f4_pair(tmem_acc, wdesc + k4 * 2, xdesc + k4 * 2, idesc_with_sf_ids(idesc, k4, k4), tmem_sfw,
                                                              tmem_sfx, (kb | k4) != 0 ? 1u : 0u);
                            } else {
                                tcgen05_cp_32x128b_warpx4(tmem_sfw, sfw_desc);
                                tcgen05_cp_32x128b_warpx4(tmem_sfx, sfx_desc);
                                if (n_tok > 128) tcgen05_cp_32x128b_warpx4(tmem_sfx + 4, sfx_desc + (1024 >> 4));
#pragma unroll
                                for (uint32_t k4 = 0; k4 < 4; ++k4)
                                    tcgen05_mma_mxf8f6f4(tmem_acc, wdesc + k4 * 2, xdesc + k4 * 2, idesc_with_sf_ids(idesc, k4, k4), tmem_sfw,
                                                         tmem_sfx, (kb | k4) != 0 ? 1u : 0u);
                            }
                        }
                        if constexpr (kPair) {
                            tcgen05_commit_pair(empty_bar + stage, 3);
                            if (ks == num_ks - 1) tcgen05_commit_pair(tmem_full_bar + as, 3);
                        } else {
                            tcgen05_commit(empty_bar + stage);
                            if (ks == num_ks - 1) tcgen05_commit(tmem_full_bar + as);
                        }
                    }
                    __syncwarp();
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else {
        setmaxnreg_inc<kRegsEpilogueWarps>();
        // ---------------------------------------------------------------- epilogue (8 warps = 2 warpgroups)
        // Warp w reads TMEM lanes [32 (w % 4), +32): 32 weight rows of this CTA's 128. The two warpgroups split the tile's
        // 16-column chunks. A lane owns one weight row (down) or, after the gate/up exchange, one output channel and 8
        // tokens; for a fixed token the lanes of a warp hold consecutive channels, so every store instruction writes one
        // contiguous segment of the token's output row (64 bytes of BF16, or 2 x 16 bytes of E4M3) straight from
        // registers: no staging, no TMA store to queue behind the operand loads. The load of the next chunk is in flight
        // while the current one is processed.
        MlpScheduler sched(p, ends, tiles_end, kCtas, cluster, num_clusters);
        MlpTask t;
        const uint32_t q = warp & 3, wg = (warp - 4) >> 2;
        const uint32_t pair_barrier = 1 + wg * 2 + (q >> 1);  // the two warps that share a 32-channel scale group (64 threads)
        const uint32_t tmem_empty_leader = kPair ? map_to_cta(smem_u32(tmem_empty_bar), 0) : 0u;
        uint32_t iter = 0, xch_parity = 0;
        const bool hi = lane >= 16;
        const uint32_t j = lane & 15;
        bool ok = *abort_flag == 0;
        while (ok && sched.next(t)) {
            const uint32_t as = iter & 1, aphase = (iter >> 1) & 1;
            ++iter;
            ok = mbar_wait<32>(tmem_full_bar + as, aphase, abort_flag, kTimeoutTmemFull, static_cast<int>(iter));
            if (!ok) break;
            tcgen05_fence_after();
            const int chunks = (t.tokens + 15) >> 4;
            const int c_begin = wg == 0 ? 0 : (chunks + 1) / 2, c_end = wg == 0 ? (chunks + 1) / 2 : chunks;
            const int w_block = t.w_block * kCtas + static_cast<int>(cta_rank);  // this CTA's 128 weight rows
            const uint32_t tmem_row = tmem_base + ((q * 32u) << 16) + as * kAccCols;
            auto release_accumulator = [&]() {
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (kPair) mbar_arrive_cluster(tmem_empty_leader + as * 8);
                    else mbar_arrive(tmem_empty_bar + as);
                }
            };
            // routing weights of this warpgroup's tokens (at most kMlpMaxTok / 2 + 8): token c_begin * 16 + 32 k + lane in wv[k]
            float wv[4] = {1.0f, 1.0f, 1.0f, 1.0f};
            if (t.phase == 0 && p.row_weight != nullptr) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int idx = c_begin * 16 + k * 32 + static_cast<int>(lane);
                    if (idx < c_end * 16) wv[k] = __ldg(p.row_weight + t.row_start + idx);
                }
            }
            uint32_t v[16], vn[16];
            if (c_begin >= c_end) release_accumulator();
            else tmem_ld_32x32b_x16(tmem_row + c_begin * 16, vn);
            for (int c = c_begin; c < c_end; ++c) {
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = vn[i];
                if (c + 1 < c_end) tmem_ld_32x32b_x16(tmem_row + (c + 1) * 16, vn);
                else release_accumulator();
                const long long row0 = static_cast<long long>(t.row_start) + c * 16;
                if (t.phase == 0) {
                    // ---- gate/up: this warp's lanes 0-15 hold gate rows, lanes 16-31 the up rows of the same 16 channels
                    const int ch0 = w_block * 64 + static_cast<int>(q) * 16;  // first output channel of this warp
                    const int cc = c - c_begin;
                    const float wsel = (cc >> 1) == 0 ? wv[0] : ((cc >> 1) == 1 ? wv[1] : ((cc >> 1) == 2 ? wv[2] : wv[3]));
                    float o[8];
                    uint32_t amax_bits[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t send = hi ? v[i] : v[8 + i];
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 16);
                        float gv = bf16_round(__uint_as_float(hi ? recv : v[i]));
                        float uv = bf16_round(__uint_as_float(hi ? v[8 + i] : recv));
                        const float w = __shfl_sync(0xffffffffu, wsel, (cc & 1) * 16 + (hi ? 8 : 0) + i);
                        if (p.clamp > 0.0f) {
                            gv = fminf(gv, p.clamp);
                            uv = fminf(fmaxf(uv, -p.clamp), p.clamp);
                        }
                        const float silu = p.fast_math ? gv * rcp_approx(1.0f + __expf(-gv)) : gv / (1.0f + expf(-gv));
                        o[i] = silu * uv * w;
                        // maximum over this half-warp's 16 channels: non-negative floats order like their bit patterns
                        uint32_t m = __float_as_uint(fabsf(o[i]));
                        m = max(m, __shfl_xor_sync(0xffffffffu, m, 1));
                        m = max(m, __shfl_xor_sync(0xffffffffu, m, 2));
                        m = max(m, __shfl_xor_sync(0xffffffffu, m, 4));
                        m = max(m, __shfl_xor_sync(0xffffffffu, m, 8));
                        amax_bits[i] = m;
                    }
                    // the other 16 channels of the scale group belong to the neighbouring warp: exchange through shared memory
                    uint32_t* xch = reinterpret_cast<uint32_t*>(smem + L::kOffXch) + ((wg * 2 + xch_parity) * 2 + (q >> 1)) * 32;  // [2 warps][16 tokens]
                    xch_parity ^= 1;
                    if (j == 0) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) xch[(q & 1) * 16 + (hi ? 8 : 0) + i] = amax_bits[i];
                    }
                    named_barrier_sync(pair_barrier, 64);
                    unsigned char* out = p.act_q + (row0 + (hi ? 8 : 0)) * p.act_q_row_stride + ch0 + j;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t other = xch[((q & 1) ^ 1) * 16 + (hi ? 8 : 0) + i];
                        const float amax = __uint_as_float(max(amax_bits[i], other));
                        float sf_inv;
                        uint32_t sf_byte;
                        ue8m0_scale_for_amax(amax, sf_inv, sf_byte);
                        out[i * p.act_q_row_stride] = static_cast<unsigned char>(__nv_cvt_float_to_fp8(o[i] * sf_inv, __NV_SATFINITE, __NV_E4M3));
                        if ((q & 1) == 0 && j == 0)
                            p.act_sf[(static_cast<long long>(ch0 >> 7) * p.act_sf_k_stride + sf_row_in_cp_order(row0 + (hi ? 8 : 0) + i)) * 4 + ((ch0 >> 5) & 3)] =
                                static_cast<unsigned char>(sf_byte);
                    }
                } else {
                    // ---- down: one weight row (output channel) per lane, 16 tokens; a store instruction = 64 contiguous bytes
                    __nv_bfloat16* out = p.out + row0 * p.out_row_stride + w_block * 128 + q * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 16; ++i) out[i * p.out_row_stride] = __float2bfloat16_rn(__uint_as_float(v[i]));
                }
            }
            if (t.phase == 0 && p.phase_mask == 3) {
                // this warp's part of the tile's activations and scales is written: tell the down tasks
                __syncwarp();
                if (lane == 0) {
                    __threadfence();
                    red_release_gpu_add(p.tile_done + t.tile, 1u);
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
    if constexpr (kPair) cluster_sync_all();  // the peer may still signal barriers of this CTA or read its shared memory
    if (warp == 2) {
        tcgen05_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols);
        else tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace dgb
