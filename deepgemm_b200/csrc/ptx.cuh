// Hand-written PTX wrappers for sm_100a: mbarrier, TMA (tiled and 1-D bulk), tcgen05
// (TMEM alloc, block-scaled MMA, smem->TMEM copy, TMEM load, commit) and the shared-memory /
// instruction descriptors they consume.
//
// Behavioural counterparts in the reference: deep_gemm/include/deep_gemm/ptx/{tcgen05,tma,ld_st,utils}.cuh
// and deep_gemm/include/deep_gemm/mma/sm100.cuh:14-165 (descriptor builders). The reference obtains
// its descriptor bitfields from CuTe; here they are built with plain shifts from the PTX ISA tables.
//
// Every wait in this file is bounded: a wait that runs out records a code in the device status
// block and returns false, so a kernel can unwind (free TMEM, return) instead of hanging the GPU.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

namespace dgb {

// ----------------------------------------------------------------------------------------------
// Device status block: one per device that loads the library (the library is a single translation
// unit, so the definition lives here).
// word 0: first error code (0 = OK), word 1: block index, word 2: detail a, word 3: detail b.
// ----------------------------------------------------------------------------------------------
__device__ int g_status[8];

enum StatusCode : int {
    kOk = 0,
    kTimeoutFull = 1,       // consumer waited for TMA data
    kTimeoutEmpty = 2,      // producer waited for a free stage
    kTimeoutSfReady = 3,    // MMA warp waited for the scale-factor transposer
    kTimeoutTmemFull = 4,   // epilogue waited for the accumulator
    kTimeoutTmemEmpty = 5,  // MMA warp waited for the epilogue to drain the accumulator
    kBadArgument = 6,
    kTimeoutPeer = 7,       // waited for a flag another rank writes
    kTimeoutGrid = 8,       // waited for a flag another CTA of this grid writes
    kTimeoutRowMover = 9,   // a row-moving warp waited for its bulk load
};

__device__ __forceinline__ void report_error(int code, int a, int b) {
    if (atomicCAS(&g_status[0], 0, code) == 0) {
        g_status[1] = static_cast<int>(blockIdx.x);
        g_status[2] = a;
        g_status[3] = b;
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
    return l;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n" : "=r"(pred));
    return pred != 0;
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                 :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
#ifdef DGB200_TEST_WAIT
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// Budget of one wait in SM clock cycles: about two seconds at 2 GHz, several orders of magnitude above any
// legitimate stage wait. The SM-local clock is used because reading %globaltimer costs hundreds of cycles.
constexpr long long kWaitBudgetCycles = 4000000000ll;

// Bounded wait. `abort_flag` is a CTA-shared word: once any role of the CTA gives up, the others
// stop at their next poll instead of each burning their own budget.
// kBackoffNs > 0 makes the caller sleep between polls: for waits that last a whole tile, so that the polling does
// not compete with the issue threads for the shared-memory pipeline.
template <int kBackoffNs = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          int code, int detail) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (kBackoffNs > 0) __nanosleep(kBackoffNs);
        if (mbar_try_wait(bar, parity)) return true;
        if (((++spins) & 0x3ffu) == 0) {
            if (*abort_flag != 0) return false;
            const long long now = clock64();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > kWaitBudgetCycles) {
                *abort_flag = static_cast<uint32_t>(code);
                report_error(code, detail, static_cast<int>(parity));
                return false;
            }
        }
    }
}

// One lane polls for the whole warp; every lane gets the outcome.
template <int kBackoffNs = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                               int code, int detail) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait<kBackoffNs>(bar, parity, abort_flag, code, detail) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ----------------------------------------------------------------------------------------------
// TMA: tiled 2-D load (CTA-local destination, completion on a CTA-local mbarrier) and 1-D bulk load
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Tiled store shared -> global (bulk async group completion). x * element size must be a multiple of 16 bytes and
// no coordinate may be negative; rows and columns beyond the tensor's extent are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
// Tiled reduction shared -> global: every element of the box is added to the tensor's element (the tensor map's data
// type, FP32 here) by the memory system; same coordinate rules and completion mechanism as the store above.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int32_t x, int32_t y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once the bulk stores of this thread's committed groups have finished reading shared memory.
__device__ __forceinline__ void bulk_wait_group_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Returns once those stores are complete (their writes performed).
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Untiled bulk copies (both addresses 16-byte aligned, size a multiple of 16 bytes): global -> shared completing on an
// mbarrier of this CTA, and shared -> global as part of the thread's bulk async-group.
__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* gmem_dst, uint32_t smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(gmem_dst), "r"(smem_src), "r"(bytes) : "memory");
}

// L2 prefetch of one contiguous span (16-byte aligned address, size a multiple of 16 bytes): starts the HBM read
// early without occupying shared memory; handled by the bulk-copy unit, no completion to wait for.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gmem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(gmem_src), "r"(bytes) : "memory");
}

// L2 prefetch of one box of a tiled tensor map (same coordinate rules as the load).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" :: "l"(map), "r"(x), "r"(y) : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: tensor memory management
// ----------------------------------------------------------------------------------------------
// Warp-collective. `num_cols` is a power of two in [32, 512]. The base address lands in `*smem_dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t num_cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(smem_dst)), "r"(num_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_addr, uint32_t num_cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_addr), "r"(num_cols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// All previously issued tcgen05.mma / tcgen05.cp of this thread arrive on `bar` when they retire.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
}

// ----------------------------------------------------------------------------------------------
// Descriptors
// ----------------------------------------------------------------------------------------------
// 64-bit shared-memory matrix descriptor (PTX ISA, tcgen05 "shared memory descriptor"):
//   [0,14)  start address >> 4          [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4   [46,48) descriptor version (1 on sm_100)
//   [49,52) base offset                 [52]    LBO mode          [61,64) swizzle mode
// Swizzle codes: 0 none, 1 128B with 32B atoms, 2 128B, 4 64B, 6 32B.
constexpr uint64_t kSwizzleNone = 0, kSwizzle128B = 2;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes, uint64_t swizzle) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
    d |= 1ull << 46;
    d |= swizzle << 61;
    return d;
}

// K-major operand tile whose rows are exactly one 128-byte swizzle span: 8-row groups are 1024 B apart.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    return make_smem_desc(smem_addr, 1024, kSwizzle128B);
}

// MN-major operand tile (rows = K, each row 128 contiguous bytes of M or N, 128-byte swizzle, as a TMA box of a
// [K, MN] tensor lands): 8-row K groups are 1024 B apart (stride offset); the leading offset is the distance between
// 128-byte chunks along MN, which a 128-wide 8-bit tile has only one of.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
    return make_smem_desc(smem_addr, 1024, kSwizzle128B) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16);
}

// Scale-factor block for tcgen05.cp 32x128b: 32 rows of 16 bytes, contiguous; 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
    return make_smem_desc(smem_addr, 128, kSwizzleNone);
}

// 32-bit instruction descriptor of the block-scaled kinds (PTX ISA, tcgen05 "instruction descriptor"):
//   [4,6) B scale-factor id   [7,10) A format   [10,13) B format   [13] negate A  [14] negate B
//   [15] A MN-major  [16] B MN-major  [17,23) N >> 3   [23] scale type (0 UE4M3, 1 UE8M0)
//   [24,29) M >> 4   [29,31) A scale-factor id
// Element format codes: kind::mxf8f6f4 -> E4M3 0, E5M2 1, E2M3 3, E3M2 4, E2M1 5; kind::mxf4* -> E2M1 1.
constexpr uint32_t kFmtE4M3 = 0, kFmtE2M1_F8F6F4 = 5, kFmtE2M1_MXF4 = 1;
constexpr uint32_t kScaleUE4M3 = 0, kScaleUE8M0 = 1;

__host__ __device__ constexpr uint32_t make_idesc_block_scaled(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                               uint32_t scale_type) {
    return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (scale_type << 23) | ((m >> 4) << 24);
}

// kind::f16 descriptor: BF16 operands (format 1), both K-major, FP32 accumulator (format 1 at bits [4,6)).
__host__ __device__ constexpr uint32_t make_idesc_bf16_f32(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_sf_id, uint32_t b_sf_id) {
    return idesc | (a_sf_id << 29) | (b_sf_id << 4);
}

// ----------------------------------------------------------------------------------------------
// tcgen05: data movement and MMA
// ----------------------------------------------------------------------------------------------
// Copies 32 rows x 16 B from shared memory into 4 TMEM columns, replicated to all four 32-lane quarters.
__device__ __forceinline__ void tcgen05_cp_32x128b_warpx4(uint32_t tmem_addr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(tmem_addr), "l"(sdesc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T with per-block scales; FP8/FP6/FP4 operands, one UE8M0 scale per 32 K.
__device__ __forceinline__ void tcgen05_mma_mxf8f6f4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                     uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, BF16 / FP16 operands, K = 16 per instruction, no scales.
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Packed E2M1 x E2M1, K = 64 per instruction, one UE4M3 scale per 16 K (NVFP4).
__device__ __forceinline__ void tcgen05_mma_mxf4nvf4_4x(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                        uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

// ----------------------------------------------------------------------------------------------
// CTA pairs (thread-block cluster of two, tcgen05 cta_group::2). One thread of the even CTA (the leader) issues copies,
// MMAs and commits for both; every address below is CTA-relative and applies to both CTAs of the pair alike.
// Reference counterparts: deep_gemm/include/deep_gemm/ptx/tcgen05.cuh:61-98, deep_gemm/include/deep_gemm/common/tma_copy.cuh:37-45
// (per-CTA loads that complete on the leader's barrier; no cluster multicast of loaded data anywhere).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}

// Shared-memory address of `local` (an address of this CTA) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}

// Arrives (count 1, no transaction bytes) on an mbarrier given by its cluster-wide shared address.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}

// Tiled load into THIS CTA's shared memory whose completion bytes are credited to an mbarrier of either CTA of the pair
// (`bar_cluster_addr` from map_to_cta). Plain per-CTA load: the data is not multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t x,
                                                 int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}

// Warp-collective, executed by the same warp of BOTH CTAs of the pair.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t num_cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(smem_dst)), "r"(num_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t tmem_addr, uint32_t num_cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_addr), "r"(num_cols) : "memory");
}

// All previously issued tcgen05 operations of this thread arrive, when they retire, on the mbarrier at this shared
// offset in every CTA named by `cta_mask` (bit r = CTA r of the cluster).
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"(cta_mask) : "memory");
}

__device__ __forceinline__ void tcgen05_cp_32x128b_warpx4_pair(uint32_t tmem_addr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" :: "r"(tmem_addr), "l"(sdesc) : "memory");
}

// D[tmem, 128 lanes per CTA] (+)= A[256 rows: 128 from each CTA's shared memory] * B[N rows: N / 2 from each CTA]^T.
__device__ __forceinline__ void tcgen05_mma_mxf8f6f4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}\n"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t tmem_addr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(tmem_addr) : "memory");
}

// Named barrier among `count` threads (a multiple of 32) of this CTA; id 0 is __syncthreads.
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t count) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(count) : "memory");
}

// Generic-proxy accesses before, async-proxy (TMA) accesses after: every state space.
__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits until at most `kPending` of this thread's committed bulk stores have not finished READING shared memory.
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(kPending) : "memory");
}

// Each lane reads 32 consecutive 32-bit columns of its own TMEM lane (lane quarter = warp index % 4).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t tmem_addr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(tmem_addr) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// Global-memory helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" :: "l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ uint4 ld_global_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

// Register re-balancing between warpgroups (all warps of a warpgroup execute the same instruction).
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" :: "n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kRegs));
}

__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ uint32_t e2m1_code(float v) {
    // thresholds between {0, .5, 1, 1.5, 2, 3, 4, 6}; a value on a threshold rounds down; -0 encodes as +0
    const float a = fabsf(v);
    uint32_t code = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    if (v < 0.0f && code != 0) code |= 8u;
    return code;
}

// Eight floats -> eight packed E2M1 codes (element i in nibble i) with the hardware conversion: round to nearest,
// ties to even, saturating at 6. Differs from e2m1_code only for values exactly on the thresholds .75, 1.75 and 3.5
// (which go up here, down there) and in the sign of zero.
__device__ __forceinline__ uint32_t pack_e2m1x8_rn(const float* v) {
    uint32_t out;
    asm volatile(
        "{\n\t"
        ".reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t"
        "}\n"
        : "=r"(out)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return out;
}

// E4M3 round-to-nearest-even with saturation at 448, as a byte and back (UE4M3 block scales are non-negative E4M3).
__device__ __forceinline__ uint32_t e4m3_byte(float x) {
    return static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
    return __half2float(__half(h));
}

// Programmatic dependent launch: wait for the preceding kernel's memory to be visible / let the next one start.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// First statement of every kernel that may be launched with programmatic stream serialization: nothing the preceding
// kernel of the stream wrote is read, and nothing it may still read is written, before the wait returns (it returns
// at once when the launch carries no such dependency); the next kernel of the stream may then be launched early and
// parks in its own wait.
__device__ __forceinline__ void pdl_prologue() {
    grid_dependency_wait();
    grid_dependency_launch_dependents();
}

// tcgen05.cp.32x128b.warpx4 reads, per 128 rows of one packed scale int, 32 rows x 4 words where word j of row r
// is the scale int of source row r + 32 j. A tensor stored with every aligned group of 128 rows in that order (row
// r of the group at position 4 (r % 32) + r / 32) can be copied by TMA and handed to tcgen05.cp as it lands.
__host__ __device__ inline long long sf_row_in_cp_order(long long row) {
    return (row & ~127ll) + ((row & 31) << 2) + ((row & 127) >> 5);
}

}  // namespace dgb
