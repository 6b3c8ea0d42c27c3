// libdgb200.so: C-ABI entry points (declared in include/dgb200.h) and the single translation unit that holds
// every sm_100a kernel of the Mega-MoE hot path. Host logic here plays the role of the reference's
// csrc/apis/{gemm,mega,layout,runtime}.hpp argument checking and csrc/jit_kernels/impls/*.hpp launch glue;
// there is no JIT: every kernel is compiled ahead of time for sm_100a.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "host_common.cuh"
#include "gemm_kernel.cuh"
#include "gemm_swap_kernel.cuh"
#include "expert_mlp_kernel.cuh"
#include "quant_kernels.cuh"
#include "moe_kernels.cuh"

namespace dgb {

namespace {

constexpr int kVersion = 100;

bool use_pdl();  // the "pdl" tuning knob (set_pdl)

// Kernel launch with, when `pdl` is set, the programmatic-stream-serialization attribute: the kernel may be launched
// while the preceding kernel of the stream still runs and parks in its pdl_prologue() until that one has completed
// (reference: the launch attribute in csrc/jit/handle.hpp:77, switched by set_pdl, csrc/apis/runtime.hpp:24-28). Only
// kernels whose first statement is pdl_prologue() may be launched this way.
template <typename... Params, typename... Args>
cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream, bool pdl,
                          Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <int BLOCK_N, int kStages, int EPI, int kKind = kKindFp8Fp4>
int launch_gemm(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_sfa, const CUtensorMap& tm_sfb,
                const CUtensorMap& tm_out, const GemmParams& p, int grid, cudaStream_t stream) {
    using L = GemmSmem<BLOCK_N, kStages, kKind, EPI == kEpiF32Acc>;
    auto kernel = dgb200_grouped_gemm_kernel<BLOCK_N, kStages, EPI, kKind>;
    static bool configured = false;  // per instantiation; the attribute is per device function, set on every device once
    static int configured_device = -1;
    int dev = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    if (!configured || configured_device != dev) {
        DGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
        configured = true;
        configured_device = dev;
    }
    DGB_CUDA(launch_kernel(kernel, dim3(grid), dim3(kGemmThreads), L::kDynamicBytes, stream, use_pdl(), tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p));
    return 0;
}

struct GemmCall {
    const void* a;
    const void* b;
    const void* sfa;  // packed UE8M0 int32: int (group, kp, row) at sfa[group * sfa_group_stride + kp * sfa_k_stride + row]
    const void* sfb;
    long long sfa_k_stride, sfa_group_stride, sfb_k_stride, sfb_group_stride;
    int num_groups_a;  // groups of A's scale factors: 1 for the contiguous layouts, num_groups for the masked one
    int kind;          // kKindFp8Fp4 (default) or kKindNvfp4
    int whole_tile_stores;  // the rows between a group's end and its 128-row tile end are private padding: the
                            // epilogue may write all 128 rows of every tile
    long long a_rows_total;  // rows of the flattened A
    long long a_row_stride_bytes, b_row_stride_bytes;  // BF16 kind only: row pitches of A and B
    int b_mn_major;  // BF16 kind: B is [groups * k, n] with n contiguous (b_row_stride_bytes = pitch of a K row); FP8 x FP4
                     // kind: likewise, dense rows of n bytes (E4M3) or n / 2 bytes (packed E2M1, two N elements per byte)
    int a_mn_major;  // BF16 kind, dense mode only: A is [k, m] with m contiguous (a_row_stride_bytes = pitch of a K row)
    GemmParams p;
    int b_is_fp4;
    int epilogue;
    int max_tiles;  // upper bound on tiles, <= 0 if unknown
};

// Process-wide tuning knobs (defaults are the measured best on B200).
struct Tuning {
    int swap_ab = -1;  // layer GEMMs: tokens on the UMMA N side (-1 = by expected rows per expert, 0 = never, 1 = always)
    int block_n = 0;  // 0 = automatic
    int mlp_kernel = -1;  // FP8 x FP4 layer GEMMs: 0 = separate gate/up and down kernels (tokens-on-M / swapped split),
                          // 1 = the fused expert-MLP kernel on single CTAs, 2 = on CTA pairs; -1 = not yet read from
                          // the environment (DGB200_MLP_KERNEL, default below)
    int fused_return = 1;  // expert-parallel layer with guest experts: the down GEMM's epilogue sends the output rows back
    int fused_dispatch = 0;  // ... and the gate/up GEMM of expert phase q pushes the dispatch rows of phase q + 1
    int pdl = 1;  // programmatic dependent launch between the kernels of the single-rank layer (set_pdl)
    int ep_comm_sms = 0;  // expert-parallel layer: SMs kept free of GEMM CTAs for kernels that move rows over NVLink on a
                          // second stream while the GEMMs run (0 = one stream: every kernel on all SMs)
    long long peer_wait_cycles = 20000000000ll;  // budget of a wait for another rank, SM clock cycles (about 10 s: ranks
                                                 // may reach their first call seconds apart)
};

Tuning& tuning() {
    static Tuning t;
    return t;
}

bool use_pdl() { return tuning().pdl != 0; }

constexpr int kDefaultMlpKernel = 0;

// Which kernels run the FP8 x FP4 layer's GEMMs. Fixed at first use for the life of the process, because the weights'
// gate/up interleave (transform_weights_for_mega_moe) depends on it: 16 rows for the fused kernel, 128 otherwise.
int mlp_kernel_choice() {
    Tuning& t = tuning();
    if (t.mlp_kernel < 0) {
        const char* env = std::getenv("DGB200_MLP_KERNEL");
        t.mlp_kernel = env != nullptr ? std::atoi(env) : kDefaultMlpKernel;
        if (t.mlp_kernel < 0 || t.mlp_kernel > 2) t.mlp_kernel = kDefaultMlpKernel;
    }
    return t.mlp_kernel;
}

int run_gemm(GemmCall& c, cudaStream_t stream) {
    GemmParams& p = c.p;
    const bool nvfp4 = c.kind == kKindNvfp4;
    const bool bf16 = c.kind == kKindBf16;
    const int k_block = nvfp4 ? 256 : (bf16 ? 64 : 128);
    DGB_REQUIRE(p.k > 0 && p.k % k_block == 0, "k (%d) must be a positive multiple of %d", p.k, k_block);
    if (nvfp4 || bf16) p.gran_a = p.gran_b = 32;  // unused by these kinds; keeps the checks below uniform
    if (bf16) {
        // no scale factors: the kernel never loads them; the fields below only have to pass the shared checks
        c.sfa = c.a;
        c.sfb = c.b;
        c.sfa_k_stride = (std::max<long long>(c.a_rows_total, 1) + 3) / 4 * 4;
        c.sfb_k_stride = p.n;
        c.sfa_group_stride = static_cast<long long>((p.k / 32 + 3) / 4) * c.sfa_k_stride;
        c.sfb_group_stride = static_cast<long long>((p.k / 32 + 3) / 4) * c.sfb_k_stride;
        p.sf_transposed = 1;
        DGB_REQUIRE(c.epilogue == kEpiBF16 || c.epilogue == kEpiF32 || c.epilogue == kEpiSwiGLUBf16,
                    "unknown epilogue %d for the BF16 kind", c.epilogue);
    }
    DGB_REQUIRE(p.n > 0 && p.n % 128 == 0, "n (%d) must be a positive multiple of 128", p.n);
    DGB_REQUIRE(p.gran_a == 32 || p.gran_a == 128, "gran_k_a must be 32 or 128, got %d", p.gran_a);
    DGB_REQUIRE(p.gran_b == 32 || p.gran_b == 128, "gran_k_b must be 32 or 128, got %d", p.gran_b);
    DGB_REQUIRE(p.num_groups > 0, "num_groups must be positive");
    DGB_REQUIRE(c.a != nullptr && c.b != nullptr && c.sfa != nullptr && c.sfb != nullptr &&
                    (p.layout != nullptr || p.mode == kModeDense),
                "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(c.a) % 16 == 0, "a must be 16-byte aligned");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(c.b) % 32 == 0, "b must be 32-byte aligned");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(c.sfa) % 16 == 0 && reinterpret_cast<uintptr_t>(c.sfb) % 16 == 0,
                "scale-factor tensors must be 16-byte aligned");
    DGB_REQUIRE(c.sfa_k_stride % 4 == 0 && c.sfb_k_stride % 4 == 0 && c.sfa_k_stride > 0 && c.sfb_k_stride >= p.n,
                "packed scale-factor MN strides must be positive multiples of 4 ints (TMA-aligned) that cover MN");
    const int packed_k_a = nvfp4 ? p.k / 64 : (p.k / p.gran_a + 3) / 4;
    const int packed_k_b = nvfp4 ? p.k / 64 : (p.k / p.gran_b + 3) / 4;
    const uint32_t sf_box_rows = nvfp4 ? 4 : 1;  // packed scale ints per row per K block
    DGB_REQUIRE(c.num_groups_a == 1 || c.sfa_group_stride == packed_k_a * c.sfa_k_stride,
                "scale factors of A: group stride must equal packed K x MN stride");
    DGB_REQUIRE(p.num_groups == 1 || c.sfb_group_stride == packed_k_b * c.sfb_k_stride,
                "scale factors of B: group stride must equal packed K x MN stride");
    p.sfa_group_rows = c.num_groups_a > 1 ? packed_k_a : 0;
    p.sfb_packed_k = packed_k_b;
    if (c.a_rows_total == 0) return 0;

    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
    int rc = 0;
    if (!bf16) {
        rc = make_tensor_map_2d(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_INT32, c.sfa, static_cast<uint64_t>(c.sfa_k_stride),
                                static_cast<uint64_t>(packed_k_a) * c.num_groups_a,
                                static_cast<uint64_t>(c.sfa_k_stride) * 4, 128, sf_box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
    }
    // Wide N tiles give each tcgen05.mma enough work (128 x 256 x 32) to cover the per-K-block issue chain.
    const bool swiglu = c.epilogue == kEpiSwiGLU || c.epilogue == kEpiSwiGLUNvfp4 || c.epilogue == kEpiSwiGLUBf16;
    // the SwiGLU epilogues pair the two 128-channel halves of a 256-wide tile (gate | up)
    DGB_REQUIRE(!swiglu || p.n % 256 == 0, "the gate/up GEMM needs n (%d) to be a multiple of 256", p.n);
    const int block_n = swiglu ? 256 : (tuning().block_n != 0 ? tuning().block_n : (p.n % 256 == 0 ? 256 : 128));
    DGB_REQUIRE((block_n == 128 || block_n == 256) && p.n % block_n == 0, "block_n %d does not divide n %d", block_n, p.n);
    if (!bf16) {
        rc = make_tensor_map_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_INT32, c.sfb, static_cast<uint64_t>(c.sfb_k_stride),
                                static_cast<uint64_t>(packed_k_b) * p.num_groups, static_cast<uint64_t>(c.sfb_k_stride) * 4,
                                static_cast<uint32_t>(block_n), sf_box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
    }
    const uint64_t a_row_bytes = nvfp4 ? p.k / 2 : p.k;  // packed E2M1 or E4M3
    if (bf16 && c.a_mn_major) {
        DGB_REQUIRE(p.mode == kModeDense, "an MN-major A is built for the dense GEMM only");
        rc = make_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c.a, static_cast<uint64_t>(c.a_rows_total),
                                static_cast<uint64_t>(p.k), static_cast<uint64_t>(c.a_row_stride_bytes), 64, 64,
                                CU_TENSOR_MAP_SWIZZLE_128B);
        p.a_mn_major = 1;
    } else if (bf16)
        rc = make_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c.a, static_cast<uint64_t>(p.k),
                                static_cast<uint64_t>(c.a_rows_total), static_cast<uint64_t>(c.a_row_stride_bytes), 64, 128,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    else
        rc = make_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.a, a_row_bytes,
                                static_cast<uint64_t>(c.a_rows_total), a_row_bytes, 128, 128,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (bf16) tm_sfa = tm_sfb = tm_a;  // valid maps for the kernel's descriptor prefetch; never used for a copy
    const uint64_t b_rows = static_cast<uint64_t>(p.num_groups) * p.n;
    const uint32_t BLOCK_N = static_cast<uint32_t>(block_n);
    if (bf16) {
        if (c.b_mn_major)
            rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c.b, static_cast<uint64_t>(p.n),
                                    static_cast<uint64_t>(p.num_groups) * p.k, static_cast<uint64_t>(c.b_row_stride_bytes), 64, 64,
                                    CU_TENSOR_MAP_SWIZZLE_128B);
        else
            rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, c.b, static_cast<uint64_t>(p.k), b_rows,
                                    static_cast<uint64_t>(c.b_row_stride_bytes), 64, BLOCK_N, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = 0;
        p.b_mn_major = c.b_mn_major ? 1 : 0;
        p.b_tx_bytes = BLOCK_N * 128;
    } else if (nvfp4) {
        // both operands stay packed in shared memory (two E2M1 per byte): plain byte tensors
        rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.b, static_cast<uint64_t>(p.k / 2), b_rows,
                                static_cast<uint64_t>(p.k / 2), 128, BLOCK_N, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = kFmtE2M1_MXF4;
        p.b_tx_bytes = BLOCK_N * 128;
    } else if (c.b_mn_major) {
        // [groups * k, n] with n contiguous: boxes of 128 channels x 128 K rows, read through MN-major descriptors
        const uint64_t k_rows = static_cast<uint64_t>(p.num_groups) * p.k;
        if (c.b_is_fp4)
            rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, c.b, static_cast<uint64_t>(p.n), k_rows,
                                    static_cast<uint64_t>(p.n / 2), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        else
            rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.b, static_cast<uint64_t>(p.n), k_rows,
                                    static_cast<uint64_t>(p.n), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = c.b_is_fp4 ? kFmtE2M1_F8F6F4 : kFmtE4M3;
        p.b_tx_bytes = BLOCK_N * (c.b_is_fp4 ? 64 : 128);
        p.b_mn_major = 1;
    } else if (c.b_is_fp4) {
        rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, c.b, static_cast<uint64_t>(p.k), b_rows,
                                static_cast<uint64_t>(p.k / 2), 128, BLOCK_N, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = kFmtE2M1_F8F6F4;
        // Packed FP4 expands to one byte per element in shared memory; the mbarrier is credited with the
        // bytes read from global memory (half the tile).
        p.b_tx_bytes = BLOCK_N * 64;
    } else {
        rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.b, static_cast<uint64_t>(p.k), b_rows,
                                static_cast<uint64_t>(p.k), 128, BLOCK_N, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = kFmtE4M3;
        p.b_tx_bytes = BLOCK_N * 128;
    }
    if (rc) return rc;

    // Output tensor map for the staged (shared memory + TMA) epilogue stores of the 256-wide FP8 x FP4 kernels.
    CUtensorMap tm_out = tm_a;
    p.tma_store = 0;
    // NVFP4: only the BF16 epilogue (the down GEMM: few K blocks per tile, so its store burst weighs most) trades a
    // pipeline stage for the staging buffers.
    const bool nvfp4_staged = nvfp4 && block_n == 256 && c.epilogue == kEpiBF16;
    if (block_n == 256 && c.epilogue == kEpiSwiGLUBf16) {
        rc = make_tensor_map_2d(&tm_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, p.act_q, static_cast<uint64_t>(p.n / 2),
                                static_cast<uint64_t>(c.a_rows_total), static_cast<uint64_t>(p.act_q_row_stride), 32, 32,
                                CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc) return rc;
        p.tma_store = c.whole_tile_stores ? 2 : 1;
    } else if (block_n == 256 && ((!nvfp4 && (c.epilogue == kEpiBF16 || c.epilogue == kEpiSwiGLU)) || nvfp4_staged) &&
        (static_cast<long long>(p.d_row_stride) * 2) % 16 == 0) {
        if (c.epilogue == kEpiBF16)
            rc = make_tensor_map_2d(&tm_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, p.d, static_cast<uint64_t>(p.n),
                                    static_cast<uint64_t>(c.a_rows_total), static_cast<uint64_t>(p.d_row_stride) * 2, 32, 32,
                                    CU_TENSOR_MAP_SWIZZLE_64B);
        else
            rc = make_tensor_map_2d(&tm_out, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.act_q, static_cast<uint64_t>(p.n / 2),
                                    static_cast<uint64_t>(c.a_rows_total), static_cast<uint64_t>(p.act_q_row_stride), 64, 32,
                                    CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc) return rc;
        p.tma_store = c.whole_tile_stores ? 2 : 1;
    }

    int sms = 0;
    rc = effective_num_sms(&sms);
    if (rc) return rc;
    int grid = sms;
    if (c.max_tiles > 0) grid = std::min(grid, c.max_tiles);

    if (c.max_tiles > 0 && block_n == 256) grid = std::min(grid, std::max(1, c.max_tiles / 2));
#define DGB_LAUNCH(EPI, KIND)                                                                                   \
    return block_n == 256 ? launch_gemm<256, 4, EPI, KIND>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream)            \
                          : launch_gemm<128, 6, EPI, KIND>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream)
    if (bf16) {
        switch (c.epilogue) {
            case kEpiBF16: DGB_LAUNCH(kEpiBF16, kKindBf16);
            case kEpiSwiGLUBf16: return launch_gemm<256, 4, kEpiSwiGLUBf16, kKindBf16>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream);
            default: DGB_LAUNCH(kEpiF32, kKindBf16);
        }
    }
    if (nvfp4) {
        if (nvfp4_staged) return launch_gemm<256, 3, kEpiBF16, kKindNvfp4>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream);
        switch (c.epilogue) {
            case kEpiBF16: DGB_LAUNCH(kEpiBF16, kKindNvfp4);
            case kEpiF32: DGB_LAUNCH(kEpiF32, kKindNvfp4);
            case kEpiSwiGLUNvfp4: DGB_LAUNCH(kEpiSwiGLUNvfp4, kKindNvfp4);
            default: return fail(DGB200_EINVAL, "unknown epilogue %d for the NVFP4 kind", c.epilogue);
        }
    }
    switch (c.epilogue) {
        case kEpiBF16: DGB_LAUNCH(kEpiBF16, kKindFp8Fp4);
        case kEpiF32: DGB_LAUNCH(kEpiF32, kKindFp8Fp4);
        case kEpiSwiGLU:
            if (p.push != nullptr) return launch_gemm<256, 4, kEpiSwiGLUPush, kKindFp8Fp4>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream);
            DGB_LAUNCH(kEpiSwiGLU, kKindFp8Fp4);
        default: return fail(DGB200_EINVAL, "unknown epilogue %d", c.epilogue);
    }
#undef DGB_LAUNCH
}


// A side stream per device with the two events of a fork / join. The two halves of a GEMM that is split by group size
// touch disjoint experts: the swapped half is launched on the side stream, so its CTAs take over SMs one by one as
// the other half's CTAs retire instead of waiting for its last tile (both are persistent kernels of one CTA per SM).
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    std::mutex mu;  // one fork .. join sequence at a time per device (the events are shared)
};

int side_stream_for_current_device(SideStream** out) {
    constexpr int kMaxDevices = 64;
    static SideStream table[kMaxDevices];
    static std::mutex create_mu;
    int dev = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    DGB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
    SideStream& s = table[dev];
    {
        std::lock_guard<std::mutex> lock(create_mu);
        if (s.stream == nullptr) {
            DGB_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
            DGB_CUDA(cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming));
            DGB_CUDA(cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming));
        }
    }
    *out = &s;
    return 0;
}

// The second stream of the expert-parallel layer with the events that order it against the caller's stream: the
// kernels that move rows between ranks run there, on the SMs the GEMMs leave free, while the GEMMs of other expert
// phases run on the caller's stream.
struct EpStreams {
    cudaStream_t comm = nullptr;
    cudaEvent_t planned = nullptr, fetched = nullptr, returned = nullptr;
    cudaEvent_t pushed[kMaxEpPhases] = {}, computed[kMaxEpPhases] = {};
    std::mutex mu;  // one layer call at a time per device enqueues on these (the events are shared)
};

int ep_streams_for_current_device(EpStreams** out) {
    constexpr int kMaxDevices = 64;
    static EpStreams table[kMaxDevices];
    static std::mutex create_mu;
    int dev = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    DGB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
    EpStreams& s = table[dev];
    {
        std::lock_guard<std::mutex> lock(create_mu);
        if (s.comm == nullptr) {
            DGB_CUDA(cudaStreamCreateWithFlags(&s.comm, cudaStreamNonBlocking));
            cudaEvent_t* all[3] = {&s.planned, &s.fetched, &s.returned};
            for (cudaEvent_t* e : all) DGB_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
            for (int q = 0; q < kMaxEpPhases; ++q) {
                DGB_CUDA(cudaEventCreateWithFlags(&s.pushed[q], cudaEventDisableTiming));
                DGB_CUDA(cudaEventCreateWithFlags(&s.computed[q], cudaEventDisableTiming));
            }
        }
    }
    *out = &s;
    return 0;
}

// Launch shape of a row-moving kernel (dispatch push, return push): as many warps per CTA as row-sized slots fit into
// an SM's shared memory (one row in flight per warp), one CTA per SM. Beside GEMMs it runs as `comm_sms` such CTAs, each
// asking for at least kCommCtaSmemBytes of dynamic shared memory so that no second one and no GEMM CTA fits on its SM:
// together they occupy exactly `comm_sms` SMs instead of a few warps on every SM (the block scheduler spreads small
// CTAs over all SMs, and a GEMM CTA needs a whole SM's registers). Alone on the GPU it runs on every SM.
constexpr int kCommCtaSmemBytes = 120 * 1024;

struct RowMoverLaunch {
    int warps;
    int smem_bytes;
};

inline RowMoverLaunch row_mover_launch(long long slot_bytes, bool beside_gemms) {
    RowMoverLaunch r;
    r.warps = static_cast<int>(std::max(1ll, std::min<long long>(kRowMoverMaxWarps, (kRowMoverSmemBudget - 512) / slot_bytes)));
    const long long need = (r.warps * 8 + 15) / 16 * 16 + r.warps * slot_bytes;
    r.smem_bytes = static_cast<int>(beside_gemms ? std::max<long long>(need, kCommCtaSmemBytes) : need);
    return r;
}

template <typename Kernel>
int allow_row_mover_smem(Kernel kernel) {
    DGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRowMoverSmemBudget));
    return 0;
}

// The layer GEMMs with swapped operands (gemm_swap_kernel.cuh): weights on M, an expert's tokens on N. Takes the same
// call description as run_gemm; only the FP8 x FP4 / FP8 x FP8 kind, the psum layout with 128-row segments, scale
// factors in tcgen05.cp order and the SwiGLU / BF16 epilogues.
template <int EPI>
int launch_gemm_swap(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_sfx, const CUtensorMap& tm_sfw,
                     const GemmParams& p, int grid, cudaStream_t stream) {
    auto kernel = dgb200_swap_gemm_kernel<EPI>;
    static bool configured = false;
    static int configured_device = -1;
    int dev = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    if (!configured || configured_device != dev) {
        DGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SwapSmem::kDynamicBytes));
        configured = true;
        configured_device = dev;
    }
    DGB_CUDA(launch_kernel(kernel, dim3(grid), dim3(kGemmThreads), SwapSmem::kDynamicBytes, stream, use_pdl(), tm_x, tm_w, tm_sfx, tm_sfw, p));
    return 0;
}

int run_gemm_swap(GemmCall& c, cudaStream_t stream) {
    GemmParams& p = c.p;
    DGB_REQUIRE(c.kind == kKindFp8Fp4 && p.mode == kModePsum && p.alignment == 128 && p.sf_transposed == 1,
                "the swapped-operand kernel serves the FP8 layer path only");
    DGB_REQUIRE(c.epilogue == kEpiSwiGLU || c.epilogue == kEpiBF16, "unknown epilogue %d for the swapped-operand kernel", c.epilogue);
    DGB_REQUIRE(p.k > 0 && p.k % 128 == 0 && p.n > 0 && p.n % 256 == 0, "k must be a multiple of 128 and n of 256");
    DGB_REQUIRE(p.num_groups > 0 && p.num_groups <= kMaxCachedGroups, "at most %d groups", kMaxCachedGroups);
    DGB_REQUIRE(p.gran_a == 32 && p.gran_b == 32, "per-32 scales only");
    DGB_REQUIRE(c.sfa_k_stride % 4 == 0 && c.sfb_k_stride % 4 == 0 && c.sfb_k_stride >= p.n && c.sfa_k_stride >= c.a_rows_total,
                "packed scale-factor strides must be multiples of 4 ints that cover MN");
    const int packed_k = p.k / 128;
    DGB_REQUIRE(p.num_groups == 1 || c.sfb_group_stride == static_cast<long long>(packed_k) * c.sfb_k_stride,
                "scale factors of B: group stride must equal packed K x MN stride");
    p.sfb_packed_k = packed_k;
    if (c.a_rows_total == 0) return 0;
    CUtensorMap tm_x, tm_w, tm_sfx, tm_sfw;
    int rc = make_tensor_map_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.a, static_cast<uint64_t>(p.k),
                                static_cast<uint64_t>(c.a_rows_total), static_cast<uint64_t>(p.k), 128, kSwapMaxTok,
                                CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map_2d(&tm_sfx, CU_TENSOR_MAP_DATA_TYPE_INT32, c.sfa, static_cast<uint64_t>(c.sfa_k_stride),
                            static_cast<uint64_t>(packed_k), static_cast<uint64_t>(c.sfa_k_stride) * 4, 256, 1,
                            CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tensor_map_2d(&tm_sfw, CU_TENSOR_MAP_DATA_TYPE_INT32, c.sfb, static_cast<uint64_t>(c.sfb_k_stride),
                            static_cast<uint64_t>(p.num_groups) * packed_k, static_cast<uint64_t>(c.sfb_k_stride) * 4, 256, 1,
                            CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const uint64_t w_rows = static_cast<uint64_t>(p.num_groups) * p.n;
    if (c.b_is_fp4) {
        rc = make_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, c.b, static_cast<uint64_t>(p.k), w_rows,
                                static_cast<uint64_t>(p.k / 2), 128, 256, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = kFmtE2M1_F8F6F4;
        p.b_tx_bytes = 256 * 64;  // the mbarrier is credited with the packed bytes
    } else {
        rc = make_tensor_map_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, c.b, static_cast<uint64_t>(p.k), w_rows,
                                static_cast<uint64_t>(p.k), 128, 256, CU_TENSOR_MAP_SWIZZLE_128B);
        p.b_fmt = kFmtE4M3;
        p.b_tx_bytes = 256 * 128;
    }
    if (rc) return rc;
    int sms = 0;
    rc = effective_num_sms(&sms);
    if (rc) return rc;
    if (c.epilogue == kEpiSwiGLU) return launch_gemm_swap<kEpiSwiGLU>(tm_x, tm_w, tm_sfx, tm_sfw, p, sms, stream);
    return launch_gemm_swap<kEpiBF16>(tm_x, tm_w, tm_sfx, tm_sfw, p, sms, stream);
}

// --------------------------------------------------------------------------------------------------------------
// Mega-MoE buffer layout. One flat buffer per rank holds the caller-written inputs and every intermediate of the
// layer (the reference's counterpart: get_symm_buffer_size_for_mega_moe, csrc/apis/mega.hpp:34-155, and
// deep_gemm/include/deep_gemm/layout/mega_moe.cuh:46-443). All regions start on 1024-byte boundaries.
// --------------------------------------------------------------------------------------------------------------
// Rows each expert's segment of the expert-sorted buffers is padded to: one M tile, so that a tile's rows (and the
// 128-row groups of its scale factors, stored in tcgen05.cp order) never straddle two experts.
constexpr int kSegmentAlignment = 128;

// Optional CUDA events the next mega-MoE call records at its stage boundaries (set per host thread, used once).
constexpr int kNumStageEvents = 6;
thread_local cudaEvent_t g_stage_events[kNumStageEvents];
thread_local int g_num_stage_events = 0;

int record_stage(int index, cudaStream_t stream) {
    if (index < g_num_stage_events && g_stage_events[index] != nullptr) DGB_CUDA(cudaEventRecord(g_stage_events[index], stream));
    return 0;
}  // rows each expert segment is padded to in the expert-sorted buffers

struct MegaLayout {
    long long x, x_sf, topk_idx, topk_weights;                            // inputs, written by the caller
    long long chunk_hist, expert_start, expert_end, total_rows, dest_row;  // dispatch plan
    long long src_of_row, row_weight;
    long long all_counts, my_base, flags;  // expert-parallel exchange: counts of every rank, this rank's bases, barrier flags
    // hot-expert row spill (expert parallel): computing rank and expert slot of this rank's entries per expert, the
    // experts this rank hosts in its guest slots, every rank's rows before / after the spill
    long long my_dest, my_slot, guest_expert, rank_rows;
    long long l1_acts, l1_sf, l2_acts, l2_sf, l2_out;  // l2_out: bf16 [max_rows, hidden], the rows the combine gathers
    long long l1_sf_stage;  // expert parallel: row-major landing area of pushed scale ints [max_rows][ints per row]
    long long l1_tmp;  // FP8 kind: bf16 [max_rows, 2 * inter], gate/up activations of the experts the swapped kernel serves
    long long combine_partial;  // expert parallel, pull combine: fp32 [max tokens, hidden], the running sums between phases
    long long push_lists;  // expert parallel: [kMaxEpPhases] entry lists (max tokens * topk ints each) of the dispatch that rides on the
                           // gate/up GEMMs, then kMaxEpPhases counters, then kMaxEpPhases PushWork descriptors
    long long returned;  // expert parallel, return push: bf16 [max tokens * topk, hidden], the output rows the computing ranks sent back
    long long tile_done;  // FP8 kind: one counter per token tile of the fused expert-MLP kernel (max_rows / 128 + local experts)
    // shared experts (token order, token_rows = capacity in rows): x scales in GEMM order, activations, output rows
    long long shared_x_sf, shared_l2_acts, shared_l2_sf, shared_out;
    long long token_rows;
    long long total;
    long long max_rows;  // capacity of the expert-sorted buffers (rows), a multiple of 128
    int num_chunks, num_local_experts;
    int num_slots;  // expert segments the plan arrays hold: the local experts plus, expert parallel, kMaxGuestExperts guest slots
};

// Quantisation of the layer: the FP8 x MXFP4 path needs nothing beyond the tensors; the NVFP4 path carries the
// per-tensor FP32 scales (device pointers; x_scale and act_scale hold one value and must be equal on every rank).
struct LayerQuant {
    int kind = kKindFp8Fp4;
    const float* x_scale = nullptr;    // scale of the NVFP4 input rows
    const float* act_scale = nullptr;  // calibrated scale the post-SwiGLU activations are quantised against
    const float* l1_scales = nullptr;  // [local experts] scales of the gate/up weights
    const float* l2_scales = nullptr;  // [local experts] scales of the down weights
    // FP8 kind only: take the activations as BF16 rows and quantise them while dispatching (the buffer's x / x_sf
    // views are then neither read nor written)
    const __nv_bfloat16* x_bf16 = nullptr;
    long long x_bf16_row_stride = 0;
    // FP8 kind only: shared experts, a dense FP8 x FP8 MLP (per-32 UE8M0 scales) over this rank's own tokens whose
    // output is one more combine slot (reference: csrc/apis/mega.hpp:211-232). inter = 0: none.
    const void* shared_l1_w = nullptr;
    const void* shared_l1_w_sf = nullptr;
    const void* shared_l2_w = nullptr;
    const void* shared_l2_w_sf = nullptr;
    int shared_inter = 0;
    // expert parallel, FP8 kind only: hot-expert row spill. guest_slots > 0: the four weight tensors of every rank have
    // room for that many guest experts after the rank's own and peer_w[i][r] is the address of tensor i (gate/up weights,
    // their scales, down weights, their scales) on rank r as mapped into this process.
    int guest_slots = 0;
    const uint64_t* peer_w[4] = {nullptr, nullptr, nullptr, nullptr};
};

// Bytes of one quantised activation row of `width` elements, and packed scale ints (4 scale bytes each) per row.
inline long long act_row_bytes(int kind, int width) { return kind == kKindNvfp4 ? width / 2 : (kind == kKindBf16 ? width * 2 : width); }
inline int sf_ints_per_row(int kind, int width) { return kind == kKindNvfp4 ? width / 64 : (kind == kKindBf16 ? 0 : width / 128); }

int make_mega_layout(int kind, int num_ranks, int num_experts, int max_tokens, int topk, int hidden, int inter, MegaLayout* out,
                     int shared_inter = 0) {
    DGB_REQUIRE(num_ranks >= 1 && num_ranks <= kMaxRanks, "num_ranks must be in [1, %d]", kMaxRanks);
    DGB_REQUIRE(num_experts > 0 && num_experts % num_ranks == 0, "num_experts must be a positive multiple of num_ranks");
    DGB_REQUIRE(max_tokens > 0 && topk > 0 && topk <= 32, "need max tokens > 0 and 0 < topk <= 32");
    const int k_block = kind == kKindNvfp4 ? 256 : 128;
    DGB_REQUIRE(hidden % k_block == 0 && inter % k_block == 0 && hidden > 0 && inter > 0,
                "hidden and intermediate_hidden must be positive multiples of %d", k_block);
    MegaLayout l{};
    l.num_local_experts = num_experts / num_ranks;
    const long long active_topk = std::min(topk, l.num_local_experts);
    const long long routed = static_cast<long long>(max_tokens) * num_ranks * active_topk;
    l.num_slots = l.num_local_experts + (num_ranks > 1 ? kMaxGuestExperts : 0);
    l.max_rows = (routed + static_cast<long long>(l.num_slots) * kSegmentAlignment + 127) / 128 * 128;
    l.num_chunks = static_cast<int>((static_cast<long long>(max_tokens) * topk + kPlanChunk - 1) / kPlanChunk);
    long long off = 0;
    auto take = [&off](long long bytes) {
        const long long at = off;
        off += (bytes + 1023) / 1024 * 1024;
        return at;
    };
    l.x = take(static_cast<long long>(max_tokens) * act_row_bytes(kind, hidden));
    l.x_sf = take(static_cast<long long>(max_tokens) * sf_ints_per_row(kind, hidden) * 4);
    l.topk_idx = take(static_cast<long long>(max_tokens) * topk * 8);
    l.topk_weights = take(static_cast<long long>(max_tokens) * topk * 4);
    l.chunk_hist = take(static_cast<long long>(l.num_chunks) * num_experts * 4);
    l.all_counts = take(static_cast<long long>(num_ranks) * num_experts * 4);
    l.my_base = take(num_experts * 4ll);
    l.flags = take(kEpFlagRows * kMaxEpRanks * 4);
    l.expert_start = take(l.num_slots * 4ll);
    l.expert_end = take(l.num_slots * 4ll);
    l.my_dest = take(num_experts * 4ll);
    l.my_slot = take(num_experts * 4ll);
    l.guest_expert = take(kMaxGuestExperts * 4);
    l.rank_rows = take(2 * kMaxEpRanks * 4);
    l.total_rows = take(16);
    l.dest_row = take(static_cast<long long>(max_tokens) * topk * 4);
    l.src_of_row = take(l.max_rows * 4);
    l.row_weight = take(l.max_rows * 4);
    l.l1_acts = take(l.max_rows * act_row_bytes(kind, hidden));
    l.l1_sf = take(l.max_rows * sf_ints_per_row(kind, hidden) * 4);
    l.l2_acts = take(l.max_rows * act_row_bytes(kind, inter));
    l.l2_sf = take(l.max_rows * sf_ints_per_row(kind, inter) * 4);
    l.l2_out = take(l.max_rows * hidden * 2);
    l.l1_tmp = kind == kKindFp8Fp4 ? take(l.max_rows * inter * 4) : 0;
    l.tile_done = kind == kKindFp8Fp4 ? take((l.max_rows / 128 + l.num_slots) * 4) : 0;
    l.l1_sf_stage = num_ranks > 1 ? take(l.max_rows * sf_ints_per_row(kind, hidden) * 4) : 0;
    l.combine_partial = num_ranks > 1 ? take(static_cast<long long>(max_tokens) * hidden * 4) : 0;
    l.push_lists = num_ranks > 1 ? take(kMaxEpPhases * (static_cast<long long>(max_tokens) * topk * 4 + 64 + static_cast<long long>(sizeof(PushWork)))) : 0;
    l.returned = num_ranks > 1 ? take(static_cast<long long>(max_tokens) * topk * hidden * 2) : 0;
    l.token_rows = (static_cast<long long>(max_tokens) + 127) / 128 * 128;
    if (shared_inter > 0) {
        DGB_REQUIRE((kind == kKindFp8Fp4 || kind == kKindBf16) && shared_inter % 128 == 0,
                    "shared experts need the FP8 x FP4 or the BF16 layer and a multiple of 128 channels");
        DGB_REQUIRE(max_tokens % 128 == 0, "with shared experts the token capacity must be a multiple of 128");
        l.shared_x_sf = take(l.token_rows * sf_ints_per_row(kind, hidden) * 4);
        l.shared_l2_acts = take(l.token_rows * act_row_bytes(kind, shared_inter));
        l.shared_l2_sf = take(l.token_rows * sf_ints_per_row(kind, shared_inter) * 4);
        l.shared_out = take(l.token_rows * hidden * 2);
    }
    l.total = off;
    *out = l;
    return 0;
}

int run_cast(bool fp4, const void* x, long long x_row_stride, int rows, int k, int gran_k, void* q, long long q_row_stride,
             float* sf_f32, void* sf_packed, long long sf_k_stride, long long sf_row_stride, cudaStream_t stream) {
    DGB_REQUIRE(rows >= 0 && k > 0 && k % 16 == 0, "k (%d) must be a positive multiple of 16", k);
    DGB_REQUIRE(gran_k == 32 || gran_k == 128, "gran_k must be 32 or 128, got %d", gran_k);
    DGB_REQUIRE(x != nullptr && q != nullptr, "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && (x_row_stride * 2) % 16 == 0, "x rows must be 16-byte aligned");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(q) % 16 == 0 && q_row_stride % (fp4 ? 8 : 16) == 0, "q rows must be 16-byte aligned");
    DGB_REQUIRE(sf_f32 != nullptr || sf_packed != nullptr, "at least one scale-factor output is required");
    DGB_REQUIRE(sf_packed == nullptr || (sf_row_stride == 1 && sf_k_stride >= rows) ||
                    (sf_k_stride == 1 && sf_row_stride >= (k + gran_k * 4 - 1) / (gran_k * 4)),
                "packed scale-factor strides must be (k stride >= rows, row stride 1) or (k stride 1, row stride >= packed k)");
    if (rows == 0) return 0;
    CastParams p{};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.x_row_stride = x_row_stride;
    p.q = q;
    p.q_row_stride = q_row_stride;
    p.sf_f32 = sf_f32;
    p.sf_packed = static_cast<uint32_t*>(sf_packed);
    p.sf_k_stride = sf_k_stride;
    p.sf_row_stride = sf_row_stride;
    p.rows = rows;
    p.k = k;
    p.gran_k = gran_k;
    const dim3 grid((k + 511) / 512, (rows + 31) / 32);
    if (fp4)
        dgb200_cast_rows_kernel<true><<<grid, 256, 0, stream>>>(p);
    else
        dgb200_cast_rows_kernel<false><<<grid, 256, 0, stream>>>(p);
    DGB_CUDA(cudaGetLastError());
    return 0;
}


// Both GEMMs of the FP8 x MXFP4 layer in one launch of the fused expert-MLP kernel (expert_mlp_kernel.cuh).
int run_expert_mlp(bool pair, const MegaLayout& l, uint8_t* base, const void* l1_w, const void* l1_w_sf, const void* l2_w,
                   const void* l2_w_sf, int hidden, int inter, float activation_clamp, int fast_math, cudaStream_t stream) {
    const int E = l.num_local_experts;
    const int ctas = pair ? 2 : 1;
    DGB_REQUIRE(E <= kMlpMaxExperts, "the fused expert-MLP kernel holds the tables of at most %d experts per rank", kMlpMaxExperts);
    DGB_REQUIRE((2 * inter) % (128 * ctas) == 0 && hidden % (128 * ctas) == 0 && hidden % 128 == 0 && inter % 128 == 0,
                "hidden and 2 x intermediate_hidden must be multiples of %d", 128 * ctas);
    MlpMaps maps;
    MlpParams p{};
    p.expert_end = reinterpret_cast<const int*>(base + l.expert_end);
    p.num_experts = E;
    p.phase_mask = 3;
    p.ph[0] = MlpPhase{2 * inter, hidden, 8192u, kFmtE2M1_F8F6F4};
    p.ph[1] = MlpPhase{hidden, inter, 8192u, kFmtE2M1_F8F6F4};
    p.act_q = base + l.l2_acts;
    p.act_q_row_stride = inter;
    p.out = reinterpret_cast<__nv_bfloat16*>(base + l.l2_out);
    p.out_row_stride = hidden;
    p.act_sf = base + l.l2_sf;
    p.act_sf_k_stride = l.max_rows;
    p.row_weight = reinterpret_cast<const float*>(base + l.row_weight);
    p.clamp = (activation_clamp > 0.0f && activation_clamp < 3.0e38f) ? activation_clamp : 0.0f;
    p.fast_math = fast_math;
    p.tile_done = reinterpret_cast<unsigned*>(base + l.tile_done);
    int sms = 0;
    int rc = effective_num_sms(&sms);
    if (rc) return rc;
    const int num_clusters = std::max(1, sms / ctas);
    p.tiles_per_group = std::max(1, (2 * num_clusters + p.ph[0].n / (128 * ctas) - 1) / (p.ph[0].n / (128 * ctas)));
    const uint64_t rows = static_cast<uint64_t>(l.max_rows);
    const void* x[2] = {base + l.l1_acts, base + l.l2_acts};
    const void* sfx[2] = {base + l.l1_sf, base + l.l2_sf};
    const void* w[2] = {l1_w, l2_w};
    const void* sfw[2] = {l1_w_sf, l2_w_sf};
    for (int ph = 0; ph < 2; ++ph) {
        const uint64_t k = static_cast<uint64_t>(p.ph[ph].k), n = static_cast<uint64_t>(p.ph[ph].n);
        for (int i = 0; i < kMlpXMaps; ++i)
            if ((rc = make_tensor_map_2d(&maps.x[ph][i], CU_TENSOR_MAP_DATA_TYPE_UINT8, x[ph], k, rows, k, 128, 16 * (i + 1), CU_TENSOR_MAP_SWIZZLE_128B)))
                return rc;
        if ((rc = make_tensor_map_2d(&maps.w[ph], CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, w[ph], 128, static_cast<uint64_t>(E) * n * (k / 128), 64,
                                     128, 256, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
        if ((rc = make_tensor_map_2d(&maps.sfx[ph], CU_TENSOR_MAP_DATA_TYPE_INT32, sfx[ph], rows, k / 128, rows * 4, 128, 2, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
        if ((rc = make_tensor_map_2d(&maps.sfw[ph], CU_TENSOR_MAP_DATA_TYPE_INT32, sfw[ph], n, static_cast<uint64_t>(E) * (k / 128), n * 4, 128, 2,
                                     CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    }
    DGB_CUDA(cudaMemsetAsync(p.tile_done, 0, static_cast<size_t>(l.max_rows / 128 + E) * 4, stream));

    const int smem_bytes = pair ? MlpSmem<true>::kTotal : MlpSmem<false>::kTotal;
    const void* kernel = pair ? reinterpret_cast<const void*>(&dgb200_expert_mlp_kernel<true>)
                              : reinterpret_cast<const void*>(&dgb200_expert_mlp_kernel<false>);
    static int configured_device[2] = {-1, -1};
    int dev = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    if (configured_device[pair ? 1 : 0] != dev) {
        DGB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured_device[pair ? 1 : 0] = dev;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(num_clusters * ctas));
    cfg.blockDim = dim3(kMlpThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void* args[2] = {&maps, &p};
    DGB_CUDA(cudaLaunchKernelExC(&cfg, kernel, args));
    return 0;
}

// The two grouped GEMMs of the layer over this rank's expert-sorted rows (shared by the single-rank and the
// expert-parallel paths): L1 writes quantised activations + scales (FP8/UE8M0 or NVFP4/UE4M3), L2 writes BF16 rows
// into l2_out in the same row order.
// Which tile orientation serves the layer's two GEMMs (the reasons are in run_layer_gemms).
enum LayerOrientation { kOrientM, kOrientSplit, kOrientSwapAll };

LayerOrientation layer_orientation(int kind, int num_groups, int hidden, int intermediate_hidden, long long expected_rows_per_expert) {
    if (kind == kKindFp8Fp4 && num_groups <= kMaxCachedGroups && (2 * intermediate_hidden) % 256 == 0 && hidden % 256 == 0) {
        if (tuning().swap_ab == 1 || (tuning().swap_ab == -1 && expected_rows_per_expert <= 40)) return kOrientSwapAll;
        if (tuning().swap_ab == 2 ||
            (tuning().swap_ab == -1 && expected_rows_per_expert >= 100 && expected_rows_per_expert <= kSwapMaxTok + 16))
            return kOrientSplit;
    }
    return kOrientM;
}

// Where the down GEMM of the expert-parallel layer may send its output rows instead of writing them to l2_out: row r goes
// to row src_of_row[r] % entries_per_rank of the `returned` buffer of rank src_of_row[r] / entries_per_rank.
struct ReturnSpec {
    const int* src_of_row;
    int entries_per_rank;
    unsigned long long returned_base[kMaxRanks];
};

int run_layer_gemms(const LayerQuant& quant, const MegaLayout& l, uint8_t* base, const void* l1_w, const void* l1_w_sf, const void* l2_w,
                    const void* l2_w_sf, int hidden, int intermediate_hidden, float activation_clamp, int fast_math,
                    cudaStream_t stream, int stage_event_base, long long expected_rows_per_expert, int group_begin = 0,
                    int group_end = 0, const ReturnSpec* ret = nullptr, bool* returned_by_gemm = nullptr,
                    const PushWork* push = nullptr) {
    const int E = l.num_local_experts + quant.guest_slots;  // guest slots follow the rank's own experts, in the plan and in the weights
    // [group_begin, group_end): the expert slots this call computes ({0, 0} = all of them)
    const int first_expert = (group_begin == 0 && group_end == 0) ? 0 : group_begin;
    const int num_call_experts = (group_begin == 0 && group_end == 0) ? E : group_end - group_begin;
    const int* expert_end = reinterpret_cast<const int*>(base + l.expert_end);
    const bool nvfp4 = quant.kind == kKindNvfp4;
    const bool bf16 = quant.kind == kKindBf16;
    // Which tile orientation serves which experts (measured on B200, hidden 7168, 256 experts):
    //   few rows per expert (decode): everything through the swapped-operand kernel, whose MMA time follows the token
    //     count (256 tokens: step 1.23 -> 1.12 ms); its fused SwiGLU epilogue is cheap while a tile holds few tokens;
    //   around 128 rows per expert: split by group size, experts of 129..kSwapMaxTok rows through the swapped kernel
    //     (one pass over their weights instead of two), all others through the tokens-on-M kernel. The swapped half of
    //     the gate/up GEMM stores BF16 gate/up values into l1_tmp and dgb200_swiglu_requant_rows_kernel finishes those
    //     rows (same bits as the fused epilogue): at this size the swapped kernel's own SwiGLU epilogue, a fully unrolled
    //     walk over up to 80 tokens per thread, is instruction-fetch bound. The split costs four more launches, which
    //     only pays where such experts are common;
    //   otherwise the tokens-on-M kernel alone (with many rows per expert both orientations run 128-row tiles).
    // dgb200_set_tuning("swap_ab", 0 / 1) forces the tokens-on-M kernel / the swapped kernel with its fused epilogue.
    if (!nvfp4 && !bf16 && mlp_kernel_choice() != 0) {
        DGB_REQUIRE(group_begin == 0 && group_end == 0, "the fused expert-MLP kernel computes all experts of a rank in one launch");
        const bool pair = mlp_kernel_choice() == 2 && (2 * intermediate_hidden) % 256 == 0 && hidden % 256 == 0;
        const int rc_mlp = run_expert_mlp(pair, l, base, l1_w, l1_w_sf, l2_w, l2_w_sf, hidden, intermediate_hidden,
                                          activation_clamp, fast_math, stream);
        if (rc_mlp) return rc_mlp;
        const int rc_ev = record_stage(stage_event_base, stream);  // one launch: the down stage's share is inside the first interval
        return rc_ev ? rc_ev : record_stage(stage_event_base + 1, stream);
    }
    const LayerOrientation orient = layer_orientation(quant.kind, E, hidden, intermediate_hidden, expected_rows_per_expert);
    int rc = 0;
    auto run_split = [&](GemmCall& c) -> int {
        if (orient == kOrientM) return run_gemm(c, stream);
        if (orient == kOrientSwapAll) return run_gemm_swap(c, stream);
        GemmCall c2 = c;
        const int split_lo = tuning().swap_ab == 2 ? 1 : 129;  // 2: every expert that fits one token tile (experiments)
        c.p.rows_lo = c2.p.rows_lo = split_lo;
        c.p.rows_hi = c2.p.rows_hi = kSwapMaxTok;
        c.p.rows_skip = 1;
        c2.p.rows_skip = 0;
        const bool gate_up = c.epilogue == kEpiSwiGLU;
        if (gate_up) {
            c2.epilogue = kEpiBF16;
            c2.p.d = base + l.l1_tmp;
            c2.p.d_row_stride = 2 * intermediate_hidden;
        }
        SideStream* side = nullptr;
        int rc1 = side_stream_for_current_device(&side);
        if (rc1) return rc1;
        std::lock_guard<std::mutex> lock(side->mu);
        DGB_CUDA(cudaEventRecord(side->fork, stream));
        DGB_CUDA(cudaStreamWaitEvent(side->stream, side->fork, 0));
        rc1 = run_gemm(c, stream);
        if (rc1 == 0) rc1 = run_gemm_swap(c2, side->stream);
        if (rc1 == 0 && gate_up) {
            const dim3 grid((kSwapMaxTok + 7) / 8, num_call_experts);
            dgb200_swiglu_requant_rows_kernel<<<grid, 256, 0, side->stream>>>(
                reinterpret_cast<const __nv_bfloat16*>(base + l.l1_tmp), reinterpret_cast<const int*>(base + l.expert_start), expert_end,
                split_lo, kSwapMaxTok, intermediate_hidden, c.p.row_weight, c.p.clamp, c.p.fast_math, c.p.act_q, c.p.act_q_row_stride,
                reinterpret_cast<unsigned*>(c.p.act_sf), c.p.act_sf_k_stride, first_expert);
            if (cudaGetLastError() != cudaSuccess) rc1 = fail(DGB200_ECUDA, "launch of the SwiGLU finisher failed");
        }
        // join even after a failed launch, so that the side stream never runs ahead of the caller's stream
        DGB_CUDA(cudaEventRecord(side->join, side->stream));
        DGB_CUDA(cudaStreamWaitEvent(stream, side->join, 0));
        return rc1;
    };
    {
        GemmCall c{};
        c.kind = quant.kind;
        c.a = base + l.l1_acts;
        c.b = l1_w;
        c.a_rows_total = l.max_rows;
        c.b_is_fp4 = 1;
        c.epilogue = nvfp4 ? kEpiSwiGLUNvfp4 : (bf16 ? kEpiSwiGLUBf16 : kEpiSwiGLU);
        c.a_row_stride_bytes = c.b_row_stride_bytes = hidden * 2ll;  // BF16 kind
        c.whole_tile_stores = 1;
        c.max_tiles = 0;
        c.sfa = base + l.l1_sf;
        c.sfb = l1_w_sf;
        c.sfa_k_stride = l.max_rows;
        c.sfa_group_stride = 0;
        c.num_groups_a = 1;
        c.sfb_k_stride = 2 * intermediate_hidden;
        c.sfb_group_stride = static_cast<long long>(sf_ints_per_row(quant.kind, hidden)) * 2 * intermediate_hidden;
        GemmParams& p = c.p;
        p.layout = expert_end;
        p.mode = kModePsum;
        p.m = static_cast<int>(l.max_rows);
        p.n = 2 * intermediate_hidden;
        p.k = hidden;
        p.num_groups = E;
        p.group_begin = group_begin;
        p.group_end = group_end;
        p.alignment = kSegmentAlignment;
        p.gran_a = 32;
        p.gran_b = 32;
        p.act_q = base + l.l2_acts;
        p.act_sf = base + l.l2_sf;
        p.act_q_row_stride = act_row_bytes(quant.kind, intermediate_hidden);
        p.act_sf_k_stride = l.max_rows;
        p.a_scale = quant.x_scale;
        p.b_scales = quant.l1_scales;
        p.out_scale = quant.act_scale;
        p.sf_transposed = 1;      // the gather / push kernels and transform_weights_for_mega_moe store tcgen05.cp order
        p.act_sf_transposed = 1;  // ... and so does this GEMM's epilogue for the next one
        p.row_weight = reinterpret_cast<const float*>(base + l.row_weight);
        p.clamp = (activation_clamp > 0.0f && activation_clamp < 3.0e38f) ? activation_clamp : 0.0f;
        p.fast_math = fast_math;
        if (push != nullptr && orient == kOrientM && !nvfp4 && !bf16) p.push = push;  // device memory; the caller checked that this variant runs
        if ((rc = run_split(c))) return rc;
    }
    if ((rc = record_stage(stage_event_base, stream))) return rc;
    {
        GemmCall c{};
        c.kind = quant.kind;
        c.a = base + l.l2_acts;
        c.b = l2_w;
        c.a_rows_total = l.max_rows;
        c.b_is_fp4 = 1;
        c.epilogue = kEpiBF16;
        c.a_row_stride_bytes = c.b_row_stride_bytes = intermediate_hidden * 2ll;  // BF16 kind
        c.whole_tile_stores = 1;
        c.max_tiles = 0;
        c.sfa = base + l.l2_sf;
        c.sfb = l2_w_sf;
        c.sfa_k_stride = l.max_rows;
        c.sfa_group_stride = 0;
        c.num_groups_a = 1;
        c.sfb_k_stride = hidden;
        c.sfb_group_stride = static_cast<long long>(sf_ints_per_row(quant.kind, intermediate_hidden)) * hidden;
        GemmParams& p = c.p;
        p.layout = expert_end;
        p.mode = kModePsum;
        p.m = static_cast<int>(l.max_rows);
        p.n = hidden;
        p.k = intermediate_hidden;
        p.num_groups = E;
        p.group_begin = group_begin;
        p.group_end = group_end;
        p.alignment = kSegmentAlignment;
        p.gran_a = 32;
        p.gran_b = 32;
        p.d = base + l.l2_out;
        p.d_row_stride = hidden;
        p.a_scale = quant.act_scale;
        p.b_scales = quant.l2_scales;
        p.sf_transposed = 1;
        // GEMM and return transfer in one kernel: only the 256-wide tokens-on-M kernel of the FP8 x FP4 kind has the
        // epilogue for it; otherwise the caller sends the rows of l2_out with a kernel of its own
        const bool fuse_return = ret != nullptr && orient == kOrientM && !nvfp4 && !bf16 && hidden % 256 == 0 &&
                                 (tuning().block_n == 0 || tuning().block_n == 256);
        if (fuse_return) {
            p.ret_src = ret->src_of_row;
            p.ret_entries_per_rank = ret->entries_per_rank;
            for (int r = 0; r < kMaxRanks; ++r) p.ret_base[r] = ret->returned_base[r];
        }
        if (returned_by_gemm != nullptr) *returned_by_gemm = fuse_return;
        if ((rc = run_split(c))) return rc;
    }
    return record_stage(stage_event_base + 1, stream);
}

// The shared experts' two dense GEMMs over this rank's tokens (token order): x (FP8, scales already in GEMM order)
// -> SwiGLU (routing weight 1) + FP8 requant -> down GEMM -> bf16 rows in shared_out, the extra combine slot.
int run_shared_gemms(const LayerQuant& quant, const MegaLayout& l, uint8_t* base, int num_tokens, int hidden,
                     float activation_clamp, int fast_math, cudaStream_t stream) {
    const int si = quant.shared_inter;
    const bool bf16 = quant.kind == kKindBf16;
    int rc = 0;
    {
        GemmCall c{};
        c.kind = quant.kind;
        c.a = base + l.x;
        c.b = quant.shared_l1_w;
        c.a_rows_total = l.token_rows;
        c.a_row_stride_bytes = c.b_row_stride_bytes = hidden * 2ll;  // BF16 kind
        c.b_is_fp4 = 0;
        c.epilogue = bf16 ? kEpiSwiGLUBf16 : kEpiSwiGLU;
        c.whole_tile_stores = 1;
        c.sfa = base + l.shared_x_sf;
        c.sfb = quant.shared_l1_w_sf;
        c.sfa_k_stride = l.token_rows;
        c.num_groups_a = 1;
        c.sfb_k_stride = 2 * si;
        GemmParams& p = c.p;
        p.mode = kModeDense;
        p.m = num_tokens;
        p.n = 2 * si;
        p.k = hidden;
        p.num_groups = 1;
        p.alignment = 128;
        p.gran_a = 32;
        p.gran_b = 32;
        p.act_q = base + l.shared_l2_acts;
        p.act_sf = base + l.shared_l2_sf;
        p.act_q_row_stride = act_row_bytes(quant.kind, si);
        p.act_sf_k_stride = l.token_rows;
        p.row_weight = nullptr;
        p.clamp = (activation_clamp > 0.0f && activation_clamp < 3.0e38f) ? activation_clamp : 0.0f;
        p.fast_math = fast_math;
        p.sf_transposed = 1;
        p.act_sf_transposed = 1;
        if ((rc = run_gemm(c, stream))) return rc;
    }
    {
        GemmCall c{};
        c.kind = quant.kind;
        c.a = base + l.shared_l2_acts;
        c.b = quant.shared_l2_w;
        c.a_rows_total = l.token_rows;
        c.a_row_stride_bytes = c.b_row_stride_bytes = si * 2ll;  // BF16 kind
        c.b_is_fp4 = 0;
        c.epilogue = kEpiBF16;
        c.whole_tile_stores = 1;
        c.sfa = base + l.shared_l2_sf;
        c.sfb = quant.shared_l2_w_sf;
        c.sfa_k_stride = l.token_rows;
        c.num_groups_a = 1;
        c.sfb_k_stride = hidden;
        GemmParams& p = c.p;
        p.mode = kModeDense;
        p.m = num_tokens;
        p.n = hidden;
        p.k = si;
        p.num_groups = 1;
        p.alignment = 128;
        p.gran_a = 32;
        p.gran_b = 32;
        p.d = base + l.shared_out;
        p.d_row_stride = hidden;
        p.sf_transposed = 1;
        if ((rc = run_gemm(c, stream))) return rc;
    }
    return 0;
}

// Scales of x for the shared experts' first GEMM when the caller quantised x into the buffer (token-major ints).
int run_shared_x_sf(const MegaLayout& l, uint8_t* base, int num_tokens, int hidden, cudaStream_t stream) {
    const int ints = hidden / 128;
    dgb200_sf_rows_to_cp_order_kernel<<<(num_tokens + 31) / 32, 256, ints * 33 * sizeof(unsigned), stream>>>(
        reinterpret_cast<const unsigned*>(base + l.x_sf), num_tokens, ints, reinterpret_cast<unsigned*>(base + l.shared_x_sf),
        l.token_rows, nullptr, nullptr, nullptr);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

int run_mega_moe_ep(const LayerQuant& quant, const MegaLayout& l, void* y, const void* l1_w, const void* l1_w_sf, const void* l2_w, const void* l2_w_sf,
                    int32_t* stats, uint8_t* base, const uint64_t* peer_buffer_ptrs, int rank, int num_ranks, int num_tokens,
                    int num_max_tokens_per_rank, int num_experts, int num_topk, int hidden, int intermediate_hidden,
                    float activation_clamp, int fast_math, cudaStream_t stream) {
    // Expert-parallel layer. The expert slots of every rank (own experts, then guest slots) are cut into `phases` phases:
    //   count -> publish counts -> flag row 0 (signal + wait) -> plan (every rank derives the same one) -> assign
    //   for each phase q: push the entries routed to phase-q slots to the ranks that compute them -> signal "dispatch q"
    //   for each phase q: wait "dispatch q" of all ranks -> scale reorder -> L1(q) -> L2(q) -> signal "outputs q"
    //   wait "outputs q" of all ranks -> combine
    // Three arrangements, chosen below:
    //   guest experts (balanced loads), one stream: a single phase; the down GEMM sends its output rows to their source
    //     ranks from its epilogue (or a return-push kernel does, where the GEMM variant cannot); the combine is a local sum;
    //   rows stay on their owners, one stream: up to kMaxEpPhases phases, and the combine pulls the rows of each finished
    //     phase while the most loaded rank still computes the next;
    //   ep_comm_sms > 0: pushes and return pushes on a second stream, on SMs the GEMMs leave free.
    // Reference: the fused kernel overlaps the same traffic tile by tile (sm100_fp8_fp4_mega_moe.cuh:533-556, :1274-1300)
    // behind three barriers (comm/barrier.cuh:47-89).
    PeerTable peers{};
    for (int r = 0; r < num_ranks; ++r) {
        DGB_REQUIRE(peer_buffer_ptrs[r] != 0, "peer buffer %d is not mapped", r);
        peers.p[r] = peer_buffer_ptrs[r];
    }
    const int E = l.num_local_experts;
    const int entries = num_tokens * num_topk;
    const int chunks = std::max(1, (entries + kPlanChunk - 1) / kPlanChunk);
    const int entries_per_rank = num_max_tokens_per_rank * num_topk;
    const bool with_shared = quant.shared_inter > 0;
    const int sf_per_row = sf_ints_per_row(quant.kind, hidden);
    const bool fused_mlp = quant.kind == kKindFp8Fp4 && mlp_kernel_choice() != 0;
    // hot-expert row spill: V = own experts + guest slots; the plan decides which rows of which experts move
    const int G = quant.guest_slots;
    const int V = E + G;
    const bool spill = G > 0;
    GuestWeightTables guest_tables{};
    if (spill) {
        DGB_REQUIRE(quant.kind == kKindFp8Fp4 && !fused_mlp, "guest experts need the FP8 x MXFP4 layer with its separate GEMM kernels");
        DGB_REQUIRE(G <= kMaxGuestExperts && V <= kMaxSpillSlots - 1, "at most %d guest experts and %d expert slots per rank",
                    kMaxGuestExperts, kMaxSpillSlots - 1);
        DGB_REQUIRE(static_cast<long long>(num_ranks) * num_experts * 6 <= 30 * 1024, "too many experts x ranks for the spill plan's tables");
        const void* local_w[4] = {l1_w, l1_w_sf, l2_w, l2_w_sf};
        const long long bytes[4] = {2ll * intermediate_hidden * hidden / 2, 2ll * intermediate_hidden * (hidden / 128) * 4,
                                    static_cast<long long>(hidden) * intermediate_hidden / 2,
                                    static_cast<long long>(hidden) * (intermediate_hidden / 128) * 4};
        for (int i = 0; i < 4; ++i) {
            DGB_REQUIRE(quant.peer_w[i] != nullptr, "guest experts need the peer addresses of all four weight tensors");
            for (int r = 0; r < num_ranks; ++r) {
                DGB_REQUIRE(quant.peer_w[i][r] != 0 && quant.peer_w[i][r] % 16 == 0, "weight tensor %d of rank %d is not mapped", i, r);
                guest_tables.peer[i][r] = quant.peer_w[i][r];
            }
            DGB_REQUIRE(quant.peer_w[i][rank] == reinterpret_cast<uintptr_t>(local_w[i]),
                        "the peer address table does not name this rank's weight tensor %d", i);
            guest_tables.local[i] = reinterpret_cast<uintptr_t>(local_w[i]);
            guest_tables.bytes[i] = bytes[i];
        }
    }
    const int* my_dest = spill ? reinterpret_cast<const int*>(base + l.my_dest) : nullptr;
    const int* my_slot = spill ? reinterpret_cast<const int*>(base + l.my_slot) : nullptr;
    // Expert phases: several when their transfers can hide something, i.e. under other phases' GEMMs on the second stream
    // (ep_comm_sms > 0) or behind the most loaded rank's GEMMs when rows stay on their owners; with balanced loads on one
    // stream a single phase (fewer launches, larger GEMMs).
    const int comm_sms = tuning().ep_comm_sms;
    const long long expected_rows = static_cast<long long>(num_max_tokens_per_rank) * num_ranks * num_topk / num_experts;
    // "fused_dispatch": with balanced loads on one stream, several phases again, and the gate/up GEMM of phase q carries the
    // dispatch rows of phase q + 1 in its epilogue warps (only the tokens-on-M variant of the FP8 x FP4 kind can)
    const bool ride = spill && comm_sms == 0 && tuning().fused_dispatch != 0 && !fused_mlp && V >= 2 &&
                      layer_orientation(quant.kind, V, hidden, intermediate_hidden, expected_rows) == kOrientM;
    const int ride_phases = tuning().fused_dispatch >= 2 ? tuning().fused_dispatch : kMaxEpPhases;
    const int phases = fused_mlp ? 1 : std::min(ride ? ride_phases : ((spill && comm_sms == 0) ? 1 : kMaxEpPhases), V);
    int* chunk_hist = reinterpret_cast<int*>(base + l.chunk_hist);
    int* dest_row = reinterpret_cast<int*>(base + l.dest_row);
    const int* expert_start = reinterpret_cast<const int*>(base + l.expert_start);
    const int* expert_end = reinterpret_cast<const int*>(base + l.expert_end);
    const long long* topk_idx = reinterpret_cast<const long long*>(base + l.topk_idx);
    const float* topk_weights = reinterpret_cast<const float*>(base + l.topk_weights);
    const long long peer_budget = tuning().peer_wait_cycles;
    // On one stream the kernels follow each other with programmatic dependent launch (every one of them starts with
    // pdl_prologue()); on two streams events sit between them and the launches are plain.
    const bool pdl = use_pdl();
    auto flag = [&](int row, int do_signal, int do_wait) {
        launch_kernel(dgb200_ep_flag_kernel, dim3(1), dim3(32), 0, stream, pdl, peers, l.flags, row, rank, num_ranks, do_signal, do_wait,
                      peer_budget);
    };
    auto phase_begin = [&](int q) { return static_cast<int>(static_cast<long long>(q) * V / phases); };
    int rc = 0;
    if ((rc = record_stage(0, stream))) return rc;

    // count this rank's entries per (global) expert and publish the totals to every rank
    launch_kernel(dgb200_moe_count_kernel, dim3(chunks), dim3(kPlanChunk), num_experts * sizeof(int), stream, pdl, topk_idx, entries, 0,
                  num_experts, chunk_hist);
    launch_kernel(dgb200_ep_share_counts_kernel, dim3(1), dim3(1024), 0, stream, pdl, chunk_hist, chunks, num_experts, rank, num_ranks, peers,
                  l.all_counts);
    flag(0, 1, 1);
    // the same global plan on every rank
    if (spill)
        launch_kernel(dgb200_ep_spill_plan_kernel, dim3(1), dim3(1024), static_cast<size_t>(num_ranks) * num_experts * 6, stream, pdl,
            reinterpret_cast<const int*>(base + l.all_counts), num_experts, num_ranks, rank, kSegmentAlignment, G,
            reinterpret_cast<int*>(base + l.my_base), reinterpret_cast<int*>(base + l.my_dest), reinterpret_cast<int*>(base + l.my_slot),
            reinterpret_cast<int*>(base + l.expert_start), reinterpret_cast<int*>(base + l.expert_end),
            reinterpret_cast<int*>(base + l.total_rows), reinterpret_cast<int*>(base + l.guest_expert),
            reinterpret_cast<int*>(base + l.rank_rows), stats);
    else
        launch_kernel(dgb200_ep_plan_kernel, dim3(1), dim3(1024), 0, stream, pdl, reinterpret_cast<const int*>(base + l.all_counts), num_experts, num_ranks, rank,
                                                       kSegmentAlignment, reinterpret_cast<int*>(base + l.my_base),
                                                       reinterpret_cast<int*>(base + l.expert_start),
                                                       reinterpret_cast<int*>(base + l.expert_end),
                                                       reinterpret_cast<int*>(base + l.total_rows), stats);
    if (entries > 0)
        launch_kernel(dgb200_ep_assign_kernel, dim3(chunks), dim3(kPlanChunk), 32 * num_experts, stream, pdl, topk_idx, entries, num_experts,
                      chunk_hist, reinterpret_cast<const int*>(base + l.my_base), dest_row);
    DGB_CUDA(cudaGetLastError());
    if ((rc = record_stage(1, stream))) return rc;

    // dispatch, phase by phase: rows + scales + weight + source id stored straight into the computing ranks' expert-sorted buffers
    if (quant.x_bf16 != nullptr && num_tokens > 0) {
        // BF16 input: quantise once into the buffer's x / x_sf views (the bits of per_token_cast_to_fp8, gran 32), push from there
        rc = run_cast(false, quant.x_bf16, quant.x_bf16_row_stride, num_tokens, hidden, 32, base + l.x, hidden, nullptr, base + l.x_sf, 1,
                      sf_per_row, stream);
        if (rc) return rc;
    }
    // Overlap: with several phases and ep_comm_sms > 0 the kernels that move rows run on a second stream, on SMs the
    // GEMMs leave free: the pushes of later phases under the GEMMs of earlier ones, and the output rows of a finished
    // phase go back to their source ranks (return push) under the GEMMs of the next; the combine is then a local sum.
    // Otherwise everything runs on the caller's stream and the combine pulls the rows phase by phase.
    const bool overlap = phases > 1 && comm_sms > 0;
    int all_sms = 0;
    if ((rc = effective_num_sms(&all_sms))) return rc;
    const long long push_slot_bytes = act_row_bytes(quant.kind, hidden) + ((4 * sf_per_row) % 16 == 0 ? 4ll * sf_per_row : 0);
    DGB_REQUIRE(push_slot_bytes % 16 == 0 && push_slot_bytes <= kRowMoverSmemBudget - 1024 && hidden * 2ll <= kRowMoverSmemBudget - 1024,
                "rows of %lld bytes do not fit the row movers' shared-memory slots", push_slot_bytes);
    if ((rc = allow_row_mover_smem(dgb200_ep_push_kernel))) return rc;
    if ((rc = allow_row_mover_smem(dgb200_ep_return_rows_kernel))) return rc;
    auto push = [&](int q, cudaStream_t on, bool few_sms) {
        if (entries <= 0) return;
        const RowMoverLaunch shape = row_mover_launch(push_slot_bytes, few_sms);
        launch_kernel(dgb200_ep_push_kernel, dim3(few_sms ? comm_sms : all_sms), dim3(shape.warps * 32), shape.smem_bytes, on, pdl && !overlap,
            base + l.x, reinterpret_cast<const unsigned*>(base + l.x_sf), topk_idx, topk_weights, dest_row, entries, num_topk,
            static_cast<int>(act_row_bytes(quant.kind, hidden)), sf_per_row, E, rank, entries_per_rank, peers, l.l1_acts,
            l.l1_sf_stage, l.row_weight, l.src_of_row, phase_begin(q), phase_begin(q + 1), my_dest, my_slot);
    };
    auto fetch_guests = [&](cudaStream_t on) {
        // the weights of the experts this rank hosts as a guest, from their owners
        launch_kernel(dgb200_ep_fetch_guest_weights_kernel, dim3(overlap ? std::max(1, comm_sms / std::max(1, G)) : 74, G), dim3(256), 0, on,
                      pdl && !overlap, reinterpret_cast<const int*>(base + l.guest_expert), E, guest_tables);
    };
    // With balanced loads on one stream the down GEMM sends its output rows to their source ranks from its epilogue
    // ("fused_return" tuning knob, on by default), so the transfer runs under the GEMM's own MMAs tile by tile; where the
    // GEMM variant in use has no such epilogue, or on the second stream, a kernel of its own sends the rows of l2_out.
    ReturnSpec return_spec{};
    return_spec.src_of_row = reinterpret_cast<const int*>(base + l.src_of_row);
    return_spec.entries_per_rank = entries_per_rank;
    for (int r = 0; r < num_ranks; ++r) return_spec.returned_base[r] = peers.p[r] + static_cast<unsigned long long>(l.returned);
    const bool fuse_return_into_gemm = spill && !overlap && tuning().fused_return != 0;
    bool returned_by_gemm = false;
    // the dispatch rows of phase q + 1 that the gate/up GEMM of phase q pushes ("fused_dispatch")
    const long long list_stride = static_cast<long long>(entries_per_rank);
    int* push_lists = reinterpret_cast<int*>(base + l.push_lists);
    int* push_counts = push_lists + kMaxEpPhases * list_stride;
    auto push_work_for = [&](int phase) {
        PushWork w{};
        w.list = push_lists + phase * list_stride;
        w.count = push_counts + phase;
        w.x = base + l.x;
        w.x_sf = reinterpret_cast<const unsigned*>(base + l.x_sf);
        w.topk_weights = topk_weights;
        w.topk_idx = topk_idx;
        w.dest_row = dest_row;
        w.my_dest = my_dest;
        w.experts_per_rank = E;
        w.topk = num_topk;
        w.row_bytes = static_cast<int>(act_row_bytes(quant.kind, hidden));
        w.sf_per_row = sf_per_row;
        w.my_rank = rank;
        w.entries_per_rank = entries_per_rank;
        for (int r = 0; r < num_ranks; ++r) {
            w.acts_base[r] = peers.p[r] + static_cast<unsigned long long>(l.l1_acts);
            w.sf_base[r] = peers.p[r] + static_cast<unsigned long long>(l.l1_sf_stage);
            w.weight_base[r] = peers.p[r] + static_cast<unsigned long long>(l.row_weight);
            w.src_base[r] = peers.p[r] + static_cast<unsigned long long>(l.src_of_row);
        }
        return w;
    };
    auto gemms = [&](int q) -> int {
        const int g0 = phase_begin(q), g1 = phase_begin(q + 1);
        returned_by_gemm = false;
        PushWork next_phase{};
        PushWork* next_phase_dev = nullptr;  // the descriptor as the kernel reads it
        if (ride && q + 1 < phases && entries > 0) {
            next_phase = push_work_for(q + 1);
            next_phase_dev = reinterpret_cast<PushWork*>(push_counts + 16 * kMaxEpPhases) + (q + 1);
            DGB_CUDA(cudaMemcpyAsync(next_phase_dev, &next_phase, sizeof(PushWork), cudaMemcpyHostToDevice, stream));
        }
        if (g1 == g0 && next_phase.list != nullptr) {
            // nothing to compute in this phase on this rank: the rows still have to leave
            push(q + 1, stream, false);
            return 0;
        }
        if (g1 == g0) return 0;
        // the scale ints every rank pushed row by row -> the GEMM's MN-major tcgen05.cp order (local, a few microseconds)
        if (sf_per_row > 0)
            launch_kernel(dgb200_sf_rows_to_cp_order_kernel, dim3(static_cast<int>(l.max_rows / 32)), dim3(256),
                sf_per_row * 33 * sizeof(unsigned), stream, pdl && !overlap,
                reinterpret_cast<const unsigned*>(base + l.l1_sf_stage), static_cast<int>(l.max_rows), sf_per_row,
                reinterpret_cast<unsigned*>(base + l.l1_sf), l.max_rows, reinterpret_cast<const int*>(base + l.total_rows),
                expert_start + g0, expert_end + g1 - 1);
        DGB_CUDA(cudaGetLastError());
        return run_layer_gemms(quant, l, base, l1_w, l1_w_sf, l2_w, l2_w_sf, hidden, intermediate_hidden, activation_clamp, fast_math, stream,
                               kNumStageEvents /* no stage events inside the loop */, expected_rows,
                               phases == 1 ? 0 : g0, phases == 1 ? 0 : g1, fuse_return_into_gemm ? &return_spec : nullptr,
                               &returned_by_gemm, next_phase_dev);
    };

    // the BF16 output rows of phase q's expert slots back to the ranks their tokens came from
    auto return_rows = [&](int q, cudaStream_t on, bool few_sms) {
        const int g0 = phase_begin(q), g1 = phase_begin(q + 1);
        if (g1 == g0) return;
        const RowMoverLaunch shape = row_mover_launch(hidden * 2ll, few_sms);
        launch_kernel(dgb200_ep_return_rows_kernel, dim3(few_sms ? comm_sms : all_sms), dim3(shape.warps * 32), shape.smem_bytes, on,
            pdl && !overlap, reinterpret_cast<const __nv_bfloat16*>(base + l.l2_out), reinterpret_cast<const int*>(base + l.src_of_row), expert_start,
            expert_end, g0, g1, hidden, entries_per_rank, peers, l.returned);
    };
    // once every rank's rows of every phase have arrived: a local sum per token, in slot order
    auto combine = [&]() {
        if (num_tokens > 0)
            launch_kernel(dgb200_moe_combine_returned_kernel, dim3(num_tokens), dim3(128), 0, stream, pdl && !overlap,
                reinterpret_cast<const __nv_bfloat16*>(base + l.returned), dest_row, num_topk, hidden,
                with_shared ? reinterpret_cast<const __nv_bfloat16*>(base + l.shared_out) : nullptr, static_cast<__nv_bfloat16*>(y));
    };

    if (!overlap) {
        if (ride && entries > 0) {
            DGB_CUDA(cudaMemsetAsync(push_counts, 0, kMaxEpPhases * sizeof(int), stream));
            launch_kernel(dgb200_ep_phase_lists_kernel, dim3((entries + 255) / 256), dim3(256), 0, stream, false, topk_idx, dest_row, entries, E,
                          my_slot, phases, V, push_lists, static_cast<int>(list_stride), push_counts);
        }
        for (int q = 0; q < (ride ? 1 : phases); ++q) {
            push(q, stream, false);
            flag(1 + q, 1, 0);
        }
        DGB_CUDA(cudaGetLastError());
        if (spill) fetch_guests(stream);
        DGB_CUDA(cudaGetLastError());
        if ((rc = record_stage(2, stream))) return rc;
        // GEMMs, phase by phase, each as soon as every rank's rows for the phase have landed. How the output rows get back
        // to the tokens' ranks depends on who has time: with balanced loads (spill) the computing rank pushes them right
        // away and the combine is a local sum; when rows stay on their owners the most loaded rank is the critical path
        // and the others idle, so those pull the rows of each finished phase themselves (phased combine).
        for (int q = 0; q < phases; ++q) {
            flag(1 + q, 0, 1);
            if ((rc = gemms(q))) return rc;
            if (ride && q + 1 < phases) flag(1 + q + 1, 1, 0);  // the next phase's rows left with this phase's gate/up GEMM
            if (spill && !returned_by_gemm) return_rows(q, stream, false);
            flag(1 + kMaxEpPhases + q, 1, 0);
        }
        if ((rc = record_stage(3, stream))) return rc;  // both GEMMs of all phases lie before this point
        if ((rc = record_stage(4, stream))) return rc;
        if (with_shared && num_tokens > 0) {
            if (quant.kind != kKindBf16 && (rc = run_shared_x_sf(l, base, num_tokens, hidden, stream))) return rc;
            if ((rc = run_shared_gemms(quant, l, base, num_tokens, hidden, activation_clamp, fast_math, stream))) return rc;
        }
        for (int q = 0; q < phases; ++q) {
            flag(1 + kMaxEpPhases + q, 0, 1);
            if (!spill && num_tokens > 0)
                launch_kernel(dgb200_moe_combine_phase_kernel, dim3(num_tokens), dim3(128), num_topk * sizeof(unsigned long long), stream, pdl,
                    peers, l.l2_out, topk_idx, dest_row, num_topk, E, hidden,
                    with_shared ? reinterpret_cast<const __nv_bfloat16*>(base + l.shared_out) : nullptr,
                    reinterpret_cast<float*>(base + l.combine_partial), static_cast<__nv_bfloat16*>(y), phase_begin(q), phase_begin(q + 1),
                    q == 0 ? 1 : 0, q == phases - 1 ? 1 : 0, my_dest, my_slot);
        }
        if (spill) combine();
        DGB_CUDA(cudaGetLastError());
        return record_stage(5, stream);
    }

    EpStreams* ep = nullptr;
    if ((rc = ep_streams_for_current_device(&ep))) return rc;
    std::lock_guard<std::mutex> ep_lock(ep->mu);
    cudaStream_t comm = ep->comm;
    auto flag_on = [&](cudaStream_t on, int row, int do_signal, int do_wait) {
        dgb200_ep_flag_kernel<<<1, 32, 0, on>>>(peers, l.flags, row, rank, num_ranks, do_signal, do_wait, peer_budget);
    };
    // second stream: every push (the first on all SMs: nothing else runs yet), the guest weights, then the return pushes
    DGB_CUDA(cudaEventRecord(ep->planned, stream));
    DGB_CUDA(cudaStreamWaitEvent(comm, ep->planned, 0));
    for (int q = 0; q < phases; ++q) {
        push(q, comm, q > 0);
        flag_on(comm, 1 + q, 1, 0);
        DGB_CUDA(cudaEventRecord(ep->pushed[q], comm));
    }
    if (spill) fetch_guests(comm);
    DGB_CUDA(cudaGetLastError());
    DGB_CUDA(cudaEventRecord(ep->fetched, comm));
    // caller's stream: the GEMMs of phase q as soon as every rank's rows for it have landed, on all SMs but comm_sms
    int rc_gemm = 0;
    for (int q = 0; q < phases && rc_gemm == 0; ++q) {
        DGB_CUDA(cudaStreamWaitEvent(stream, ep->pushed[q], 0));
        flag_on(stream, 1 + q, 0, 1);
        if (q == 0 && (rc = record_stage(2, stream))) rc_gemm = rc;  // the rows of the first phase are here
        if (phase_begin(q + 1) > E) DGB_CUDA(cudaStreamWaitEvent(stream, ep->fetched, 0));  // guest slots: their weights are here
        reserved_sms() = comm_sms;
        if (rc_gemm == 0) rc_gemm = gemms(q);
        reserved_sms() = 0;
        DGB_CUDA(cudaEventRecord(ep->computed[q], stream));
        // second stream: this phase's output rows back to their source ranks, then "outputs q" to every rank
        DGB_CUDA(cudaStreamWaitEvent(comm, ep->computed[q], 0));
        return_rows(q, comm, q < phases - 1);  // nothing runs next to the last one: all SMs
        flag_on(comm, 1 + kMaxEpPhases + q, 1, 0);
    }
    DGB_CUDA(cudaGetLastError());
    // join: the second stream never runs ahead of the caller's stream, whatever happened above
    DGB_CUDA(cudaEventRecord(ep->returned, comm));
    if ((rc = record_stage(3, stream))) return rc;  // both GEMMs of all phases lie before this point
    if ((rc = record_stage(4, stream))) return rc;
    if (rc_gemm == 0 && with_shared && num_tokens > 0) {
        if (quant.kind != kKindBf16) rc_gemm = run_shared_x_sf(l, base, num_tokens, hidden, stream);
        if (rc_gemm == 0) rc_gemm = run_shared_gemms(quant, l, base, num_tokens, hidden, activation_clamp, fast_math, stream);
    }
    DGB_CUDA(cudaStreamWaitEvent(stream, ep->returned, 0));
    if (rc_gemm) return rc_gemm;
    for (int q = 0; q < phases; ++q) flag_on(stream, 1 + kMaxEpPhases + q, 0, 1);
    combine();
    DGB_CUDA(cudaGetLastError());
    return record_stage(5, stream);
}


// The whole layer on this rank (single rank: plan, gather, two GEMMs, combine; several ranks: run_mega_moe_ep).
int run_mega_moe(const LayerQuant& quant, void* y, const void* l1_w, const void* l1_w_sf, const void* l2_w, const void* l2_w_sf,
                 int32_t* cumulative_local_expert_recv_stats, void* buffer, const uint64_t* peer_buffer_ptrs,
                 int32_t rank, int32_t num_ranks, int32_t num_tokens, int32_t num_max_tokens_per_rank,
                 int32_t num_experts, int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                 float activation_clamp, int32_t fast_math, cudaStream_t stream) {
    MegaLayout l;
    int rc = make_mega_layout(quant.kind, num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden, &l,
                              quant.shared_inter);
    if (rc) return rc;
    const bool with_shared = quant.shared_inter > 0;
    DGB_REQUIRE(!with_shared || (quant.shared_l1_w != nullptr && quant.shared_l2_w != nullptr &&
                                 (quant.kind == kKindBf16 || (quant.shared_l1_w_sf != nullptr && quant.shared_l2_w_sf != nullptr))),
                "null shared-expert weight pointer");
    DGB_REQUIRE(rank >= 0 && rank < num_ranks && peer_buffer_ptrs != nullptr &&
                    peer_buffer_ptrs[rank] == reinterpret_cast<uint64_t>(buffer),
                "rank / peer pointer table do not describe this buffer");
    DGB_REQUIRE(num_tokens >= 0 && num_tokens <= num_max_tokens_per_rank, "num_tokens (%d) exceeds the buffer capacity (%d)",
                num_tokens, num_max_tokens_per_rank);
    DGB_REQUIRE(y != nullptr && l1_w != nullptr && l2_w != nullptr && buffer != nullptr &&
                    (quant.kind == kKindBf16 || (l1_w_sf != nullptr && l2_w_sf != nullptr)),
                "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(buffer) % 256 == 0, "buffer must be 256-byte aligned");
    DGB_REQUIRE((2 * intermediate_hidden) % 128 == 0 && intermediate_hidden % 64 == 0, "intermediate_hidden must be a multiple of 64");
    if (num_tokens == 0 && num_ranks == 1) return 0;

    uint8_t* base = static_cast<uint8_t*>(buffer);
    const int E = l.num_local_experts;
    const int entries = num_tokens * num_topk;
    const int chunks = (entries + kPlanChunk - 1) / kPlanChunk;
    int* chunk_hist = reinterpret_cast<int*>(base + l.chunk_hist);
    int* expert_start = reinterpret_cast<int*>(base + l.expert_start);
    int* expert_end = reinterpret_cast<int*>(base + l.expert_end);
    int* total_rows = reinterpret_cast<int*>(base + l.total_rows);
    int* dest_row = reinterpret_cast<int*>(base + l.dest_row);
    int* src_of_row = reinterpret_cast<int*>(base + l.src_of_row);
    float* row_weight = reinterpret_cast<float*>(base + l.row_weight);
    const long long* topk_idx = reinterpret_cast<const long long*>(base + l.topk_idx);
    const float* topk_weights = reinterpret_cast<const float*>(base + l.topk_weights);

    struct ClearEvents { ~ClearEvents() { g_num_stage_events = 0; } } clear_events_on_exit;
    if ((rc = record_stage(0, stream))) return rc;
    if (num_ranks > 1)
        return run_mega_moe_ep(quant, l, y, l1_w, l1_w_sf, l2_w, l2_w_sf, cumulative_local_expert_recv_stats, base, peer_buffer_ptrs, rank,
                               num_ranks, num_tokens, num_max_tokens_per_rank, num_experts, num_topk, hidden,
                               intermediate_hidden, activation_clamp, fast_math, stream);

    // 1. dispatch plan: stable counting sort of the (token, k) entries by expert
    DGB_CUDA(cudaMemsetAsync(src_of_row, 0xff, l.max_rows * 4, stream));
    const bool pdl = use_pdl();
    DGB_CUDA(launch_kernel(dgb200_moe_count_kernel, dim3(chunks), dim3(kPlanChunk), E * sizeof(int), stream, pdl, topk_idx, entries, 0, E,
                           chunk_hist));
    DGB_CUDA(launch_kernel(dgb200_moe_scan_kernel, dim3(1), dim3(1024), 0, stream, pdl, chunk_hist, chunks, E, kSegmentAlignment,
                           expert_start, expert_end, total_rows, cumulative_local_expert_recv_stats));
    DGB_CUDA(launch_kernel(dgb200_moe_assign_kernel, dim3(chunks), dim3(kPlanChunk), 32 * E, stream, pdl, topk_idx, topk_weights, entries, 0,
                           E, chunk_hist, expert_start, dest_row, src_of_row, row_weight));

    if ((rc = record_stage(1, stream))) return rc;
    // 2. gather quantised rows + scales into expert-sorted order
    const long long upper_rows = std::min<long long>(l.max_rows, static_cast<long long>(entries) + static_cast<long long>(E) * kSegmentAlignment);
    const int gather_blocks = static_cast<int>((upper_rows + 31) / 32);
    const int sf_per_row = sf_ints_per_row(quant.kind, hidden);
    if (quant.x_bf16 != nullptr && quant.kind == kKindNvfp4) {
        DGB_CUDA(launch_kernel(dgb200_moe_quant_dispatch_nvfp4_kernel, dim3((num_tokens + 7) / 8), dim3(256), 0, stream, pdl, quant.x_bf16,
                               quant.x_bf16_row_stride, quant.x_scale, dest_row, num_tokens, num_topk, hidden, base + l.l1_acts,
                               reinterpret_cast<unsigned*>(base + l.l1_sf), l.max_rows));
    } else if (quant.x_bf16 != nullptr) {
        PeerTable self_table{};
        for (int r = 0; r < kMaxEpRanks; ++r) self_table.p[r] = reinterpret_cast<unsigned long long>(base);
        DGB_CUDA(launch_kernel(dgb200_moe_quant_dispatch_kernel, dim3((num_tokens + 7) / 8), dim3(256), 0, stream, pdl, quant.x_bf16,
                               quant.x_bf16_row_stride, topk_idx, topk_weights, dest_row, num_tokens, num_topk, hidden, num_experts, 0, entries,
                               self_table, l.l1_acts, l.l1_sf, l.max_rows, l.row_weight, l.src_of_row, 0,
                               with_shared ? base + l.x : nullptr, with_shared ? reinterpret_cast<unsigned*>(base + l.shared_x_sf) : nullptr,
                               l.token_rows));
    } else {
        DGB_CUDA(launch_kernel(dgb200_moe_gather_kernel, dim3(gather_blocks), dim3(256), sf_per_row * 33 * sizeof(unsigned), stream, pdl,
                               base + l.x, reinterpret_cast<const unsigned*>(base + l.x_sf), src_of_row, total_rows, num_topk,
                               static_cast<int>(act_row_bytes(quant.kind, hidden)), sf_per_row, base + l.l1_acts,
                               reinterpret_cast<unsigned*>(base + l.l1_sf), l.max_rows));
    }

    if ((rc = record_stage(2, stream))) return rc;
    // 3 + 4. L1 (gate/up GEMM, fused SwiGLU + FP8 requant) and L2 (down GEMM, rows scattered to their combine slots)
    rc = run_layer_gemms(quant, l, base, l1_w, l1_w_sf, l2_w, l2_w_sf, hidden, intermediate_hidden, activation_clamp, fast_math, stream, 3,
                         static_cast<long long>(num_tokens) * num_topk / num_experts);
    if (rc) return rc;
    if (with_shared) {
        if (quant.x_bf16 == nullptr && quant.kind != kKindBf16 && (rc = run_shared_x_sf(l, base, num_tokens, hidden, stream))) return rc;
        if ((rc = run_shared_gemms(quant, l, base, num_tokens, hidden, activation_clamp, fast_math, stream))) return rc;
    }
    // 5. combine: y[t] = sum over the top-k slots of the rows the L2 GEMM wrote
    PeerTable self{};
    self.p[0] = reinterpret_cast<unsigned long long>(base);
    DGB_CUDA(launch_kernel(dgb200_moe_combine_kernel, dim3(num_tokens), dim3(128), (num_topk + 1) * sizeof(unsigned long long), stream, pdl,
                           self, l.l2_out, topk_idx, dest_row, num_topk, E, hidden,
                           with_shared ? reinterpret_cast<const __nv_bfloat16*>(base + l.shared_out) : nullptr,
                           static_cast<__nv_bfloat16*>(y)));
    return record_stage(5, stream);
}

// Byte offsets of the buffer regions, in the order the C header documents.
int export_mega_layout(int kind, int num_ranks, int num_experts, int max_tokens, int topk, int hidden, int inter, int64_t* out) {
    DGB_REQUIRE(out != nullptr, "null output");
    MegaLayout l;
    const int rc = make_mega_layout(kind, num_ranks, num_experts, max_tokens, topk, hidden, inter, &l);
    if (rc) return rc;
    const long long fields[16] = {l.total, l.x, l.x_sf, l.topk_idx, l.topk_weights, l.l1_acts, l.l1_sf, l.l2_acts, l.l2_sf,
                                  l.max_rows, l.dest_row, l.src_of_row, l.expert_start, l.expert_end, l.l2_out, l.row_weight};
    for (int i = 0; i < 16; ++i) out[i] = fields[i];
    return 0;
}

// --------------------------------------------------------------------------------------------------------------
// Scratch of the allocation-free dispatch-plan entry point: per-chunk expert histograms (the same role the
// caller-provided buffer plays for the layer call) plus one word for the row total. File-scope device memory, so
// every GPU that loads the library holds these ~129 KB until the process exits.
// --------------------------------------------------------------------------------------------------------------
constexpr int kNoAllocMaxEntries = 65536;  // num_tokens * num_topk
constexpr int kNoAllocMaxExperts = 512;
constexpr int kNoAllocScratchInts = (kNoAllocMaxEntries / kPlanChunk) * kNoAllocMaxExperts + 64;
static __device__ __align__(256) int g_noalloc_plan_scratch[kNoAllocScratchInts];

// Device address of the scratch array on the current device, looked up once per device. In host code the array's
// name is only a handle for the runtime; cudaGetSymbolAddress turns it into the address a kernel can use.
int noalloc_scratch_for_current_device(int** out) {
    constexpr int kMaxDevices = 64;
    static int* cached[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    DGB_CUDA(cudaGetDevice(&dev));
    DGB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        int* ptr = nullptr;
        DGB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_plan_scratch));
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return 0;
}

}  // namespace
}  // namespace dgb

using namespace dgb;

extern "C" {

const char* dgb200_last_error(void) { return last_error_storage().c_str(); }

int dgb200_version(void) { return kVersion; }

int dgb200_set_num_sms(int num_sms) {
    DGB_REQUIRE(num_sms >= 0, "num_sms must be >= 0");
    num_sms_setting() = num_sms;
    return 0;
}

int dgb200_set_tuning(const char* name, int32_t value) {
    DGB_REQUIRE(name != nullptr, "null name");
    if (std::strcmp(name, "swap_ab") == 0) {
        DGB_REQUIRE(value >= -1 && value <= 2, "swap_ab must be -1 (automatic), 0, 1 or 2");
        tuning().swap_ab = value;
    } else if (std::strcmp(name, "block_n") == 0) {
        DGB_REQUIRE(value == 0 || value == 128 || value == 256, "block_n must be 0 (automatic), 128 or 256");
        tuning().block_n = value;
    } else if (std::strcmp(name, "fused_dispatch") == 0) {
        DGB_REQUIRE(value >= 0 && value <= kMaxEpPhases, "fused_dispatch must be 0 (off), 1 (on, %d phases) or a phase count up to %d", kMaxEpPhases, kMaxEpPhases);
        tuning().fused_dispatch = value;
    } else if (std::strcmp(name, "fused_return") == 0) {
        DGB_REQUIRE(value == 0 || value == 1, "fused_return must be 0 or 1");
        tuning().fused_return = value;
    } else if (std::strcmp(name, "pdl") == 0) {
        DGB_REQUIRE(value == 0 || value == 1, "pdl must be 0 or 1");
        tuning().pdl = value;
    } else if (std::strcmp(name, "ep_comm_sms") == 0) {
        DGB_REQUIRE(value >= 0 && value <= 64, "ep_comm_sms must be in [0, 64]");
        tuning().ep_comm_sms = value;
    } else if (std::strcmp(name, "peer_wait_us") == 0) {
        DGB_REQUIRE(value >= 1, "peer_wait_us must be at least 1 microsecond");
        tuning().peer_wait_cycles = static_cast<long long>(value) * 2000;  // SM clock below 2 GHz: at least `value` us
    } else {
        return fail(DGB200_EINVAL, "unknown tuning knob '%s'", name);
    }
    return 0;
}


int dgb200_get_num_sms(void) {
    int sms = 0;
    if (effective_num_sms(&sms) != 0) return -1;
    return sms;
}

int dgb200_device_status(int32_t* out_words, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    DGB_CUDA(cudaStreamSynchronize(s));
    int words[8];
    DGB_CUDA(cudaMemcpyFromSymbol(words, g_status, sizeof(words)));
    if (out_words != nullptr) std::memcpy(out_words, words, sizeof(words));
    if (words[0] != 0) {
        const int zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        DGB_CUDA(cudaMemcpyToSymbol(g_status, zeros, sizeof(zeros)));
        return fail(DGB200_EDEVICE, "device status: code %d at block %d (detail %d, %d)", words[0], words[1], words[2],
                    words[3]);
    }
    return 0;
}

namespace {
int run_m_grouped_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride,
    const void* b, int b_mn_major, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, int32_t store_padding, void* stream) {
    DGB_REQUIRE(m >= 0, "m must be >= 0");
    DGB_REQUIRE(layout_kind == DGB200_LAYOUT_ROW_IDS || layout_kind == DGB200_LAYOUT_PSUM, "unknown layout kind %d",
                layout_kind);
    DGB_REQUIRE(alignment > 0 && alignment % 4 == 0, "alignment (%d) must be a positive multiple of 4", alignment);
    DGB_REQUIRE(layout_kind == DGB200_LAYOUT_PSUM || alignment % 128 == 0,
                "the row-id layout needs an M alignment that is a multiple of 128, got %d", alignment);
    DGB_REQUIRE(d != nullptr || m == 0, "null output");
    DGB_REQUIRE(d_row_stride >= n && (d_row_stride * (d_is_fp32 ? 4 : 2)) % 16 == 0,
                "d row stride must cover n and keep rows 16-byte aligned");
    DGB_REQUIRE(sfa_k_stride >= m, "sfa MN stride (%lld) smaller than m (%d)", static_cast<long long>(sfa_k_stride), m);
    GemmCall c{};
    c.a = a;
    c.b = b;
    c.b_mn_major = b_mn_major;
    c.a_rows_total = m;
    c.b_is_fp4 = b_is_fp4;
    c.epilogue = d_is_fp32 ? kEpiF32 : kEpiBF16;
    GemmParams& p = c.p;
    c.sfa = sfa;
    c.sfb = sfb;
    c.sfa_k_stride = sfa_k_stride;
    c.sfa_group_stride = 0;
    c.num_groups_a = 1;
    c.sfb_k_stride = sfb_k_stride;
    c.sfb_group_stride = sfb_group_stride;
    p.d = d;
    p.d_row_stride = d_row_stride;
    p.layout = grouped_layout;
    p.mode = layout_kind == DGB200_LAYOUT_PSUM ? kModePsum : kModeRowIds;
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_groups = num_groups;
    p.alignment = alignment;
    p.gran_a = gran_k_a;
    p.gran_b = gran_k_b;
    p.store_padding = store_padding;
    const long long m_blocks = (static_cast<long long>(m) + 127) / 128 + (p.mode == kModePsum ? num_groups : 0);
    c.max_tiles = static_cast<int>(std::min<long long>(m_blocks * (n / 128 > 0 ? n / 128 : 1), 1 << 30));
    return run_gemm(c, static_cast<cudaStream_t>(stream));
}
}  // namespace

int dgb200_m_grouped_fp8_fp4_gemm_nt_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, int32_t store_padding, void* stream) {
    return run_m_grouped_contiguous(a, sfa, sfa_k_stride, b, 0, sfb, sfb_k_stride, sfb_group_stride, d, d_row_stride, grouped_layout,
                                    m, n, k, num_groups, gran_k_a, gran_k_b, b_is_fp4, d_is_fp32, layout_kind, alignment,
                                    store_padding, stream);
}

int dgb200_m_grouped_fp8_fp4_gemm_nn_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, int32_t store_padding, void* stream) {
    DGB_REQUIRE(n % 32 == 0, "an MN-major b needs n (%d) to be a multiple of 32", n);
    return run_m_grouped_contiguous(a, sfa, sfa_k_stride, b, 1, sfb, sfb_k_stride, sfb_group_stride, d, d_row_stride, grouped_layout,
                                    m, n, k, num_groups, gran_k_a, gran_k_b, b_is_fp4, d_is_fp32, layout_kind, alignment,
                                    store_padding, stream);
}

int dgb200_fp8_fp4_gemm_nt(const void* a, const void* sfa, int64_t sfa_k_stride, const void* b, const void* sfb,
                           int64_t sfb_k_stride, void* d, int64_t d_row_stride, int32_t m, int32_t n, int32_t k,
                           int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32, int32_t accumulate,
                           void* stream) {
    DGB_REQUIRE(m >= 0, "m must be >= 0");
    DGB_REQUIRE(!accumulate || d_is_fp32, "accumulation needs a float32 d");
    DGB_REQUIRE(d != nullptr || m == 0, "null output");
    DGB_REQUIRE(d_row_stride >= n && (d_row_stride * (d_is_fp32 ? 4 : 2)) % 16 == 0,
                "d row stride must cover n and keep rows 16-byte aligned");
    DGB_REQUIRE(sfa_k_stride >= m, "sfa MN stride (%lld) smaller than m (%d)", static_cast<long long>(sfa_k_stride), m);
    GemmCall c{};
    c.a = a;
    c.b = b;
    c.a_rows_total = m;
    c.b_is_fp4 = b_is_fp4;
    c.epilogue = d_is_fp32 ? kEpiF32 : kEpiBF16;
    c.sfa = sfa;
    c.sfb = sfb;
    c.sfa_k_stride = sfa_k_stride;
    c.num_groups_a = 1;
    c.sfb_k_stride = sfb_k_stride;
    GemmParams& p = c.p;
    p.d = d;
    p.d_row_stride = d_row_stride;
    p.mode = kModeDense;
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_groups = 1;
    p.alignment = 128;
    p.gran_a = gran_k_a;
    p.gran_b = gran_k_b;
    p.accumulate = accumulate ? 1 : 0;
    const long long m_blocks = (static_cast<long long>(m) + 127) / 128;
    c.max_tiles = static_cast<int>(std::min<long long>(m_blocks * (n / 128 > 0 ? n / 128 : 1), 1 << 30));
    return run_gemm(c, static_cast<cudaStream_t>(stream));
}

int dgb200_m_grouped_fp8_fp4_gemm_nt_masked(
    const void* a, const void* sfa, int64_t sfa_k_stride, int64_t sfa_group_stride,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride,
    void* d, int64_t d_row_stride, const int32_t* masked_m,
    int32_t num_groups, int32_t max_m, int32_t n, int32_t k, int32_t expected_m,
    int32_t gran_k_a, int32_t gran_k_b, int32_t b_is_fp4, int32_t d_is_fp32, void* stream) {
    (void)expected_m;
    DGB_REQUIRE(max_m > 0 && max_m % 4 == 0, "max_m (%d) must be a positive multiple of 4", max_m);
    DGB_REQUIRE(d != nullptr, "null output");
    DGB_REQUIRE(d_row_stride >= n && (d_row_stride * (d_is_fp32 ? 4 : 2)) % 16 == 0,
                "d row stride must cover n and keep rows 16-byte aligned");
    DGB_REQUIRE(sfa_k_stride >= max_m, "sfa MN stride smaller than max_m");
    GemmCall c{};
    c.a = a;
    c.b = b;
    c.a_rows_total = static_cast<long long>(num_groups) * max_m;
    c.b_is_fp4 = b_is_fp4;
    c.epilogue = d_is_fp32 ? kEpiF32 : kEpiBF16;
    GemmParams& p = c.p;
    c.sfa = sfa;
    c.sfb = sfb;
    c.sfa_k_stride = sfa_k_stride;
    c.sfa_group_stride = sfa_group_stride;
    c.num_groups_a = num_groups;
    c.sfb_k_stride = sfb_k_stride;
    c.sfb_group_stride = sfb_group_stride;
    p.d = d;
    p.d_row_stride = d_row_stride;
    p.layout = masked_m;
    p.mode = kModeMasked;
    p.m = max_m;
    p.n = n;
    p.k = k;
    p.num_groups = num_groups;
    p.alignment = 4;
    p.gran_a = gran_k_a;
    p.gran_b = gran_k_b;
    p.store_padding = 0;
    c.max_tiles = 0;
    return run_gemm(c, static_cast<cudaStream_t>(stream));
}

namespace {
// Shared body of the BF16 GEMM entry points: A [rows, k] and B [num_groups * n, k] BF16 K-major, D BF16 or FP32.
int run_bf16_gemm(const void* a, int64_t a_row_stride, int32_t a_mn_major, const void* b, int64_t b_row_stride, int32_t b_mn_major, void* d,
                  int64_t d_row_stride, int32_t d_is_fp32, int32_t accumulate, const int32_t* layout, int mode, long long a_rows_total, int32_t m, int32_t n, int32_t k,
                  int32_t num_groups, int32_t alignment, int32_t store_padding, int max_tiles, void* stream) {
    DGB_REQUIRE(d != nullptr || a_rows_total == 0, "null output");
    DGB_REQUIRE(d_row_stride >= n && (d_row_stride * (d_is_fp32 ? 4 : 2)) % 16 == 0,
                "d row stride must cover n and keep rows 16-byte aligned");
    DGB_REQUIRE(a_row_stride >= (a_mn_major ? m : k) && a_row_stride % 8 == 0 && b_row_stride >= (b_mn_major ? n : k) && b_row_stride % 8 == 0,
                "a and b row strides must cover their rows and keep them 16-byte aligned");
    GemmCall c{};
    c.kind = kKindBf16;
    c.a = a;
    c.b = b;
    c.a_rows_total = a_rows_total;
    c.a_row_stride_bytes = a_row_stride * 2;
    c.b_row_stride_bytes = b_row_stride * 2;
    c.b_mn_major = b_mn_major ? 1 : 0;
    c.a_mn_major = a_mn_major ? 1 : 0;
    c.num_groups_a = 1;
    c.epilogue = d_is_fp32 ? kEpiF32 : kEpiBF16;
    GemmParams& p = c.p;
    p.d = d;
    p.d_row_stride = d_row_stride;
    p.layout = layout;
    p.mode = mode;
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_groups = num_groups;
    p.alignment = alignment;
    p.store_padding = store_padding;
    p.accumulate = accumulate ? 1 : 0;
    DGB_REQUIRE(!accumulate || d_is_fp32, "accumulation needs a float32 d");
    c.max_tiles = max_tiles;
    return run_gemm(c, static_cast<cudaStream_t>(stream));
}
}  // namespace

int dgb200_m_grouped_bf16_gemm_nt_contiguous(const void* a, int64_t a_row_stride, const void* b, int64_t b_row_stride,
                                             int32_t b_mn_major, void* d, int64_t d_row_stride, const int32_t* grouped_layout, int32_t m, int32_t n,
                                             int32_t k, int32_t num_groups, int32_t d_is_fp32, int32_t layout_kind,
                                             int32_t alignment, int32_t store_padding, void* stream) {
    DGB_REQUIRE(m >= 0, "m must be >= 0");
    DGB_REQUIRE(layout_kind == DGB200_LAYOUT_ROW_IDS || layout_kind == DGB200_LAYOUT_PSUM, "unknown layout kind %d",
                layout_kind);
    DGB_REQUIRE(alignment > 0 && alignment % 4 == 0, "alignment (%d) must be a positive multiple of 4", alignment);
    DGB_REQUIRE(layout_kind == DGB200_LAYOUT_PSUM || alignment % 128 == 0,
                "the row-id layout needs an M alignment that is a multiple of 128, got %d", alignment);
    const int mode = layout_kind == DGB200_LAYOUT_PSUM ? kModePsum : kModeRowIds;
    const long long m_blocks = (static_cast<long long>(m) + 127) / 128 + (mode == kModePsum ? num_groups : 0);
    const int max_tiles = static_cast<int>(std::min<long long>(m_blocks * (n / 128 > 0 ? n / 128 : 1), 1 << 30));
    return run_bf16_gemm(a, a_row_stride, 0, b, b_row_stride, b_mn_major, d, d_row_stride, d_is_fp32, 0, grouped_layout, mode, m, m, n, k,
                         num_groups, alignment, store_padding, max_tiles, stream);
}

int dgb200_m_grouped_bf16_gemm_nt_masked(const void* a, const void* b, void* d, int64_t d_row_stride, const int32_t* masked_m,
                                         int32_t num_groups, int32_t max_m, int32_t n, int32_t k, int32_t expected_m,
                                         int32_t d_is_fp32, void* stream) {
    (void)expected_m;
    DGB_REQUIRE(max_m > 0 && max_m % 4 == 0, "max_m (%d) must be a positive multiple of 4", max_m);
    return run_bf16_gemm(a, k, 0, b, k, 0, d, d_row_stride, d_is_fp32, 0, masked_m, kModeMasked,
                         static_cast<long long>(num_groups) * max_m, max_m, n, k, num_groups, 4, 0, 0, stream);
}

int dgb200_bf16_gemm_nt(const void* a, int64_t a_row_stride, int32_t a_mn_major, const void* b, int64_t b_row_stride,
                        int32_t b_mn_major, void* d, int64_t d_row_stride, int32_t m, int32_t n, int32_t k, int32_t d_is_fp32,
                        int32_t accumulate, void* stream) {
    DGB_REQUIRE(m >= 0, "m must be >= 0");
    const long long m_blocks = (static_cast<long long>(m) + 127) / 128;
    const int max_tiles = static_cast<int>(std::min<long long>(m_blocks * (n / 128 > 0 ? n / 128 : 1), 1 << 30));
    DGB_REQUIRE(!a_mn_major || m % 8 == 0, "an MN-major a needs m (%d) to be a multiple of 8", m);
    return run_bf16_gemm(a, a_row_stride, a_mn_major, b, b_row_stride, b_mn_major, d, d_row_stride, d_is_fp32, accumulate, nullptr,
                         kModeDense, m, m, n, k, 1, 128,
                         0, max_tiles, stream);
}

int dgb200_per_token_cast_to_fp8(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, int32_t gran_k, void* q,
                                 int64_t q_row_stride, float* sf_f32, void* sf_packed, int64_t sf_k_stride,
                                 int64_t sf_row_stride, void* stream) {
    return run_cast(false, x, x_row_stride, rows, k, gran_k, q, q_row_stride, sf_f32, sf_packed, sf_k_stride, sf_row_stride,
                    static_cast<cudaStream_t>(stream));
}

int dgb200_per_token_cast_to_fp4(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, int32_t gran_k, void* q,
                                 int64_t q_row_stride, float* sf_f32, void* sf_packed, int64_t sf_k_stride,
                                 int64_t sf_row_stride, void* stream) {
    return run_cast(true, x, x_row_stride, rows, k, gran_k, q, q_row_stride, sf_f32, sf_packed, sf_k_stride, sf_row_stride,
                    static_cast<cudaStream_t>(stream));
}

int dgb200_transform_sf_into_required_layout(const float* sf, int64_t stride_g, int64_t stride_mn, int64_t stride_k,
                                             void* out, int32_t num_groups, int32_t mn, int32_t sf_k, int32_t gran_mn,
                                             const int32_t* psum_layout, int32_t num_psum_groups,
                                             int32_t psum_alignment, void* stream) {
    DGB_REQUIRE(sf != nullptr && out != nullptr, "null tensor pointer");
    DGB_REQUIRE(num_groups > 0 && mn >= 0 && sf_k > 0 && gran_mn > 0, "bad scale-factor shape");
    DGB_REQUIRE(psum_layout == nullptr || (num_psum_groups > 0 && psum_alignment > 0), "bad psum layout");
    if (mn == 0) return 0;
    PackSfParams p{};
    p.sf = sf;
    p.in_stride_g = stride_g;
    p.in_stride_mn = stride_mn;
    p.in_stride_k = stride_k;
    p.out = static_cast<uint32_t*>(out);
    p.aligned_mn = (static_cast<long long>(mn) + 3) / 4 * 4;
    p.num_groups = num_groups;
    p.mn = mn;
    p.sf_k = sf_k;
    p.gran_mn = gran_mn;
    p.psum_layout = psum_layout;
    p.num_psum_groups = num_psum_groups;
    p.psum_alignment = psum_alignment;
    const long long total = static_cast<long long>(num_groups) * ((sf_k + 3) / 4) * mn;
    const int grid = static_cast<int>(std::min<long long>((total + 255) / 256, 148 * 16));
    dgb200_pack_sf_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

namespace {
// The K-grouped epilogue adds its accumulators into d (TMA reductions for whole tiles, row by row for the tail of m), so d
// must hold c before the kernel starts; the kernel then reads and writes d only.
int prepare_k_grouped_output(CUtensorMap* tm_out, GemmParams& p, const float* c, float* d, int num_groups, int m, int n,
                             cudaStream_t stream) {
    if (c != d)
        DGB_CUDA(cudaMemcpyAsync(d, c, static_cast<size_t>(num_groups) * m * n * 4, cudaMemcpyDeviceToDevice, stream));
    p.c = d;
    p.tma_store = 1;  // whole 128-row tiles only: a slab must not reach into the next group's rows
    return make_tensor_map_2d(tm_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, d, static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_groups) * m, static_cast<uint64_t>(n) * 4, 16, 32, CU_TENSOR_MAP_SWIZZLE_64B);
}
}  // namespace

int dgb200_per_channel_cast_to_fp8(const void* x, int32_t k, int32_t mn, int32_t gran_k, void* q, float* sf, void* stream) {
    DGB_REQUIRE(k >= 0 && mn > 0 && mn % 2 == 0, "mn (%d) must be a positive even number", mn);
    DGB_REQUIRE(gran_k == 32 || gran_k == 128, "gran_k must be 32 or 128, got %d", gran_k);
    DGB_REQUIRE(k % gran_k == 0, "k (%d) must be a multiple of gran_k (%d)", k, gran_k);
    if (k == 0) return 0;
    DGB_REQUIRE(x != nullptr && q != nullptr && sf != nullptr, "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(x) % 4 == 0 && reinterpret_cast<uintptr_t>(q) % 2 == 0 &&
                    reinterpret_cast<uintptr_t>(sf) % 8 == 0,
                "x, q and sf must be 4-, 2- and 8-byte aligned");
    const dim3 grid((mn / 2 + 255) / 256, k / gran_k);
    dgb200_cast_channels_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), k, mn, gran_k, static_cast<unsigned char*>(q), sf);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

int64_t dgb200_k_grouped_sf_workspace_bytes(int32_t num_groups, int32_t m, int32_t n, int32_t sum_k) {
    if (num_groups <= 0 || m <= 0 || n <= 0 || sum_k < 0) return 0;
    const long long rows = sum_k / 128 + 2ll * num_groups;  // one packed row per K block at most (scales per 32 K rows)
    return rows * ((static_cast<long long>(m) + 3) / 4 * 4 + (static_cast<long long>(n) + 3) / 4 * 4) * 4;
}

int dgb200_k_grouped_fp8_gemm_tn_contiguous(const void* a, const float* sfa, int32_t sf_rows, const void* b, const float* sfb,
                                            const float* c, float* d, const int32_t* ks, int32_t use_psum_layout,
                                            int32_t k_alignment, int32_t gran_k, int32_t num_groups, int32_t m, int32_t n,
                                            int32_t sum_k, void* sf_workspace, void* stream_) {
    DGB_REQUIRE(gran_k == 32 || gran_k == 128, "gran_k must be 32 or 128, got %d", gran_k);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DGB_REQUIRE(num_groups > 0 && num_groups <= kMaxCachedGroups, "num_groups must be in [1, %d]", kMaxCachedGroups);
    DGB_REQUIRE(m > 0 && m % 16 == 0 && n > 0 && n % 128 == 0, "m (%d) must be a positive multiple of 16 and n (%d) of 128", m, n);
    DGB_REQUIRE(sum_k >= 0 && sum_k % 128 == 0, "the K rows of a and b (%d) must be a multiple of 128", sum_k);
    DGB_REQUIRE(!use_psum_layout || (k_alignment > 0 && k_alignment % 128 == 0),
                "the psum layout needs a K alignment that is a multiple of 128, got %d", k_alignment);
    DGB_REQUIRE(sf_rows >= 0, "sf_rows must be >= 0");
    DGB_REQUIRE(c != nullptr && d != nullptr && ks != nullptr, "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0 && reinterpret_cast<uintptr_t>(d) % 16 == 0, "c and d must be 16-byte aligned");
    if (sum_k == 0) {
        if (c != d) DGB_CUDA(cudaMemcpyAsync(d, c, static_cast<size_t>(num_groups) * m * n * 4, cudaMemcpyDeviceToDevice, stream));
        return 0;
    }
    DGB_REQUIRE(a != nullptr && b != nullptr && sfa != nullptr && sfb != nullptr && sf_workspace != nullptr, "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(sf_workspace) % 16 == 0,
                "a, b and the workspace must be 16-byte aligned");
    const long long kp_rows = sum_k / 128 + 2ll * num_groups;
    const long long aligned_m = (static_cast<long long>(m) + 3) / 4 * 4, aligned_n = (static_cast<long long>(n) + 3) / 4 * 4;
    uint32_t* sfa_packed = static_cast<uint32_t*>(sf_workspace);
    uint32_t* sfb_packed = sfa_packed + kp_rows * aligned_m;
    {
        const dim3 grid_a(static_cast<unsigned>(std::min<long long>((static_cast<long long>(sum_k / 128 / 4 + 1) * m + 255) / 256, 64)), num_groups);
        dgb200_pack_k_grouped_sf_kernel<<<grid_a, 256, 0, stream>>>(sfa, sf_rows, ks, use_psum_layout, k_alignment, gran_k, m, aligned_m, sfa_packed);
        const dim3 grid_b(static_cast<unsigned>(std::min<long long>((static_cast<long long>(sum_k / 128 / 4 + 1) * n + 255) / 256, 64)), num_groups);
        dgb200_pack_k_grouped_sf_kernel<<<grid_b, 256, 0, stream>>>(sfb, sf_rows, ks, use_psum_layout, k_alignment, gran_k, n, aligned_n, sfb_packed);
        DGB_CUDA(cudaGetLastError());
    }
    GemmParams p{};
    p.d = d;
    p.c = c;
    p.d_row_stride = n;
    p.layout = ks;
    p.mode = kModeKGrouped;
    p.m = m;
    p.n = n;
    p.k = sum_k;
    p.num_groups = num_groups;
    p.alignment = use_psum_layout ? k_alignment : 128;
    p.kg_psum = use_psum_layout ? 1 : 0;
    p.gran_a = p.gran_b = gran_k;
    p.b_fmt = kFmtE4M3;
    // Wide tiles halve the shared-memory fill per MMA cycle, which bounds the 128-wide tile (measured 1.1 - 1.8 vs
    // 1.7 - 2.0 PFLOP/s over 1024 .. 8192 K rows per group).
    const int block_n = tuning().block_n != 0 ? tuning().block_n : (n % 256 == 0 ? 256 : 128);
    DGB_REQUIRE(n % block_n == 0, "block_n %d does not divide n %d", block_n, n);
    p.b_tx_bytes = block_n * 128;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
    int rc = make_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a, static_cast<uint64_t>(m), static_cast<uint64_t>(sum_k),
                                static_cast<uint64_t>(m), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, b, static_cast<uint64_t>(n), static_cast<uint64_t>(sum_k),
                            static_cast<uint64_t>(n), 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map_2d(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_INT32, sfa_packed, static_cast<uint64_t>(aligned_m),
                            static_cast<uint64_t>(kp_rows), static_cast<uint64_t>(aligned_m) * 4, 128, 1, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tensor_map_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_INT32, sfb_packed, static_cast<uint64_t>(aligned_n),
                            static_cast<uint64_t>(kp_rows), static_cast<uint64_t>(aligned_n) * 4, static_cast<uint32_t>(block_n), 1,
                            CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    int sms = 0;
    rc = effective_num_sms(&sms);
    if (rc) return rc;
    const long long tiles = static_cast<long long>(num_groups) * ((m + 127) / 128) * (n / block_n);
    const int grid = static_cast<int>(std::min<long long>(sms, tiles));
    // the wide tile halves the shared-memory fill per MMA cycle (the 128-wide one is bound by it)
    CUtensorMap tm_out;
    if ((rc = prepare_k_grouped_output(&tm_out, p, c, d, num_groups, m, n, stream))) return rc;
    if (block_n == 256) return launch_gemm<256, 4, kEpiF32Acc, kKindFp8Fp4>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream);
    return launch_gemm<128, 6, kEpiF32Acc, kKindFp8Fp4>(tm_a, tm_b, tm_sfa, tm_sfb, tm_out, p, grid, stream);
}

int dgb200_k_grouped_bf16_gemm_tn_contiguous(const void* a, const void* b, const float* c, float* d, const int32_t* ks,
                                             int32_t use_psum_layout, int32_t k_alignment, int32_t num_groups, int32_t m,
                                             int32_t n, int32_t sum_k, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DGB_REQUIRE(num_groups > 0 && num_groups <= kMaxCachedGroups, "num_groups must be in [1, %d]", kMaxCachedGroups);
    DGB_REQUIRE(m > 0 && m % 8 == 0 && n > 0 && n % 128 == 0, "m (%d) must be a positive multiple of 8 and n (%d) of 128", m, n);
    DGB_REQUIRE(sum_k >= 0 && sum_k % 64 == 0, "the K rows of a and b (%d) must be a multiple of 64", sum_k);
    DGB_REQUIRE(!use_psum_layout || (k_alignment > 0 && k_alignment % 64 == 0),
                "the psum layout needs a K alignment that is a multiple of 64, got %d", k_alignment);
    DGB_REQUIRE(c != nullptr && d != nullptr && ks != nullptr, "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(c) % 16 == 0 && reinterpret_cast<uintptr_t>(d) % 16 == 0, "c and d must be 16-byte aligned");
    if (sum_k == 0) {
        if (c != d) DGB_CUDA(cudaMemcpyAsync(d, c, static_cast<size_t>(num_groups) * m * n * 4, cudaMemcpyDeviceToDevice, stream));
        return 0;
    }
    DGB_REQUIRE(a != nullptr && b != nullptr, "null tensor pointer");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0, "a and b must be 16-byte aligned");
    GemmParams p{};
    p.d = d;
    p.c = c;
    p.d_row_stride = n;
    p.layout = ks;
    p.mode = kModeKGrouped;
    p.m = m;
    p.n = n;
    p.k = sum_k;
    p.num_groups = num_groups;
    p.alignment = use_psum_layout ? k_alignment : 128;
    p.kg_psum = use_psum_layout ? 1 : 0;
    p.gran_a = p.gran_b = 32;
    p.sf_transposed = 1;
    const int block_n = tuning().block_n != 0 ? tuning().block_n : (n % 256 == 0 ? 256 : 128);
    DGB_REQUIRE(n % block_n == 0, "block_n %d does not divide n %d", block_n, n);
    p.b_tx_bytes = block_n * 128;
    CUtensorMap tm_a, tm_b;
    int rc = make_tensor_map_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, static_cast<uint64_t>(m), static_cast<uint64_t>(sum_k),
                                static_cast<uint64_t>(m) * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, static_cast<uint64_t>(n), static_cast<uint64_t>(sum_k),
                            static_cast<uint64_t>(n) * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    int sms = 0;
    rc = effective_num_sms(&sms);
    if (rc) return rc;
    const long long tiles = static_cast<long long>(num_groups) * ((m + 127) / 128) * (n / block_n);
    const int grid = static_cast<int>(std::min<long long>(sms, tiles));
    CUtensorMap tm_out;
    if ((rc = prepare_k_grouped_output(&tm_out, p, c, d, num_groups, m, n, stream))) return rc;
    if (block_n == 256) return launch_gemm<256, 4, kEpiF32Acc, kKindBf16>(tm_a, tm_b, tm_a, tm_a, tm_out, p, grid, stream);
    return launch_gemm<128, 6, kEpiF32Acc, kKindBf16>(tm_a, tm_b, tm_a, tm_a, tm_out, p, grid, stream);
}

int dgb200_route_sigmoid_topk(const float* logits, int32_t tokens, int32_t experts, int32_t topk, int64_t* topk_idx,
                              float* topk_weights, void* stream) {
    DGB_REQUIRE(logits != nullptr && topk_idx != nullptr && topk_weights != nullptr, "null tensor pointer");
    DGB_REQUIRE(tokens >= 0 && experts > 0 && experts <= 1024, "experts must be in [1, 1024]");
    DGB_REQUIRE(topk > 0 && topk <= 32 && topk <= experts, "topk must be in [1, min(32, experts)]");
    if (tokens == 0) return 0;
    const int grid = (tokens + 7) / 8;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long* idx = reinterpret_cast<long long*>(topk_idx);
    if (experts <= 256)
        DGB_CUDA(launch_kernel(dgb200_route_sigmoid_topk_kernel<8>, dim3(grid), dim3(256), 0, s, use_pdl(), logits, tokens, experts, topk, idx,
                               topk_weights));
    else
        DGB_CUDA(launch_kernel(dgb200_route_sigmoid_topk_kernel<32>, dim3(grid), dim3(256), 0, s, use_pdl(), logits, tokens, experts, topk, idx,
                               topk_weights));
    return 0;
}

int dgb200_get_token_alignment_for_mega_moe(void) { return 128; }

int dgb200_get_segment_alignment_for_mega_moe(void) { return kSegmentAlignment; }

int dgb200_get_weight_tile_rows_for_mega_moe(void) { return mlp_kernel_choice() != 0 ? 128 : 0; }

int dgb200_get_gate_up_interleave_for_mega_moe(void) { return mlp_kernel_choice() != 0 ? kMlpGateUpInterleave : 128; }

int dgb200_get_symm_buffer_layout_for_mega_moe(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                               int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                               int64_t* out) {
    return export_mega_layout(kKindFp8Fp4, num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                              intermediate_hidden, out);
}

int dgb200_get_symm_buffer_layout_for_nvfp4_mega_moe(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                                     int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                                     int64_t* out) {
    return export_mega_layout(kKindNvfp4, num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                              intermediate_hidden, out);
}

int dgb200_fp8_fp4_mega_moe(void* y, const void* l1_w, const void* l1_w_sf, const void* l2_w, const void* l2_w_sf,
                            int32_t* cumulative_local_expert_recv_stats, void* buffer, const uint64_t* peer_buffer_ptrs,
                            int32_t rank, int32_t num_ranks, int32_t num_tokens, int32_t num_max_tokens_per_rank,
                            int32_t num_experts, int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                            float activation_clamp, int32_t fast_math, void* stream) {
    LayerQuant quant;
    return run_mega_moe(quant, y, l1_w, l1_w_sf, l2_w, l2_w_sf, cumulative_local_expert_recv_stats, buffer, peer_buffer_ptrs, rank,
                        num_ranks, num_tokens, num_max_tokens_per_rank, num_experts, num_topk, hidden, intermediate_hidden,
                        activation_clamp, fast_math, static_cast<cudaStream_t>(stream));
}

int dgb200_fp8_fp4_mega_moe_bf16_input(void* y, const void* x, int64_t x_row_stride, const float* logits, const void* l1_w,
                                       const void* l1_w_sf, const void* l2_w, const void* l2_w_sf,
                                       int32_t* cumulative_local_expert_recv_stats, void* buffer,
                                       const uint64_t* peer_buffer_ptrs, int32_t rank, int32_t num_ranks, int32_t num_tokens,
                                       int32_t num_max_tokens_per_rank, int32_t num_experts, int32_t num_topk, int32_t hidden,
                                       int32_t intermediate_hidden, float activation_clamp, int32_t fast_math, void* stream) {
    DGB_REQUIRE(x != nullptr && reinterpret_cast<uintptr_t>(x) % 16 == 0 && x_row_stride >= hidden && (x_row_stride * 2) % 16 == 0,
                "x must be 16-byte aligned BF16 rows of at least `hidden` elements");
    if (logits != nullptr && num_tokens > 0) {
        MegaLayout l;
        int rc = make_mega_layout(kKindFp8Fp4, num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden, &l);
        if (rc) return rc;
        DGB_REQUIRE(buffer != nullptr && num_tokens <= num_max_tokens_per_rank, "bad buffer or token count");
        uint8_t* base = static_cast<uint8_t*>(buffer);
        rc = dgb200_route_sigmoid_topk(logits, num_tokens, num_experts, num_topk, reinterpret_cast<int64_t*>(base + l.topk_idx),
                                       reinterpret_cast<float*>(base + l.topk_weights), stream);
        if (rc) return rc;
    }
    LayerQuant quant;
    quant.x_bf16 = static_cast<const __nv_bfloat16*>(x);
    quant.x_bf16_row_stride = x_row_stride;
    return run_mega_moe(quant, y, l1_w, l1_w_sf, l2_w, l2_w_sf, cumulative_local_expert_recv_stats, buffer, peer_buffer_ptrs, rank,
                        num_ranks, num_tokens, num_max_tokens_per_rank, num_experts, num_topk, hidden, intermediate_hidden,
                        activation_clamp, fast_math, static_cast<cudaStream_t>(stream));
}

int dgb200_get_symm_buffer_layout_for_mega_moe_ex(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                                  int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                                  int32_t shared_intermediate_hidden, int64_t* out) {
    DGB_REQUIRE(out != nullptr && shared_intermediate_hidden >= 0, "null output or negative shared size");
    MegaLayout l;
    const int rc = make_mega_layout(kKindFp8Fp4, num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                                    intermediate_hidden, &l, shared_intermediate_hidden);
    if (rc) return rc;
    const long long fields[26] = {l.total, l.x, l.x_sf, l.topk_idx, l.topk_weights, l.l1_acts, l.l1_sf, l.l2_acts, l.l2_sf,
                                  l.max_rows, l.dest_row, l.src_of_row, l.expert_start, l.expert_end, l.l2_out, l.row_weight,
                                  l.shared_x_sf, l.shared_l2_acts, l.shared_l2_sf, l.shared_out, l.flags,
                                  l.my_base, l.my_dest, l.my_slot, l.guest_expert, l.rank_rows};
    for (int i = 0; i < 26; ++i) out[i] = fields[i];
    return 0;
}

int dgb200_fp8_fp4_mega_moe_ex(const dgb200_mega_moe_args* a, void* stream) {
    DGB_REQUIRE(a != nullptr && a->struct_size == sizeof(dgb200_mega_moe_args),
                "dgb200_mega_moe_args: struct_size does not match this library (%zu bytes)", sizeof(dgb200_mega_moe_args));
    LayerQuant quant;
    if (a->x_bf16 != nullptr) {
        DGB_REQUIRE(reinterpret_cast<uintptr_t>(a->x_bf16) % 16 == 0 && a->x_bf16_row_stride >= a->hidden &&
                        (a->x_bf16_row_stride * 2) % 16 == 0,
                    "x_bf16 must be 16-byte aligned BF16 rows of at least `hidden` elements");
        quant.x_bf16 = static_cast<const __nv_bfloat16*>(a->x_bf16);
        quant.x_bf16_row_stride = a->x_bf16_row_stride;
    }
    if (a->shared_intermediate_hidden > 0) {
        quant.shared_l1_w = a->shared_l1_w;
        quant.shared_l1_w_sf = a->shared_l1_w_sf;
        quant.shared_l2_w = a->shared_l2_w;
        quant.shared_l2_w_sf = a->shared_l2_w_sf;
        quant.shared_inter = a->shared_intermediate_hidden;
    }
    if (a->num_guest_experts > 0 && a->num_ranks > 1) {
        quant.guest_slots = a->num_guest_experts;
        quant.peer_w[0] = a->peer_l1_w;
        quant.peer_w[1] = a->peer_l1_w_sf;
        quant.peer_w[2] = a->peer_l2_w;
        quant.peer_w[3] = a->peer_l2_w_sf;
    }
    if (a->logits != nullptr && a->num_tokens > 0) {
        MegaLayout l;
        int rc = make_mega_layout(kKindFp8Fp4, a->num_ranks, a->num_experts, a->num_max_tokens_per_rank, a->num_topk, a->hidden,
                                  a->intermediate_hidden, &l, quant.shared_inter);
        if (rc) return rc;
        DGB_REQUIRE(a->buffer != nullptr && a->num_tokens <= a->num_max_tokens_per_rank, "bad buffer or token count");
        uint8_t* base = static_cast<uint8_t*>(a->buffer);
        rc = dgb200_route_sigmoid_topk(a->logits, a->num_tokens, a->num_experts, a->num_topk,
                                       reinterpret_cast<int64_t*>(base + l.topk_idx), reinterpret_cast<float*>(base + l.topk_weights),
                                       stream);
        if (rc) return rc;
    }
    return run_mega_moe(quant, a->y, a->l1_w, a->l1_w_sf, a->l2_w, a->l2_w_sf, a->cumulative_local_expert_recv_stats, a->buffer,
                        a->peer_buffer_ptrs, a->rank, a->num_ranks, a->num_tokens, a->num_max_tokens_per_rank, a->num_experts,
                        a->num_topk, a->hidden, a->intermediate_hidden, a->activation_clamp, a->fast_math,
                        static_cast<cudaStream_t>(stream));
}

int dgb200_nvfp4_mega_moe(void* y, const void* l1_w, const void* l1_w_sf, const float* l1_w_scales, const void* l2_w,
                          const void* l2_w_sf, const float* l2_w_scales, const float* x_scale, const float* act_scale,
                          int32_t* cumulative_local_expert_recv_stats, void* buffer, const uint64_t* peer_buffer_ptrs,
                          int32_t rank, int32_t num_ranks, int32_t num_tokens, int32_t num_max_tokens_per_rank,
                          int32_t num_experts, int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                          float activation_clamp, int32_t fast_math, void* stream) {
    DGB_REQUIRE(l1_w_scales != nullptr && l2_w_scales != nullptr && x_scale != nullptr && act_scale != nullptr,
                "null per-tensor scale pointer");
    LayerQuant quant;
    quant.kind = kKindNvfp4;
    quant.x_scale = x_scale;
    quant.act_scale = act_scale;
    quant.l1_scales = l1_w_scales;
    quant.l2_scales = l2_w_scales;
    return run_mega_moe(quant, y, l1_w, l1_w_sf, l2_w, l2_w_sf, cumulative_local_expert_recv_stats, buffer, peer_buffer_ptrs, rank,
                        num_ranks, num_tokens, num_max_tokens_per_rank, num_experts, num_topk, hidden, intermediate_hidden,
                        activation_clamp, fast_math, static_cast<cudaStream_t>(stream));
}

int dgb200_nvfp4_mega_moe_bf16_input(void* y, const void* x, int64_t x_row_stride, const float* logits, const void* l1_w,
                                     const void* l1_w_sf, const float* l1_w_scales, const void* l2_w, const void* l2_w_sf,
                                     const float* l2_w_scales, const float* x_scale, const float* act_scale,
                                     int32_t* cumulative_local_expert_recv_stats, void* buffer, int32_t num_tokens,
                                     int32_t num_max_tokens_per_rank, int32_t num_experts, int32_t num_topk, int32_t hidden,
                                     int32_t intermediate_hidden, float activation_clamp, int32_t fast_math, void* stream) {
    DGB_REQUIRE(l1_w_scales != nullptr && l2_w_scales != nullptr && x_scale != nullptr && act_scale != nullptr,
                "null per-tensor scale pointer");
    DGB_REQUIRE(x != nullptr && reinterpret_cast<uintptr_t>(x) % 16 == 0 && x_row_stride >= hidden && (x_row_stride * 2) % 16 == 0,
                "x must be 16-byte aligned BF16 rows of at least `hidden` elements");
    if (logits != nullptr && num_tokens > 0) {
        MegaLayout l;
        int rc = make_mega_layout(kKindNvfp4, 1, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden, &l);
        if (rc) return rc;
        DGB_REQUIRE(buffer != nullptr && num_tokens <= num_max_tokens_per_rank, "bad buffer or token count");
        uint8_t* base = static_cast<uint8_t*>(buffer);
        rc = dgb200_route_sigmoid_topk(logits, num_tokens, num_experts, num_topk, reinterpret_cast<int64_t*>(base + l.topk_idx),
                                       reinterpret_cast<float*>(base + l.topk_weights), stream);
        if (rc) return rc;
    }
    LayerQuant quant;
    quant.kind = kKindNvfp4;
    quant.x_scale = x_scale;
    quant.act_scale = act_scale;
    quant.l1_scales = l1_w_scales;
    quant.l2_scales = l2_w_scales;
    quant.x_bf16 = static_cast<const __nv_bfloat16*>(x);
    quant.x_bf16_row_stride = x_row_stride;
    const uint64_t self = reinterpret_cast<uint64_t>(buffer);
    return run_mega_moe(quant, y, l1_w, l1_w_sf, l2_w, l2_w_sf, cumulative_local_expert_recv_stats, buffer, &self, 0, 1, num_tokens,
                        num_max_tokens_per_rank, num_experts, num_topk, hidden, intermediate_hidden, activation_clamp, fast_math,
                        static_cast<cudaStream_t>(stream));
}

int dgb200_get_symm_buffer_layout_for_bf16_mega_moe(int32_t num_ranks, int32_t num_experts, int32_t num_max_tokens_per_rank,
                                                    int32_t num_topk, int32_t hidden, int32_t intermediate_hidden,
                                                    int32_t shared_intermediate_hidden, int64_t* out) {
    DGB_REQUIRE(out != nullptr && shared_intermediate_hidden >= 0, "null output or negative shared size");
    MegaLayout l;
    const int rc = make_mega_layout(kKindBf16, num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                                    intermediate_hidden, &l, shared_intermediate_hidden);
    if (rc) return rc;
    const long long fields[26] = {l.total, l.x, l.x_sf, l.topk_idx, l.topk_weights, l.l1_acts, l.l1_sf, l.l2_acts, l.l2_sf,
                                  l.max_rows, l.dest_row, l.src_of_row, l.expert_start, l.expert_end, l.l2_out, l.row_weight,
                                  l.shared_x_sf, l.shared_l2_acts, l.shared_l2_sf, l.shared_out, l.flags,
                                  l.my_base, l.my_dest, l.my_slot, l.guest_expert, l.rank_rows};
    for (int i = 0; i < 26; ++i) out[i] = fields[i];
    return 0;
}

int dgb200_bf16_mega_moe(void* y, const void* l1_w, const void* l2_w, const void* shared_l1_w, const void* shared_l2_w,
                         int32_t shared_intermediate_hidden, int32_t* cumulative_local_expert_recv_stats, void* buffer,
                         const uint64_t* peer_buffer_ptrs, int32_t rank, int32_t num_ranks, int32_t num_tokens,
                         int32_t num_max_tokens_per_rank, int32_t num_experts, int32_t num_topk, int32_t hidden,
                         int32_t intermediate_hidden, float activation_clamp, int32_t fast_math, void* stream) {
    LayerQuant quant;
    quant.kind = kKindBf16;
    DGB_REQUIRE(shared_intermediate_hidden >= 0, "negative shared size");
    if (shared_intermediate_hidden > 0) {
        quant.shared_l1_w = shared_l1_w;
        quant.shared_l2_w = shared_l2_w;
        quant.shared_inter = shared_intermediate_hidden;
    }
    return run_mega_moe(quant, y, l1_w, nullptr, l2_w, nullptr, cumulative_local_expert_recv_stats, buffer, peer_buffer_ptrs, rank,
                        num_ranks, num_tokens, num_max_tokens_per_rank, num_experts, num_topk, hidden, intermediate_hidden,
                        activation_clamp, fast_math, static_cast<cudaStream_t>(stream));
}

int dgb200_set_mega_moe_stage_events(void* const* events, int32_t count) {
    DGB_REQUIRE(count >= 0 && count <= kNumStageEvents, "count must be in [0, %d]", kNumStageEvents);
    DGB_REQUIRE(count == 0 || events != nullptr, "null event array");
    for (int i = 0; i < count; ++i) g_stage_events[i] = static_cast<cudaEvent_t>(events[i]);
    g_num_stage_events = count;
    return 0;
}

int dgb200_moe_dispatch_plan_noalloc(const int64_t* topk_idx, int32_t num_tokens, int32_t num_topk, int32_t num_experts,
                                     int32_t alignment, int32_t* dest_row, int32_t* expert_start, int32_t* expert_end,
                                     void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DGB_REQUIRE(topk_idx != nullptr && dest_row != nullptr && expert_start != nullptr && expert_end != nullptr,
                "null tensor pointer");
    DGB_REQUIRE(num_tokens >= 0 && num_topk > 0 && num_experts > 0 && alignment > 0, "bad shape");
    const long long entries = static_cast<long long>(num_tokens) * num_topk;
    DGB_REQUIRE(entries <= kNoAllocMaxEntries,
                "num_tokens * num_topk = %lld exceeds the built-in scratch (%d entries); use the layer call with a caller buffer",
                entries, kNoAllocMaxEntries);
    DGB_REQUIRE(num_experts <= kNoAllocMaxExperts, "num_experts = %d exceeds the built-in scratch (%d experts)", num_experts,
                kNoAllocMaxExperts);
    int* scratch = nullptr;
    const int rc = noalloc_scratch_for_current_device(&scratch);
    if (rc) return rc;
    int* total_rows = scratch;        // 1 word (rewritten by every call)
    int* chunk_hist = scratch + 64;   // [chunks][num_experts], every word the later kernels read is rewritten first
    const int n = static_cast<int>(entries);
    const int chunks = std::max(1, (n + kPlanChunk - 1) / kPlanChunk);
    const long long* idx = reinterpret_cast<const long long*>(topk_idx);
    dgb200_moe_count_kernel<<<chunks, kPlanChunk, num_experts * sizeof(int), stream>>>(idx, n, 0, num_experts, chunk_hist);
    dgb200_moe_scan_kernel<<<1, 1024, 0, stream>>>(chunk_hist, chunks, num_experts, alignment, expert_start, expert_end,
                                                    total_rows, nullptr);
    if (n > 0)
        dgb200_ep_assign_kernel<<<chunks, kPlanChunk, 32 * num_experts, stream>>>(idx, n, num_experts, chunk_hist, expert_start,
                                                                              dest_row);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

int dgb200_ep_plan_with_guest_experts(const int32_t* all_counts, int32_t num_ranks, int32_t num_experts, int32_t rank,
                                      int32_t alignment, int32_t num_guest_experts, int32_t* my_base, int32_t* my_dest,
                                      int32_t* my_slot, int32_t* slot_start, int32_t* slot_end, int32_t* guest_expert,
                                      int32_t* rank_rows, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DGB_REQUIRE(all_counts != nullptr && my_base != nullptr && my_dest != nullptr && my_slot != nullptr && slot_start != nullptr &&
                    slot_end != nullptr && guest_expert != nullptr && rank_rows != nullptr,
                "null tensor pointer");
    DGB_REQUIRE(num_ranks >= 1 && num_ranks <= kMaxEpRanks && num_experts > 0 && num_experts % num_ranks == 0 && rank >= 0 &&
                    rank < num_ranks && alignment > 0,
                "need 1 <= num_ranks <= %d, num_experts a positive multiple of it, 0 <= rank < num_ranks, alignment > 0", kMaxEpRanks);
    DGB_REQUIRE(num_guest_experts >= 0 && num_guest_experts <= kMaxGuestExperts &&
                    num_experts / num_ranks + num_guest_experts <= kMaxSpillSlots - 1,
                "at most %d guest experts and %d expert slots per rank", kMaxGuestExperts, kMaxSpillSlots - 1);
    DGB_REQUIRE(static_cast<long long>(num_ranks) * num_experts * 6 <= 30 * 1024, "too many experts x ranks for the plan's tables");
    // the row total is internal to the layer call; here it lands behind the rank_rows output ([2][num_ranks] + 1 word)
    dgb200_ep_spill_plan_kernel<<<1, 1024, static_cast<size_t>(num_ranks) * num_experts * 6, stream>>>(
        all_counts, num_experts, num_ranks, rank, alignment, num_guest_experts, my_base, my_dest, my_slot, slot_start, slot_end,
        rank_rows + 2 * num_ranks, guest_expert, rank_rows, nullptr);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

int dgb200_nvfp4_tensor_scale(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, float* out_scale, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    DGB_REQUIRE(x != nullptr && out_scale != nullptr, "null tensor pointer");
    DGB_REQUIRE(rows >= 0 && k > 0 && k % 8 == 0 && (x_row_stride * 2) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0,
                "x rows must be 16-byte aligned and k a multiple of 8");
    DGB_CUDA(cudaMemsetAsync(out_scale, 0, sizeof(float), stream));
    if (rows > 0) {
        const long long vecs = static_cast<long long>(rows) * (k / 8);
        const int grid = static_cast<int>(std::min<long long>((vecs + 255) / 256, 148 * 8));
        dgb200_amax_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), x_row_stride, rows, k, out_scale);
    }
    dgb200_finish_tensor_scale_kernel<<<1, 1, 0, stream>>>(out_scale);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

int dgb200_per_token_cast_to_nvfp4(const void* x, int64_t x_row_stride, int32_t rows, int32_t k, const float* tensor_scale,
                                   void* q, int64_t q_row_stride, void* sf_packed, int64_t sf_k_stride,
                                   int64_t sf_row_stride, void* stream) {
    DGB_REQUIRE(x != nullptr && q != nullptr && sf_packed != nullptr && tensor_scale != nullptr, "null tensor pointer");
    DGB_REQUIRE(rows >= 0 && k > 0 && k % 64 == 0, "k (%d) must be a positive multiple of 64", k);
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0 && (x_row_stride * 2) % 16 == 0, "x rows must be 16-byte aligned");
    DGB_REQUIRE(reinterpret_cast<uintptr_t>(q) % 8 == 0 && q_row_stride % 8 == 0, "q rows must be 8-byte aligned");
    DGB_REQUIRE((sf_row_stride == 1 && sf_k_stride >= rows) || (sf_k_stride == 1 && sf_row_stride >= k / 64),
                "packed scale-factor strides must be (k stride >= rows, row stride 1) or (k stride 1, row stride >= k / 64)");
    if (rows == 0) return 0;
    CastNvfp4Params p{};
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.x_row_stride = x_row_stride;
    p.q = static_cast<unsigned char*>(q);
    p.q_row_stride = q_row_stride;
    p.tensor_scale = tensor_scale;
    p.sf_packed = static_cast<uint32_t*>(sf_packed);
    p.sf_k_stride = sf_k_stride;
    p.sf_row_stride = sf_row_stride;
    p.rows = rows;
    p.k = k;
    const dim3 grid((k + 511) / 512, (rows + 31) / 32);
    dgb200_cast_rows_nvfp4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    DGB_CUDA(cudaGetLastError());
    return 0;
}

int dgb200_m_grouped_nvfp4_gemm_nt_contiguous(
    const void* a, const void* sfa, int64_t sfa_k_stride, const float* a_scale,
    const void* b, const void* sfb, int64_t sfb_k_stride, int64_t sfb_group_stride, const float* b_scales,
    void* d, int64_t d_row_stride, const int32_t* grouped_layout,
    int32_t m, int32_t n, int32_t k, int32_t num_groups, int32_t d_is_fp32,
    int32_t layout_kind, int32_t alignment, void* stream) {
    DGB_REQUIRE(m >= 0, "m must be >= 0");
    DGB_REQUIRE(layout_kind == DGB200_LAYOUT_ROW_IDS || layout_kind == DGB200_LAYOUT_PSUM, "unknown layout kind %d", layout_kind);
    DGB_REQUIRE(alignment > 0 && alignment % 4 == 0, "alignment (%d) must be a positive multiple of 4", alignment);
    DGB_REQUIRE(layout_kind == DGB200_LAYOUT_PSUM || alignment % 128 == 0,
                "the row-id layout needs an M alignment that is a multiple of 128, got %d", alignment);
    DGB_REQUIRE(d != nullptr || m == 0, "null output");
    DGB_REQUIRE(a_scale != nullptr && b_scales != nullptr, "null per-tensor scale pointer");
    DGB_REQUIRE(d_row_stride >= n && (d_row_stride * (d_is_fp32 ? 4 : 2)) % 16 == 0,
                "d row stride must cover n and keep rows 16-byte aligned");
    DGB_REQUIRE(sfa_k_stride >= m, "sfa MN stride smaller than m");
    GemmCall c{};
    c.kind = kKindNvfp4;
    c.a = a;
    c.b = b;
    c.a_rows_total = m;
    c.b_is_fp4 = 1;
    c.epilogue = d_is_fp32 ? kEpiF32 : kEpiBF16;
    c.sfa = sfa;
    c.sfb = sfb;
    c.sfa_k_stride = sfa_k_stride;
    c.num_groups_a = 1;
    c.sfb_k_stride = sfb_k_stride;
    c.sfb_group_stride = sfb_group_stride;
    GemmParams& p = c.p;
    p.d = d;
    p.d_row_stride = d_row_stride;
    p.layout = grouped_layout;
    p.mode = layout_kind == DGB200_LAYOUT_PSUM ? kModePsum : kModeRowIds;
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_groups = num_groups;
    p.alignment = alignment;
    p.a_scale = a_scale;
    p.b_scales = b_scales;
    c.max_tiles = 0;
    return run_gemm(c, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
