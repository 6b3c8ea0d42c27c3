// Dispatch (count / slot assignment / gather) and combine kernels of the MoE layer. All HBM-bound integer and
// byte work: coalesced 16-byte vectors, scale factors transposed through shared memory.
//
// Reference counterparts (inside the fused kernel deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh):
//   count + slot assignment  :329-399   (atomics; arrival-order dependent)
//   token pull into the L1 ring :461-599
//   combine                  :1323-1452
// Differences by design: slot assignment here is a deterministic stable sort of the (token, k) entries by expert
// (entry order = token-major), so the permutation is reproducible bit for bit; and each expert segment is padded
// only to `alignment` rows (4..128) instead of to a full M block, because the GEMM clips its stores per group.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "quant_kernels.cuh"

namespace dgb {

constexpr int kPlanChunk = 1024;  // (token, k) entries per CTA in the count / assign kernels

// chunk_hist[chunk][e] = number of entries of `chunk` routed to local expert e.
// An entry is local when expert_lo <= topk_idx < expert_lo + num_local_experts.
__global__ void __launch_bounds__(kPlanChunk)
dgb200_moe_count_kernel(const long long* __restrict__ topk_idx, int num_entries, int expert_lo, int num_local_experts,
                        int* __restrict__ chunk_hist) {
    pdl_prologue();
    extern __shared__ int hist[];
    for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * kPlanChunk + threadIdx.x;
    if (i < num_entries) {
        const long long e = topk_idx[i] - expert_lo;
        if (e >= 0 && e < num_local_experts) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < num_local_experts; e += blockDim.x)
        chunk_hist[static_cast<long long>(blockIdx.x) * num_local_experts + e] = hist[e];
}

// One CTA. Turns chunk_hist into exclusive per-chunk bases, and produces per expert: count, aligned segment start,
// segment end (the psum layout the grouped GEMM walks). total_rows[0] = end of the last segment.
__global__ void __launch_bounds__(1024)
dgb200_moe_scan_kernel(int* __restrict__ chunk_hist, int num_chunks, int num_local_experts, int alignment,
                       int* __restrict__ expert_start, int* __restrict__ expert_end, int* __restrict__ total_rows,
                       int* __restrict__ cumulative_stats) {
    pdl_prologue();
    __shared__ int warp_sums[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < num_local_experts; base += 1024) {
        const int e = base + static_cast<int>(threadIdx.x);
        int count = 0;
        if (e < num_local_experts) {
            for (int c = 0; c < num_chunks; ++c) {
                int* slot = chunk_hist + static_cast<long long>(c) * num_local_experts + e;
                const int t = *slot;
                *slot = count;
                count += t;
            }
            if (cumulative_stats != nullptr) cumulative_stats[e] += count;
        }
        const int padded = (count + alignment - 1) / alignment * alignment;
        // block-wide exclusive scan of `padded`
        int incl = padded;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        for (int off = 1; off < 32; off <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += n;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, w, off);
                if (lane >= off) w += n;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int start = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - padded;
        if (e < num_local_experts) {
            expert_start[e] = start;
            expert_end[e] = start + count;
        }
        __syncthreads();
        if (threadIdx.x == 1023) carry = start + padded;
        __syncthreads();
    }
    if (threadIdx.x == 0) total_rows[0] = carry;
}

// dest_row[entry] = expert_start[e] + (entries of the same expert that precede it), or -1 when not local;
// src_of_row[dest] = entry; row_weight[dest] = topk_weights[entry].
__global__ void __launch_bounds__(kPlanChunk)
dgb200_moe_assign_kernel(const long long* __restrict__ topk_idx, const float* __restrict__ topk_weights, int num_entries,
                         int expert_lo, int num_local_experts, const int* __restrict__ chunk_hist,
                         const int* __restrict__ expert_start, int* __restrict__ dest_row, int* __restrict__ src_of_row,
                         float* __restrict__ row_weight) {
    pdl_prologue();
    extern __shared__ unsigned char warp_hist[];  // [32 warps][num_local_experts], counts <= 32
    for (int i = threadIdx.x; i < 32 * num_local_experts; i += blockDim.x) warp_hist[i] = 0;
    __syncthreads();
    const int i = blockIdx.x * kPlanChunk + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int e = -1;
    if (i < num_entries) {
        const long long g = topk_idx[i] - expert_lo;
        if (g >= 0 && g < num_local_experts) e = static_cast<int>(g);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_hist[warp * num_local_experts + e] = static_cast<unsigned char>(__popc(peers));
    __syncthreads();
    if (i >= num_entries) return;
    if (e < 0) {
        dest_row[i] = -1;
        return;
    }
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_hist[w * num_local_experts + e];
    const int dest = expert_start[e] + chunk_hist[static_cast<long long>(blockIdx.x) * num_local_experts + e] + before +
                     rank_in_warp;
    dest_row[i] = dest;
    src_of_row[dest] = i;
    row_weight[dest] = topk_weights[i];
}

// Gathers quantised token rows and their packed scales into expert-sorted order. One CTA per 32 destination rows.
//   x      [tokens, row_bytes] bytes (e4m3: hidden; packed e2m1: hidden / 2)
//   x_sf   int32 [tokens, sf_per_row] token-major, 4 scale bytes per int (UE8M0 per 32: hidden / 128 ints;
//          UE4M3 per 16: hidden / 64 ints)
//   acts   [rows, row_bytes]               acts_sf int32 MN-major with every 128 rows in tcgen05.cp order: int (kp, row)
//                                          at acts_sf[kp * sf_k_stride + sf_row_in_cp_order(row)]
// Rows whose src_of_row is negative (segment padding) are left untouched.
__global__ void __launch_bounds__(256)
dgb200_moe_gather_kernel(const unsigned char* __restrict__ x, const unsigned* __restrict__ x_sf,
                         const int* __restrict__ src_of_row, const int* __restrict__ total_rows, int topk, int row_bytes,
                         int sf_per_row, unsigned char* __restrict__ acts, unsigned* __restrict__ acts_sf,
                         long long sf_k_stride) {
    pdl_prologue();
    extern __shared__ unsigned sf_tile[];  // [sf_per_row][33]
    const int row0 = blockIdx.x * 32;
    if (row0 >= total_rows[0]) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int rr = 0; rr < 4; ++rr) {
        const int r = warp * 4 + rr;
        const int src = src_of_row[row0 + r];
        if (src < 0) continue;
        const int token = src / topk;
        const uint4* from = reinterpret_cast<const uint4*>(x + static_cast<long long>(token) * row_bytes);
        uint4* to = reinterpret_cast<uint4*>(acts + static_cast<long long>(row0 + r) * row_bytes);
        for (int c = lane; c < row_bytes / 16; c += 32) to[c] = ld_global_nc_v4(from + c);
        for (int c = lane; c < sf_per_row; c += 32) sf_tile[c * 33 + r] = x_sf[static_cast<long long>(token) * sf_per_row + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < sf_per_row * 32; i += 256) {
        const int c = i >> 5, r = i & 31;
        if (src_of_row[row0 + r] >= 0)
            acts_sf[static_cast<long long>(c) * sf_k_stride + sf_row_in_cp_order(row0 + r)] = sf_tile[c * 33 + r];
    }
}

// Router of the benchmark layer: per token, the `topk` largest logits (descending; ties -> lower expert index),
// weights = sigmoid(logit) renormalised to sum to one. One warp per token, expert e held by lane e % 32.
// The reference leaves routing to the caller (tests/test_mega_moe.py:124-125 uses torch.topk).
template <int kMaxPerLane>
__global__ void __launch_bounds__(256)
dgb200_route_sigmoid_topk_kernel(const float* __restrict__ logits, int tokens, int experts, int topk,
                                 long long* __restrict__ topk_idx, float* __restrict__ topk_weights) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= tokens) return;
    float v[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < experts ? logits[static_cast<long long>(t) * experts + e] : -INFINITY;
    }
    float my_score = 0.0f, sum = 0.0f;
    int my_idx = 0;
    for (int k = 0; k < topk; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i)
            if (v[i] > best) { best = v[i]; best_e = i * 32 + lane; }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, off);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < kMaxPerLane; ++i)
                if (i == (best_e >> 5)) v[i] = -INFINITY;
        }
        const float score = 1.0f / (1.0f + expf(-best));
        sum += score;
        if (lane == k) { my_score = score; my_idx = best_e; }
    }
    if (lane < topk) {
        topk_idx[static_cast<long long>(t) * topk + lane] = my_idx;
        topk_weights[static_cast<long long>(t) * topk + lane] = my_score / sum;
    }
}

constexpr int kMaxEpRanks = 8;
struct PeerTable {
    unsigned long long p[kMaxEpRanks];  // address of every rank's buffer as mapped into this process
};

// y[t, :] = bf16( sum over valid k, in ascending k, of float(row(t, k)[:]) ), where row(t, k) is the L2 GEMM's output
// row for entry (t, k): row dest_row[t * topk + k] of the `rows` buffer of the rank that owns expert topk_idx[t, k]
// (read in place over NVLink when that is another rank: the combine pulls, nothing is pushed). Slots with
// dest_row < 0 are skipped. One CTA per token; a thread owns 8 consecutive channels (one 16-byte vector per slot).
// With shared experts their output row of the token (local, bf16 [tokens, hidden] at `shared_rows`) is one more slot,
// added after the top-k slots (the reference gives it combine slot index num_topk, ...mega_moe.cuh:1275-1278).
// Reference: the combine of the fused kernel, deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:1323-1452.
__global__ void __launch_bounds__(128)
dgb200_moe_combine_kernel(const PeerTable peers, long long rows_offset, const long long* __restrict__ topk_idx,
                          const int* __restrict__ dest_row, int topk, int experts_per_rank, int hidden,
                          const __nv_bfloat16* __restrict__ shared_rows, __nv_bfloat16* __restrict__ y) {
    pdl_prologue();
    const int t = blockIdx.x;
    extern __shared__ unsigned long long slot_rows[];  // address of each slot's row (top-k slots, then the shared one), 0 = skip
    if (threadIdx.x == topk)
        slot_rows[topk] = shared_rows != nullptr
            ? reinterpret_cast<unsigned long long>(shared_rows + static_cast<long long>(t) * hidden) : 0ull;
    if (threadIdx.x < topk) {
        const int d = dest_row[static_cast<long long>(t) * topk + threadIdx.x];
        unsigned long long addr = 0;
        if (d >= 0) {
            const int owner = static_cast<int>(topk_idx[static_cast<long long>(t) * topk + threadIdx.x]) / experts_per_rank;
            addr = peers.p[owner] + rows_offset + static_cast<unsigned long long>(d) * hidden * 2;
        }
        slot_rows[threadIdx.x] = addr;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k <= topk; ++k) {
            const unsigned long long addr = slot_rows[k];
            if (addr == 0) continue;
            const uint4 v = ld_global_nc_v4(reinterpret_cast<const uint4*>(addr) + c);
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] += __uint_as_float(w[i] << 16);
                acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(y + static_cast<long long>(t) * hidden)[c] = o;
    }
}

// ==================================================================================================================
// Expert-parallel dispatch: ranks own contiguous blocks of experts (expert e lives on rank e / experts_per_rank, as
// in the reference: deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:372,389). Every rank holds one
// buffer with the same layout; `peers[r]` is the address of rank r's buffer as mapped into this process.
// Protocol of one layer call (all ranks in lockstep, each phase a kernel on the caller's stream):
//   count  -> per-chunk histogram of this rank's entries over ALL experts
//   share  -> per expert: this rank's entry count, written into every rank's all_counts[this rank][expert]
//   barrier
//   plan   -> every rank derives the same global layout from all_counts: rows of expert e on its owner are ordered
//             by (source rank, entry), segments padded to `alignment`
//   push   -> each entry's FP8 row, packed scales, routing weight and source id are stored straight into the owner's
//             expert-sorted buffers (P2P stores; the reference pulls instead, :461-599)
//   barrier -> L1 GEMM -> L2 GEMM (epilogue stores rows into the source rank's combine slots) -> barrier -> combine
// ==================================================================================================================

// One CTA. chunk_hist[chunk][e] (counts) -> exclusive bases over chunks; per-expert totals go to all ranks.
__global__ void __launch_bounds__(1024)
dgb200_ep_share_counts_kernel(int* __restrict__ chunk_hist, int num_chunks, int num_experts, int my_rank, int num_ranks,
                              const PeerTable peers, long long all_counts_offset) {
    pdl_prologue();
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        int count = 0;
        for (int c = 0; c < num_chunks; ++c) {
            int* slot = chunk_hist + static_cast<long long>(c) * num_experts + e;
            const int t = *slot;
            *slot = count;
            count += t;
        }
        for (int r = 0; r < num_ranks; ++r) {
            int* dst = reinterpret_cast<int*>(peers.p[r] + all_counts_offset) + static_cast<long long>(my_rank) * num_experts + e;
            *dst = count;
        }
    }
}

// Cross-rank flags of the expert-parallel layer. The flags region of the buffer is int [kEpFlagRows][kMaxEpRanks]:
//   rows 0 .. kEpFlagRows - 5:  flag rows; slot s holds the epoch rank s last signalled on that row
//   rows kEpFlagRows - 4, - 3:  this rank's own count of signals sent per flag row (word = row)
//   rows kEpFlagRows - 2, - 1:  this rank's own count of waits completed per flag row
// Rows: 0 = "my per-expert counts are published"; 1 + q = "my rows for expert phase q are pushed" (dispatch);
// 1 + kMaxEpPhases + q = "my experts of phase q have their outputs ready" (combine). All ranks make the same sequence of
// calls, so the n-th wait on a row pairs with every rank's n-th signal on it: the epochs live and die with the buffer
// (zeroed once when the buffer is created, on every rank, before the first call), a replayed launch advances them like
// a fresh one, and flags only grow, so nothing ever needs a reset. One warp; lane s signals rank s and / or waits for
// rank s. Bounded: a peer that does not show up within the budget is reported through the status block (peer timeout,
// detail = the rank), not waited for forever.
constexpr int kMaxEpPhases = 4;
constexpr int kEpFlagRows = 1 + 2 * kMaxEpPhases + 4;  // 9 flag rows, then 2 + 2 rows of this rank's own counters

__global__ void __launch_bounds__(32)
dgb200_ep_flag_kernel(const PeerTable peers, long long flags_offset, int row, int my_rank, int num_ranks, int do_signal,
                      int do_wait, long long budget_cycles) {
    pdl_prologue();
    const int lane = threadIdx.x;
    int* local = reinterpret_cast<int*>(peers.p[my_rank] + flags_offset);
    int* sent = local + (kEpFlagRows - 4) * kMaxEpRanks + row;
    int* waited = local + (kEpFlagRows - 2) * kMaxEpRanks + row;
    if (do_signal) {
        int epoch = 0;
        if (lane == 0) {
            epoch = *sent + 1;
            *sent = epoch;
        }
        epoch = __shfl_sync(0xffffffffu, epoch, 0);
        __threadfence_system();  // everything this rank stored before (to any rank) is visible before the flag
        if (lane < num_ranks) {
            int* remote = reinterpret_cast<int*>(peers.p[lane] + flags_offset) + row * kMaxEpRanks + my_rank;
            asm volatile("st.release.sys.global.s32 [%0], %1;" :: "l"(remote), "r"(epoch) : "memory");
        }
    }
    if (do_wait) {
        int epoch = 0;
        if (lane == 0) {
            epoch = *waited + 1;
            *waited = epoch;
        }
        epoch = __shfl_sync(0xffffffffu, epoch, 0);
        if (lane < num_ranks) {
            const int* mine = local + row * kMaxEpRanks + lane;
            const long long t0 = clock64();
            while (true) {
                int seen;
                asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
                if (seen - epoch >= 0) break;
                if (clock64() - t0 > budget_cycles) {
                    report_error(kTimeoutPeer, lane, seen);
                    break;
                }
                __nanosleep(100);
            }
        }
        __threadfence_system();
    }
}

// One CTA. From all_counts[source rank][expert] derives, identically on every rank:
//   my_base[e]   first row, on the owner of expert e, of THIS rank's entries for e
//   expert_start / expert_end for the local experts (the psum layout the local GEMMs walk), total_rows, stats.
__global__ void __launch_bounds__(1024)
dgb200_ep_plan_kernel(const int* __restrict__ all_counts, int num_experts, int num_ranks, int my_rank, int alignment,
                      int* __restrict__ my_base, int* __restrict__ expert_start, int* __restrict__ expert_end,
                      int* __restrict__ total_rows, int* __restrict__ cumulative_stats) {
    pdl_prologue();
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int per_rank = num_experts / num_ranks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int owner = 0; owner < num_ranks; ++owner) {
        if (threadIdx.x == 0) carry = 0;
        __syncthreads();
        for (int base = 0; base < per_rank; base += 1024) {
            const int local = base + static_cast<int>(threadIdx.x);
            const int e = owner * per_rank + local;
            int total = 0, before_me = 0;
            if (local < per_rank) {
                for (int s = 0; s < num_ranks; ++s) {
                    const int c = all_counts[static_cast<long long>(s) * num_experts + e];
                    if (s < my_rank) before_me += c;
                    total += c;
                }
            }
            const int padded = (total + alignment - 1) / alignment * alignment;
            int incl = padded;
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += n;
            }
            if (lane == 31) warp_sums[warp] = incl;
            __syncthreads();
            if (warp == 0) {
                int w = warp_sums[lane];
                for (int off = 1; off < 32; off <<= 1) {
                    const int n = __shfl_up_sync(0xffffffffu, w, off);
                    if (lane >= off) w += n;
                }
                warp_sums[lane] = w;
            }
            __syncthreads();
            const int start = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - padded;
            if (local < per_rank) {
                my_base[e] = start + before_me;
                if (owner == my_rank) {
                    expert_start[local] = start;
                    expert_end[local] = start + total;
                    if (cumulative_stats != nullptr) cumulative_stats[local] += total;
                }
            }
            __syncthreads();
            if (threadIdx.x == 1023) carry = start + padded;
            __syncthreads();
        }
        if (owner == my_rank && threadIdx.x == 0) total_rows[0] = carry;
        __syncthreads();
    }
}

// The combine of the expert-parallel layer, one phase of the local experts at a time: phase q adds, for every token, the
// rows of the slots whose expert (numbered within its owner) lies in [local_expert_begin, local_expert_end), read in
// place from the owners over NVLink. The running sum of a token is kept in FP32 in `partial` ([tokens, hidden]) between
// phases: the first phase starts from zero (or from the shared experts' row), the last one writes bf16 y. The rows of a
// phase can be pulled as soon as every rank has finished that phase's experts, while later phases are still being
// computed; within a phase the slots are added in ascending order. Tokens without a slot in a middle phase are skipped.
__global__ void __launch_bounds__(128)
dgb200_moe_combine_phase_kernel(const PeerTable peers, long long rows_offset, const long long* __restrict__ topk_idx,
                                const int* __restrict__ dest_row, int topk, int experts_per_rank, int hidden,
                                const __nv_bfloat16* __restrict__ shared_rows, float* __restrict__ partial,
                                __nv_bfloat16* __restrict__ y, int local_expert_begin, int local_expert_end, int first, int last,
                                const int* __restrict__ my_dest, const int* __restrict__ my_slot) {
    pdl_prologue();
    const int t = blockIdx.x;
    extern __shared__ unsigned long long slot_rows[];  // address of each slot's row of this phase, 0 = skip
    __shared__ int any;
    if (threadIdx.x == 0) any = 0;
    __syncthreads();
    if (threadIdx.x < topk) {
        const int d = dest_row[static_cast<long long>(t) * topk + threadIdx.x];
        unsigned long long addr = 0;
        if (d >= 0) {
            const int e = static_cast<int>(topk_idx[static_cast<long long>(t) * topk + threadIdx.x]);
            // computing rank and expert slot: the owner and the expert's index there, or what the spill plan says
            const int owner = my_dest != nullptr ? my_dest[e] : e / experts_per_rank;
            const int local_expert = my_slot != nullptr ? my_slot[e] : e - owner * experts_per_rank;
            if (local_expert >= local_expert_begin && local_expert < local_expert_end) {
                addr = peers.p[owner] + rows_offset + static_cast<unsigned long long>(d) * hidden * 2;
                any = 1;
            }
        }
        slot_rows[threadIdx.x] = addr;
    }
    __syncthreads();
    if (!any && !first && !last) return;
    float* part = partial + static_cast<long long>(t) * hidden;
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (!first) {
            const float4 a = reinterpret_cast<const float4*>(part)[2 * c], b = reinterpret_cast<const float4*>(part)[2 * c + 1];
            acc[0] = a.x; acc[1] = a.y; acc[2] = a.z; acc[3] = a.w; acc[4] = b.x; acc[5] = b.y; acc[6] = b.z; acc[7] = b.w;
        }
        for (int k = 0; k < topk; ++k) {
            const unsigned long long addr = slot_rows[k];
            if (addr == 0) continue;
            const uint4 v = ld_global_nc_v4(reinterpret_cast<const uint4*>(addr) + c);
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] += __uint_as_float(w[i] << 16);
                acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
        }
        if (last) {
            if (shared_rows != nullptr) {  // the shared experts' row is the slot after the top-k ones
                const uint4 v = ld_global_nc_v4(reinterpret_cast<const uint4*>(shared_rows + static_cast<long long>(t) * hidden) + c);
                const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] += __uint_as_float(w[i] << 16);
                    acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
                }
            }
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]);
            o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]);
            o.w = pack_bf16x2(acc[6], acc[7]);
            reinterpret_cast<uint4*>(y + static_cast<long long>(t) * hidden)[c] = o;
        } else {
            reinterpret_cast<float4*>(part)[2 * c] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            reinterpret_cast<float4*>(part)[2 * c + 1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
    }
}

// ---- hot-expert row spill -------------------------------------------------------------------------------------------------
// With skewed routing the rank that owns the popular experts receives several times the mean number of rows and every
// other rank waits for it. Each rank therefore keeps kMaxGuestExperts spare expert slots after its own experts, and the
// plan may move the rows that some source ranks route to a hot expert onto a less loaded rank, which computes them in a
// guest slot with a copy of the expert's weights fetched from the owner (dgb200_ep_fetch_guest_weights_kernel). A row's
// arithmetic does not depend on the rank that computes it, so the layer's output is the same bits as without the spill.
// No reference counterpart: the reference keeps every expert's rows on its owner (sm100_fp8_fp4_mega_moe.cuh:372,389).
constexpr int kMaxGuestExperts = 8;
constexpr int kMaxSpillSlots = 256;  // expert slots per rank (own + guest) the plan's tables index with one byte

// One CTA. The spill table and this rank's plan under it, derived identically on every rank from
// all_counts[source rank][expert] with integer arithmetic only:
//   load[r] = rows of the experts r owns; repeat at most ranks * guest_slots times:
//     hi = the most loaded rank, lo = the least loaded rank other than hi with a free guest slot (ties: lower rank);
//     gap = load[hi] - load[lo]; stop when gap < max(256, total rows / (32 * ranks));
//     e = the expert owned by hi with the most rows still on hi (ties: lower e); stop when it has none;
//     walk the source ranks from the last to the first: the rows (s, e) still on hi move to lo while
//     2 * moved + count[s][e] < gap; stop when nothing moved; lo hosts e in the guest slot it already has for e, else in
//     its next free one.
// Outputs: my_base / my_dest / my_slot [experts]: first row, computing rank and expert slot there of THIS rank's entries
// for e; slot_start / slot_end [per_rank + guest_slots]: this rank's own segments (the psum layout its GEMMs walk), each
// padded to `alignment`, rows inside a slot ordered by (source rank, entry); total_rows; guest_expert [guest_slots]:
// the experts this rank hosts (-1 = unused); rank_rows [2][ranks]: every rank's rows before and after the spill.
// Dynamic shared memory: the counts (ranks * experts ints) and the two byte tables (2 * ranks * experts bytes).
__global__ void __launch_bounds__(1024)
dgb200_ep_spill_plan_kernel(const int* __restrict__ all_counts, int num_experts, int num_ranks, int my_rank, int alignment,
                            int guest_slots, int* __restrict__ my_base, int* __restrict__ my_dest, int* __restrict__ my_slot,
                            int* __restrict__ slot_start, int* __restrict__ slot_end, int* __restrict__ total_rows,
                            int* __restrict__ guest_expert, int* __restrict__ rank_rows, int* __restrict__ cumulative_stats) {
    pdl_prologue();
    extern __shared__ int spill_smem[];
    int* counts = spill_smem;                                                              // [ranks][experts]
    unsigned char* dest = reinterpret_cast<unsigned char*>(counts + num_ranks * num_experts);  // [experts][ranks]
    unsigned char* slot = dest + num_ranks * num_experts;                                  // [experts][ranks]
    __shared__ int rows_of[kMaxEpRanks * kMaxSpillSlots];   // rows per (rank, slot), then the slot's first row
    __shared__ int rows_cnt[kMaxEpRanks * kMaxSpillSlots];
    __shared__ int load[kMaxEpRanks], used[kMaxEpRanks], guest[kMaxEpRanks][kMaxGuestExperts];
    __shared__ int total_all;
    const int per_rank = num_experts / num_ranks;
    const int slots = per_rank + guest_slots;
    const int tid = static_cast<int>(threadIdx.x), lane = tid & 31;

    for (int i = tid; i < num_ranks * num_experts; i += blockDim.x) {
        counts[i] = all_counts[i];
        const int e = i / num_ranks, s = i - e * num_ranks;
        dest[e * num_ranks + s] = static_cast<unsigned char>(e / per_rank);
        slot[e * num_ranks + s] = static_cast<unsigned char>(e % per_rank);
    }
    if (tid < kMaxEpRanks) {
        used[tid] = 0;
        for (int g = 0; g < kMaxGuestExperts; ++g) guest[tid][g] = -1;
    }
    __syncthreads();
    if (tid < num_ranks) {
        int sum = 0;
        for (int e = tid * per_rank; e < (tid + 1) * per_rank; ++e)
            for (int s = 0; s < num_ranks; ++s) sum += counts[s * num_experts + e];
        load[tid] = sum;
        rank_rows[tid] = sum;
    }
    __syncthreads();
    if (tid == 0) {
        int sum = 0;
        for (int r = 0; r < num_ranks; ++r) sum += load[r];
        total_all = sum;
    }
    __syncthreads();

    if (tid < 32 && guest_slots > 0) {  // the greedy moves, one warp
        const int min_gap = max(256, total_all / (32 * num_ranks));
        for (int iter = 0; iter < num_ranks * guest_slots; ++iter) {
            int hi = 0, lo = -1;
            for (int r = 1; r < num_ranks; ++r)
                if (load[r] > load[hi]) hi = r;
            for (int r = 0; r < num_ranks; ++r)
                if (r != hi && used[r] < guest_slots && (lo < 0 || load[r] < load[lo])) lo = r;
            if (lo < 0) break;
            const int gap = load[hi] - load[lo];
            if (gap < min_gap) break;
            // the expert of hi with the most rows still on hi, ties to the lower expert
            int best_rows = -1, best_e = 0x7fffffff;
            for (int local = lane; local < per_rank; local += 32) {
                const int e = hi * per_rank + local;
                int v = 0;
                for (int s = 0; s < num_ranks; ++s)
                    if (dest[e * num_ranks + s] == hi) v += counts[s * num_experts + e];
                if (v > best_rows) { best_rows = v; best_e = e; }
            }
            for (int off = 16; off > 0; off >>= 1) {
                const int r2 = __shfl_xor_sync(0xffffffffu, best_rows, off), e2 = __shfl_xor_sync(0xffffffffu, best_e, off);
                if (r2 > best_rows || (r2 == best_rows && e2 < best_e)) { best_rows = r2; best_e = e2; }
            }
            if (best_rows <= 0) break;
            int moved = 0;
            if (lane == 0) {
                const int e = best_e;
                int g = -1;
                for (int i = 0; i < used[lo]; ++i)
                    if (guest[lo][i] == e) g = i;
                const bool hosted = g >= 0;
                if (!hosted) g = used[lo];
                for (int s = num_ranks - 1; s >= 0; --s) {
                    const int c = counts[s * num_experts + e];
                    if (c > 0 && dest[e * num_ranks + s] == hi && 2 * moved + c < gap) {
                        dest[e * num_ranks + s] = static_cast<unsigned char>(lo);
                        slot[e * num_ranks + s] = static_cast<unsigned char>(per_rank + g);
                        moved += c;
                    }
                }
                if (moved > 0) {
                    if (!hosted) { guest[lo][g] = e; used[lo] += 1; }
                    load[hi] -= moved;
                    load[lo] += moved;
                }
            }
            moved = __shfl_sync(0xffffffffu, moved, 0);
            __syncwarp();
            if (moved == 0) break;
        }
    }
    __syncthreads();

    // rows per (rank, slot), then each rank's segment starts
    for (int i = tid; i < num_ranks * kMaxSpillSlots; i += blockDim.x) rows_cnt[i] = 0;
    __syncthreads();
    for (int i = tid; i < num_ranks * num_experts; i += blockDim.x) {
        const int e = i / num_ranks, s = i - e * num_ranks;
        const int c = counts[s * num_experts + e];
        if (c > 0) atomicAdd(&rows_cnt[dest[i] * kMaxSpillSlots + slot[i]], c);
    }
    __syncthreads();
    if (tid < num_ranks) {
        int cursor = 0;
        for (int v = 0; v < slots; ++v) {
            rows_of[tid * kMaxSpillSlots + v] = cursor;
            cursor = (cursor + rows_cnt[tid * kMaxSpillSlots + v] + alignment - 1) / alignment * alignment;
        }
        rank_rows[num_ranks + tid] = load[tid];
        if (tid == my_rank) total_rows[0] = cursor;
    }
    __syncthreads();
    for (int e = tid; e < num_experts; e += blockDim.x) {
        const int d = dest[e * num_ranks + my_rank], v = slot[e * num_ranks + my_rank];
        int before = 0, total = 0;
        for (int s = 0; s < num_ranks; ++s) {
            const int c = counts[s * num_experts + e];
            if (s < my_rank && dest[e * num_ranks + s] == d) before += c;
            total += c;
        }
        my_base[e] = rows_of[d * kMaxSpillSlots + v] + before;
        my_dest[e] = d;
        my_slot[e] = v;
        if (cumulative_stats != nullptr && e / per_rank == my_rank) cumulative_stats[e - my_rank * per_rank] += total;
    }
    for (int v = tid; v < slots; v += blockDim.x) {
        slot_start[v] = rows_of[my_rank * kMaxSpillSlots + v];
        slot_end[v] = rows_of[my_rank * kMaxSpillSlots + v] + rows_cnt[my_rank * kMaxSpillSlots + v];
    }
    if (tid < guest_slots) guest_expert[tid] = guest[my_rank][tid];
}

// Copies the weights of the experts this rank hosts in its guest slots from their owners: four tensors per expert
// (gate/up weights, their scales, down weights, their scales), `bytes[i]` each, expert-major on every rank with the
// guest slots after the rank's own experts. gridDim.y = guest slots; the CTAs of a row share the expert's bytes.
struct GuestWeightTables {
    unsigned long long peer[4][kMaxEpRanks];  // base address of tensor i on every rank, as mapped into this process
    unsigned long long local[4];              // the same tensors of this rank
    long long bytes[4];                       // bytes of one expert in tensor i (multiples of 16)
};
__global__ void __launch_bounds__(256)
dgb200_ep_fetch_guest_weights_kernel(const int* __restrict__ guest_expert, int experts_per_rank, const GuestWeightTables t) {
    pdl_prologue();
    const int e = guest_expert[blockIdx.y];
    if (e < 0) return;
    const int owner = e / experts_per_rank, local_expert = e - owner * experts_per_rank;
    const long long slot_index = experts_per_rank + static_cast<long long>(blockIdx.y);
#pragma unroll 1
    for (int i = 0; i < 4; ++i) {
        const uint4* from = reinterpret_cast<const uint4*>(t.peer[i][owner] + static_cast<unsigned long long>(local_expert * t.bytes[i]));
        uint4* to = reinterpret_cast<uint4*>(t.local[i] + static_cast<unsigned long long>(slot_index * t.bytes[i]));
        const long long vecs = t.bytes[i] / 16;
        const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
        long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
        for (; c + 3 * stride < vecs; c += 4 * stride) {  // four independent loads in flight per thread
            const uint4 v0 = ld_global_nc_v4(from + c), v1 = ld_global_nc_v4(from + c + stride);
            const uint4 v2 = ld_global_nc_v4(from + c + 2 * stride), v3 = ld_global_nc_v4(from + c + 3 * stride);
            to[c] = v0;
            to[c + stride] = v1;
            to[c + 2 * stride] = v2;
            to[c + 3 * stride] = v3;
        }
        for (; c < vecs; c += stride) to[c] = ld_global_nc_v4(from + c);
    }
}

// dest_row[entry] = row on the owner rank (my_base[e] + stable rank of the entry among this rank's entries for e).
__global__ void __launch_bounds__(kPlanChunk)
dgb200_ep_assign_kernel(const long long* __restrict__ topk_idx, int num_entries, int num_experts,
                        const int* __restrict__ chunk_hist, const int* __restrict__ my_base, int* __restrict__ dest_row) {
    pdl_prologue();
    extern __shared__ unsigned char warp_hist[];  // [32 warps][num_experts]
    for (int i = threadIdx.x; i < 32 * num_experts; i += blockDim.x) warp_hist[i] = 0;
    __syncthreads();
    const int i = blockIdx.x * kPlanChunk + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int e = -1;
    if (i < num_entries) {
        const long long g = topk_idx[i];
        if (g >= 0 && g < num_experts) e = static_cast<int>(g);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_hist[warp * num_experts + e] = static_cast<unsigned char>(__popc(peers));
    __syncthreads();
    if (i >= num_entries) return;
    if (e < 0) {
        dest_row[i] = -1;
        return;
    }
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_hist[w * num_experts + e];
    dest_row[i] = my_base[e] + chunk_hist[static_cast<long long>(blockIdx.x) * num_experts + e] + before + rank_in_warp;
}

// Entry lists of the dispatch that rides on the gate/up GEMMs (GemmParams::push): every valid entry (token, k) of this
// rank whose expert slot belongs to phase q >= 1 is appended to list q (any order: an entry's destination row is fixed
// by the plan). Phase 0 is sent by dgb200_ep_push_kernel before the first GEMM. counts must be zero on entry.
__global__ void __launch_bounds__(256)
dgb200_ep_phase_lists_kernel(const long long* __restrict__ topk_idx, const int* __restrict__ dest_row, int num_entries,
                             int experts_per_rank, const int* __restrict__ my_slot, int num_phases, int num_slots,
                             int* __restrict__ lists, int list_stride, int* __restrict__ counts) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_entries || dest_row[i] < 0) return;
    const int expert = static_cast<int>(topk_idx[i]);
    const int slot = my_slot != nullptr ? my_slot[expert] : expert % experts_per_rank;
    int phase = 0;
    while (phase + 1 < num_phases && slot >= static_cast<int>(static_cast<long long>(phase + 1) * num_slots / num_phases)) ++phase;
    if (phase == 0) return;
    lists[static_cast<long long>(phase) * list_stride + atomicAdd(&counts[phase], 1)] = i;
}

// ---- rows between ranks through the bulk-copy unit --------------------------------------------------------------------------
// The kernels that move rows between ranks (dispatch push, return push) read local memory and write a peer's. While GEMMs
// hold most SMs they run on a handful of SMs, so what they move is bounded by the bytes each SM keeps in flight: every
// warp owns one row-sized slot of shared memory and one mbarrier, and its first lane copies a row as
//   cp.async.bulk global -> slot (completes on the mbarrier) ; cp.async.bulk slot -> peer global (bulk group),
// so a CTA has one row per warp in flight (some 200 KB per SM) without holding it in registers. Every wait is bounded.
constexpr int kRowMoverMaxWarps = 32;
constexpr int kRowMoverSmemBudget = 216 * 1024;

struct RowMover {
    uint32_t slot;        // shared-memory address of this warp's slot
    uint64_t* bar;        // its mbarrier
    uint32_t parity;      // phase the next load completes
    volatile uint32_t* abort_flag;
};

// Shared-memory carve-up of a row-moving CTA: [warps] mbarriers, then [warps] slots of slot_bytes (16-byte multiples).
__device__ __forceinline__ RowMover row_mover_init(unsigned char* smem, int slot_bytes, volatile uint32_t* abort_flag) {
    const int warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    if (threadIdx.x == 0) *abort_flag = 0;
    if ((threadIdx.x & 31) == 0) mbar_init(&bars[warp], 1);
    fence_mbar_init();
    __syncthreads();
    RowMover m;
    m.bar = &bars[warp];
    m.slot = smem_u32(smem + ((warps * 8 + 15) / 16 * 16) + static_cast<long long>(warp) * slot_bytes);
    m.parity = 0;
    m.abort_flag = abort_flag;
    return m;
}

// Called by lane 0 of a warp: copies bytes0 from src0 to dst0 and (bytes1 > 0) bytes1 from src1 to dst1 through the warp's
// slot. Returns false when a wait ran out (recorded in the status block).
__device__ __forceinline__ bool row_mover_copy(RowMover& m, const void* src0, void* dst0, uint32_t bytes0, const void* src1, void* dst1,
                                               uint32_t bytes1) {
    bulk_wait_group_read_all();  // the store that last used the slot has read it
    mbar_arrive_expect_tx(m.bar, bytes0 + bytes1);
    bulk_load_1d(m.slot, src0, bytes0, m.bar);
    if (bytes1 > 0) bulk_load_1d(m.slot + bytes0, src1, bytes1, m.bar);
    if (!mbar_wait(m.bar, m.parity, m.abort_flag, kTimeoutRowMover, static_cast<int>(blockIdx.x))) return false;
    m.parity ^= 1u;
    bulk_store_1d(dst0, m.slot, bytes0);
    if (bytes1 > 0) bulk_store_1d(dst1, m.slot + bytes0, bytes1);
    bulk_commit_group();
    return true;
}

// Dispatch push of the expert-parallel layer: every entry (token, k) of this rank whose expert slot lies in
// [local_expert_begin, local_expert_end) is stored into the buffers of the rank that computes it: the token's quantised
// row and its packed scale ints (row-major staging area of the receiver, which brings them into GEMM order itself: one
// 4-byte remote store per scale int, each in another cache line, cost 40 % of the push), the routing weight and the
// source id. A warp examines 32 entries at a time (one per lane), then its first lane moves the rows of those that
// belong to the phase one after the other, so a launch that pushes one phase of the experts skips the other entries
// cheaply. Any grid; dynamic shared memory: row_mover_smem_bytes(warps, row_bytes + 4 * sf_per_row) or more.
__global__ void __launch_bounds__(1024)
dgb200_ep_push_kernel(const unsigned char* __restrict__ x, const unsigned* __restrict__ x_sf,
                      const long long* __restrict__ topk_idx, const float* __restrict__ topk_weights,
                      const int* __restrict__ dest_row, int num_entries, int topk, int row_bytes, int sf_per_row,
                      int experts_per_rank, int my_rank, int entries_per_rank, const PeerTable peers,
                      long long acts_offset, long long sf_offset, long long weight_offset,
                      long long src_offset, int local_expert_begin, int local_expert_end,
                      const int* __restrict__ my_dest, const int* __restrict__ my_slot) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char mover_smem[];
    __shared__ uint32_t abort_flag;
    const int sf_bytes = sf_per_row * 4;
    const int bulk_sf_bytes = sf_bytes % 16 == 0 ? sf_bytes : 0;  // a bulk copy moves multiples of 16 bytes; else plain stores
    RowMover mover = row_mover_init(mover_smem, row_bytes + bulk_sf_bytes, &abort_flag);
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int num_warps = gridDim.x * warps_per_cta;
    bool ok = true;
    for (int first = (blockIdx.x * warps_per_cta + (threadIdx.x >> 5)) * 32; first < num_entries && ok; first += num_warps * 32) {
        int my_row = -1, my_owner = 0;
        if (first + lane < num_entries) {
            my_row = dest_row[first + lane];
            if (my_row >= 0) {
                // the rank that computes this entry and the expert slot there: the expert's owner and its index among the
                // owner's experts, unless the plan spilled the rows this rank routes to the expert (my_dest / my_slot)
                const int expert = static_cast<int>(topk_idx[first + lane]);
                my_owner = my_dest != nullptr ? my_dest[expert] : expert / experts_per_rank;
                const int local_expert = my_slot != nullptr ? my_slot[expert] : expert - my_owner * experts_per_rank;
                if (local_expert < local_expert_begin || local_expert >= local_expert_end) my_row = -1;
            }
        }
        unsigned todo = __ballot_sync(0xffffffffu, my_row >= 0);
        while (todo != 0 && ok) {
            const int src_lane = __ffs(todo) - 1;
            todo &= todo - 1;
            const int entry = first + src_lane;
            const int dest = __shfl_sync(0xffffffffu, my_row, src_lane);
            const int owner = __shfl_sync(0xffffffffu, my_owner, src_lane);
            if (lane == 0) {
                const int token = entry / topk;
                const unsigned long long base = peers.p[owner];
                ok = row_mover_copy(mover, x + static_cast<long long>(token) * row_bytes,
                                    reinterpret_cast<void*>(base + acts_offset + static_cast<long long>(dest) * row_bytes),
                                    static_cast<uint32_t>(row_bytes), x_sf + static_cast<long long>(token) * sf_per_row,
                                    reinterpret_cast<void*>(base + sf_offset + static_cast<long long>(dest) * sf_bytes),
                                    static_cast<uint32_t>(bulk_sf_bytes));
                if (bulk_sf_bytes == 0)
                    for (int c = 0; c < sf_per_row; ++c)
                        reinterpret_cast<unsigned*>(base + sf_offset)[static_cast<long long>(dest) * sf_per_row + c] =
                            x_sf[static_cast<long long>(token) * sf_per_row + c];
                reinterpret_cast<float*>(base + weight_offset)[dest] = topk_weights[entry];
                reinterpret_cast<int*>(base + src_offset)[dest] = my_rank * entries_per_rank + entry;
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
    }
    if (lane == 0) bulk_wait_group_all();  // this warp's stores are complete before the kernel ends
}

// Return push of the expert-parallel layer: the BF16 output rows of the expert slots [slot_begin, slot_end) of this rank
// go back to the ranks their tokens came from, row `entry` of the receiver's `returned` buffer ([entries per rank, hidden]
// bf16; src_of_row[r] = source rank * entries_per_rank + entry, written by the dispatch push). A warp per row, rows of
// the slots dealt round-robin to the grid's warps. The receiver sums a token's rows itself once all of them have arrived
// (dgb200_moe_combine_returned_kernel). Dynamic shared memory as for the dispatch push, slot = one row.
__global__ void __launch_bounds__(1024)
dgb200_ep_return_rows_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ src_of_row,
                             const int* __restrict__ slot_start, const int* __restrict__ slot_end_rows, int slot_begin,
                             int slot_end, int hidden, int entries_per_rank, const PeerTable peers, long long returned_offset) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char mover_smem[];
    __shared__ uint32_t abort_flag;
    const int row_bytes = hidden * 2;
    RowMover mover = row_mover_init(mover_smem, row_bytes, &abort_flag);
    if ((threadIdx.x & 31) != 0) return;  // one lane per warp drives the copies
    const int warps_per_cta = blockDim.x >> 5;
    const int num_warps = gridDim.x * warps_per_cta;
    const int warp = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    bool ok = true;
    for (int v = slot_begin; v < slot_end && ok; ++v) {
        const int end = slot_end_rows[v];
        for (int r = slot_start[v] + warp; r < end && ok; r += num_warps) {
            const int src = src_of_row[r];
            const int rank = src / entries_per_rank, entry = src - rank * entries_per_rank;
            // a row whose push never arrived (a rank that timed out) carries a stale source id: skip what cannot be a rank
            if (src < 0 || rank >= kMaxEpRanks || peers.p[rank] == 0) continue;
            ok = row_mover_copy(mover, rows + static_cast<long long>(r) * hidden,
                                reinterpret_cast<void*>(peers.p[rank] + returned_offset + static_cast<long long>(entry) * row_bytes),
                                static_cast<uint32_t>(row_bytes), nullptr, nullptr, 0u);
        }
    }
    bulk_wait_group_all();
}

// y[t, :] = bf16( sum over valid k, in ascending k, of float(returned[t * topk + k, :]) ) (+ the shared experts' row of the
// token as one more slot): the combine over rows that dgb200_ep_return_rows_kernel of every computing rank stored into
// this rank's `returned` buffer. Slots with dest_row < 0 (masked) are skipped. One CTA per token, a thread owns 8
// consecutive channels; the same order of additions as the single-rank combine.
__global__ void __launch_bounds__(128)
dgb200_moe_combine_returned_kernel(const __nv_bfloat16* __restrict__ returned, const int* __restrict__ dest_row, int topk,
                                   int hidden, const __nv_bfloat16* __restrict__ shared_rows, __nv_bfloat16* __restrict__ y) {
    pdl_prologue();
    const int t = blockIdx.x;
    __shared__ int valid[32];
    if (threadIdx.x < 32) valid[threadIdx.x] = static_cast<int>(threadIdx.x) < topk && dest_row[static_cast<long long>(t) * topk + threadIdx.x] >= 0;
    __syncthreads();
    for (int c = threadIdx.x; c < hidden / 8; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k <= topk; ++k) {
            const __nv_bfloat16* row;
            if (k < topk) {
                if (!valid[k]) continue;
                row = returned + (static_cast<long long>(t) * topk + k) * hidden;
            } else {
                if (shared_rows == nullptr) continue;
                row = shared_rows + static_cast<long long>(t) * hidden;
            }
            const uint4 v = ld_global_nc_v4(reinterpret_cast<const uint4*>(row) + c);
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] += __uint_as_float(w[i] << 16);
                acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
            }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(y + static_cast<long long>(t) * hidden)[c] = o;
    }
}

// Fused activation quantisation + dispatch (the step the reference leaves to torch ops before its layer call,
// README.md:72: per_token_cast_to_fp8 into the buffer, then the in-kernel dispatch pull): one warp per token reads the
// BF16 row once, quantises it to E4M3 with one UE8M0 scale per 32 elements (the arithmetic of
// dgb200_cast_rows_kernel<false>, i.e. per_token_cast_to_fp8(use_ue8m0=True, gran_k=32)) and writes row and packed
// scales straight into each of its top-k destination rows of the expert-sorted buffers, on this rank or a peer.
// `write_meta` also stores the routing weight and the source entry next to the row (the expert-parallel push does
// that; on a single rank the plan kernels already have).
__global__ void __launch_bounds__(256)
dgb200_moe_quant_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long x_row_stride,
                                 const long long* __restrict__ topk_idx, const float* __restrict__ topk_weights,
                                 const int* __restrict__ dest_row, int tokens, int topk, int hidden, int experts_per_rank,
                                 int my_rank, int entries_per_rank, const PeerTable peers, long long acts_offset,
                                 long long sf_offset, long long sf_k_stride, long long weight_offset, long long src_offset,
                                 int write_meta, unsigned char* __restrict__ self_q, unsigned* __restrict__ self_sf,
                                 long long self_sf_k_stride) {
    pdl_prologue();
    // self_q / self_sf (may be null): also keep the quantised row in token order (e4m3 [tokens, hidden]; scales MN-major
    // in tcgen05.cp row order), which is what the shared experts' GEMM reads.
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (token >= tokens) return;
    int my_dest = -1;
    unsigned long long my_base = 0;
    if (lane < topk) {
        const int entry = token * topk + lane;
        const int d = dest_row[entry];
        if (d >= 0) {
            my_dest = d;
            my_base = peers.p[static_cast<int>(topk_idx[entry]) / experts_per_rank];
            if (write_meta) {
                reinterpret_cast<float*>(my_base + weight_offset)[d] = topk_weights[entry];
                reinterpret_cast<int*>(my_base + src_offset)[d] = my_rank * entries_per_rank + entry;
            }
        }
    }
    const __nv_bfloat16* row = x + static_cast<long long>(token) * x_row_stride;
    for (int col0 = 0; col0 < hidden; col0 += 512) {
        const int col = col0 + lane * 16;
        const bool valid = col < hidden;  // hidden is a multiple of 128
        float v[16];
        if (valid) {
            const uint4* src = reinterpret_cast<const uint4*>(row + col);
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
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));  // two lanes share a 32-element scale group
        const uint32_t e = ue8m0_ceil_bits(fmaxf(amax, 1e-4f) / 448.0f);
        const float inv = 1.0f / __uint_as_float(e << 23);
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_fp8x4_e4m3 q4(make_float4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv));
            o[i] = q4.__x;
        }
        // packed scale int of 128 elements = the scale bytes of lanes L, L + 2, L + 4, L + 6 (L a multiple of 8)
        const uint32_t e2 = __shfl_down_sync(0xffffffffu, e, 2), e4 = __shfl_down_sync(0xffffffffu, e, 4),
                       e6 = __shfl_down_sync(0xffffffffu, e, 6);
        const uint32_t sf_int = e | (e2 << 8) | (e4 << 16) | (e6 << 24);
        if (self_q != nullptr && valid) {
            st_global_v4(self_q + static_cast<long long>(token) * hidden + col, o[0], o[1], o[2], o[3]);
            if ((lane & 7) == 0) self_sf[static_cast<long long>(col >> 7) * self_sf_k_stride + sf_row_in_cp_order(token)] = sf_int;
        }
        for (int k = 0; k < topk; ++k) {
            const int d = __shfl_sync(0xffffffffu, my_dest, k);
            const unsigned long long base = __shfl_sync(0xffffffffu, my_base, k);
            if (d < 0 || !valid) continue;
            st_global_v4(reinterpret_cast<unsigned char*>(base + acts_offset) + static_cast<long long>(d) * hidden + col, o[0], o[1],
                         o[2], o[3]);
            if ((lane & 7) == 0) {
                unsigned* sf = reinterpret_cast<unsigned*>(base + sf_offset);
                if (sf_k_stride > 0)
                    sf[static_cast<long long>(col >> 7) * sf_k_stride + sf_row_in_cp_order(d)] = sf_int;
                else  // row-major staging (see dgb200_ep_push_kernel): -sf_k_stride ints per row
                    sf[static_cast<long long>(d) * (-sf_k_stride) + (col >> 7)] = sf_int;
            }
        }
    }
}

// The same fusion for the NVFP4 layer on a single rank: one warp per token reads the BF16 row once, quantises it to packed
// E2M1 with one UE4M3 scale per 16 elements against the given per-tensor scale (the arithmetic of
// dgb200_cast_rows_nvfp4_kernel, bit for bit: sf = e4m3_rn(amax / 6 / s_t), code = e2m1(v / (float(sf) * s_t)) with the
// reference's tie-down thresholds) and writes the packed row and its scale ints (one per 64 elements, MN-major in
// tcgen05.cp row order) into each of its top-k destination rows of the expert-sorted buffers. No reference counterpart.
__global__ void __launch_bounds__(256)
dgb200_moe_quant_dispatch_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long x_row_stride,
                                       const float* __restrict__ tensor_scale, const int* __restrict__ dest_row, int tokens,
                                       int topk, int hidden, unsigned char* __restrict__ acts, unsigned* __restrict__ acts_sf,
                                       long long sf_k_stride) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int token = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (token >= tokens) return;
    const int my_dest = lane < topk ? dest_row[token * topk + lane] : -1;
    const float s_t = __ldg(tensor_scale);
    const __nv_bfloat16* row = x + static_cast<long long>(token) * x_row_stride;
    for (int col0 = 0; col0 < hidden; col0 += 512) {
        const int col = col0 + lane * 16;  // one NVFP4 block per lane
        const bool valid = col < hidden;   // hidden is a multiple of 64
        float v[16];
        float amax = 0.0f;
        if (valid) {
            const uint4* src = reinterpret_cast<const uint4*>(row + col);
            const uint4 r0 = ld_global_nc_v4(src), r1 = ld_global_nc_v4(src + 1);
            const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.0f;
        }
        const uint32_t sf_byte = e4m3_byte(amax / 6.0f / s_t);
        const float factor = e4m3_to_float(sf_byte) * s_t;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo |= (factor > 0.0f ? e2m1_code(v[i] / factor) : 0u) << (4 * i);
            hi |= (factor > 0.0f ? e2m1_code(v[8 + i] / factor) : 0u) << (4 * i);
        }
        // packed scale int of 64 elements = the scale bytes of lanes L .. L + 3 (L a multiple of 4)
        const uint32_t b1 = __shfl_down_sync(0xffffffffu, sf_byte, 1), b2 = __shfl_down_sync(0xffffffffu, sf_byte, 2),
                       b3 = __shfl_down_sync(0xffffffffu, sf_byte, 3);
        const uint32_t sf_int = sf_byte | (b1 << 8) | (b2 << 16) | (b3 << 24);
        for (int k = 0; k < topk; ++k) {
            const int d = __shfl_sync(0xffffffffu, my_dest, k);
            if (d < 0 || !valid) continue;
            *reinterpret_cast<uint2*>(acts + static_cast<long long>(d) * (hidden / 2) + col / 2) = make_uint2(lo, hi);
            if ((lane & 3) == 0) acts_sf[static_cast<long long>(col >> 6) * sf_k_stride + sf_row_in_cp_order(d)] = sf_int;
        }
    }
}

// Token-major packed scale factors [tokens][ints_per_row] -> MN-major with every 128 rows in tcgen05.cp order
// (out[c * k_stride + sf_row_in_cp_order(t)]): the form the GEMM reads when the activations stay in token order
// (shared experts). 32 tokens per CTA through a padded shared-memory tile.
__global__ void __launch_bounds__(256)
dgb200_sf_rows_to_cp_order_kernel(const unsigned* __restrict__ sf, int tokens, int ints_per_row, unsigned* __restrict__ out,
                                  long long k_stride, const int* __restrict__ rows_limit, const int* __restrict__ first_row,
                                  const int* __restrict__ last_row_end) {
    pdl_prologue();
    extern __shared__ unsigned sf_tile[];  // [ints_per_row][33]
    if (rows_limit != nullptr) tokens = min(tokens, rows_limit[0]);  // row count only known on the device
    int begin = 0;
    if (first_row != nullptr) {  // only the rows [first_row[0], last_row_end[0]) (a range of expert segments; both multiples of 32 or the end)
        begin = first_row[0];
        tokens = min(tokens, last_row_end[0]);
    }
    const int t0 = begin + blockIdx.x * 32;
    if (t0 >= tokens) return;
    for (int i = threadIdx.x; i < 32 * ints_per_row; i += 256) {
        const int r = i / ints_per_row, c = i - r * ints_per_row;
        if (t0 + r < tokens) sf_tile[c * 33 + r] = sf[static_cast<long long>(t0 + r) * ints_per_row + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * ints_per_row; i += 256) {
        const int c = i >> 5, r = i & 31;
        if (t0 + r < tokens) out[static_cast<long long>(c) * k_stride + sf_row_in_cp_order(t0 + r)] = sf_tile[c * 33 + r];
    }
}

// SwiGLU + FP8 requant over rows of BF16 gate/up activations that a GEMM wrote without the fused epilogue (the
// swapped-operand kernel's SwiGLU epilogue is instruction-fetch bound, so for the experts it serves the gate/up GEMM
// stores BF16 and this kernel finishes; the arithmetic is the fused epilogue's, bit for bit: the accumulators are
// rounded to BF16 there too before anything else happens).
//   tmp  bf16 [rows, 2 * inter], columns in blocks of 256 = [gate 128 | up 128] (the L1 weight row order)
//   out  e4m3 [rows, inter] + packed UE8M0 scales (one int per row and 128 channels, rows in tcgen05.cp order)
// grid (ceil(max rows per expert / 8), experts); a warp owns a row, a lane 4 consecutive channels of a 128-block.
// Only experts whose row count lies in [rows_lo, rows_hi] are processed.
__global__ void __launch_bounds__(256)
dgb200_swiglu_requant_rows_kernel(const __nv_bfloat16* __restrict__ tmp, const int* __restrict__ expert_start,
                                  const int* __restrict__ expert_end, int rows_lo, int rows_hi, int inter,
                                  const float* __restrict__ row_weight, float clamp, int fast_math,
                                  unsigned char* __restrict__ act_q, long long act_q_row_stride,
                                  unsigned* __restrict__ act_sf, long long act_sf_k_stride, int first_expert) {
    pdl_prologue();
    const int e = first_expert + blockIdx.y;
    const int start = expert_start[e], rows = expert_end[e] - start;
    if (rows < rows_lo || rows > rows_hi) return;
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const long long row = static_cast<long long>(start) + r;
    const float w = row_weight != nullptr ? row_weight[row] : 1.0f;
    const __nv_bfloat16* src = tmp + row * 2 * inter;
    for (int blk = 0; blk < inter / 128; ++blk) {
        const uint2 g2 = *reinterpret_cast<const uint2*>(src + blk * 256 + lane * 4);
        const uint2 u2 = *reinterpret_cast<const uint2*>(src + blk * 256 + 128 + lane * 4);
        const unsigned gw[2] = {g2.x, g2.y}, uw[2] = {u2.x, u2.y};
        float o[4];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float gv = __uint_as_float((i & 1) ? (gw[i >> 1] & 0xffff0000u) : (gw[i >> 1] << 16));
            float uv = __uint_as_float((i & 1) ? (uw[i >> 1] & 0xffff0000u) : (uw[i >> 1] << 16));
            if (clamp > 0.0f) {
                gv = fminf(gv, clamp);
                uv = fminf(fmaxf(uv, -clamp), clamp);
            }
            const float silu = fast_math ? gv * rcp_approx(1.0f + __expf(-gv)) : gv / (1.0f + expf(-gv));
            o[i] = silu * uv * w;
            amax = fmaxf(amax, fabsf(o[i]));
        }
        // a scale group is 32 channels = 8 lanes
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float s = amax * (1.0f / 448.0f);
        const unsigned bits = __float_as_uint(s);
        unsigned ex = (bits >> 23) & 0xffu;
        if (bits & 0x7fffffu) ++ex;
        ex = min(max(ex, 1u), 254u);
        const float sf_inv = __uint_as_float((254u - ex) << 23);
        const __nv_fp8x4_e4m3 q4(make_float4(o[0] * sf_inv, o[1] * sf_inv, o[2] * sf_inv, o[3] * sf_inv));
        *reinterpret_cast<unsigned*>(act_q + row * act_q_row_stride + blk * 128 + lane * 4) = q4.__x;
        // the block's packed scale int = the scale bytes of lanes 0, 8, 16, 24
        const unsigned e1 = __shfl_sync(0xffffffffu, ex, 8), e2 = __shfl_sync(0xffffffffu, ex, 16), e3 = __shfl_sync(0xffffffffu, ex, 24);
        if (lane == 0) act_sf[static_cast<long long>(blk) * act_sf_k_stride + sf_row_in_cp_order(row)] = ex | (e1 << 8) | (e2 << 16) | (e3 << 24);
    }
}

}  // namespace dgb
