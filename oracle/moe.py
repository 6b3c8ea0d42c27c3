"""CPU oracle: routing, dispatch permutation and the full MoE layer. TEST INFRASTRUCTURE ONLY (see quant.py).

The reference has no torch implementation of the whole layer (its test compares the fused kernel bitwise against
DeepEP + grouped GEMM + a TileLang SwiGLU kernel, tests/test_mega_moe.py:281-329). This file composes the
reference's own arithmetic into the layer, step by step as the fused kernel performs it
(deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh): the cited lines give each step's source.
"""
from typing import Optional, Tuple

import torch

from .quant import align, dequantize_fp4, dequantize_fp8, ue8m0_ceil


def route_sigmoid_topk(logits: torch.Tensor, topk: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router of the benchmark configurations: scores = sigmoid(logits); the ``topk`` largest per token (ties go to
    the lower expert index, listed in descending score order); weights renormalised to sum to 1.
    Returns (topk_idx int64 [T, topk], topk_weights fp32 [T, topk])."""
    order = torch.sort(logits.float(), dim=1, descending=True, stable=True).indices[:, :topk]
    scores = torch.sigmoid(logits.float()).gather(1, order)
    return order.contiguous(), (scores / scores.sum(dim=1, keepdim=True)).contiguous()


def dispatch_plan(topk_idx: torch.Tensor, num_experts: int, alignment: int, expert_lo: int = 0):
    """Deterministic dispatch permutation: the (token, k) entries, in token-major order, stably sorted by expert;
    expert e occupies rows [start[e], end[e]) with start[e] = align(end[e-1], alignment). Entries whose expert is
    outside [expert_lo, expert_lo + num_experts) (or negative = masked, tests/test_mega_moe.py:131-134) get -1.

    The reference assigns slots with atomics (sm100_fp8_fp4_mega_moe.cuh:363-377), so its order inside an expert
    depends on arrival; this stable order is the definition the CUDA path is held to bit for bit.
    Returns (dest_row int32 [T * topk], src_of_row int32 [total_rows], expert_start, expert_end int32 [E])."""
    flat = topk_idx.reshape(-1).to(torch.int64) - expert_lo
    local = (flat >= 0) & (flat < num_experts)
    counts = torch.bincount(flat[local], minlength=num_experts)
    start = torch.zeros(num_experts, dtype=torch.int64)
    end = torch.zeros(num_experts, dtype=torch.int64)
    cursor = 0
    for e in range(num_experts):
        start[e] = cursor
        end[e] = cursor + int(counts[e])
        cursor = align(int(end[e]), alignment)
    total_rows = cursor
    dest = torch.full((flat.numel(),), -1, dtype=torch.int64)
    src = torch.full((total_rows,), -1, dtype=torch.int64)
    entries = torch.nonzero(local).reshape(-1)
    order = torch.sort(flat[entries], stable=True).indices
    sorted_entries = entries[order]
    sorted_experts = flat[sorted_entries]
    rank_in_expert = torch.arange(sorted_entries.numel()) - torch.cumsum(counts, 0)[sorted_experts] + counts[sorted_experts]
    rows = start[sorted_experts] + rank_in_expert
    dest[sorted_entries] = rows
    src[rows] = sorted_entries
    return dest.to(torch.int32), src.to(torch.int32), start.to(torch.int32), end.to(torch.int32)


def swiglu_requant(gate_up: torch.Tensor, weight: torch.Tensor, clamp: Optional[float]):
    """L1 epilogue on fp32 accumulators [rows, 2I] laid out [gate | up]:
    round to bf16 -> clamp (gate <= c, |up| <= c) -> silu(gate) * up * weight in fp32 -> per-32 amax ->
    sf = 2^ceil(log2(amax * (1/448))) -> e4m3(value / sf).
    Follows sm100_fp8_fp4_mega_moe.cuh:1046-1126 with math::get_e4m3_sf_and_sf_inv
    (deep_gemm/include/deep_gemm/common/math.cuh:83-99); the formula is the TileLang baseline's
    (third-party/tilelang_ops/swiglu_apply_weight_to_fp8.py:89-94). Returns (q e4m3 [rows, I], sf fp32 [rows, I/32])."""
    half = gate_up.shape[1] // 2
    gate = gate_up[:, :half].bfloat16().float()
    up = gate_up[:, half:].bfloat16().float()
    if clamp is not None:
        gate = gate.clamp(max=clamp)
        up = up.clamp(min=-clamp, max=clamp)
    act = gate / (1.0 + torch.exp(-gate)) * up * weight.float().unsqueeze(1)
    amax = act.view(act.shape[0], -1, 32).abs().amax(dim=2)
    sf = ue8m0_ceil(amax * torch.tensor(1.0 / 448.0, dtype=torch.float32))
    q = (act.view(act.shape[0], -1, 32) * (1.0 / sf.unsqueeze(2))).to(torch.float8_e4m3fn).view(act.shape)
    return q, sf


def shared_expert_rows(x_q: torch.Tensor, x_sf: torch.Tensor, s1_q: torch.Tensor, s1_sf: torch.Tensor, s2_q: torch.Tensor,
                       s2_sf: torch.Tensor, clamp: Optional[float] = None) -> torch.Tensor:
    """Shared experts: a dense FP8 x FP8 MLP (per-32 UE8M0 scales on both operands, recipe (1, 1, 32)) over every
    token, with routing weight 1: x -> [gate | up] GEMM -> swiglu_requant -> down GEMM -> bf16 rows [T, H].
    Follows the reference's own baseline (tests/test_mega_moe.py:254-279: fp8_gemm_nt, swiglu_apply_weight_to_fp8 with
    topk_weights=None, fp8_gemm_nt); weights s1_q e4m3 [2 SI, H] with s1_sf fp32 [2 SI, H/32], s2_q [H, SI]."""
    x = dequantize_fp8(x_q, x_sf, 32)
    acc1 = x @ dequantize_fp8(s1_q, s1_sf, 32).T
    a2_q, a2_sf = swiglu_requant(acc1, torch.ones(x.shape[0]), clamp)
    return (dequantize_fp8(a2_q, a2_sf, 32) @ dequantize_fp8(s2_q, s2_sf, 32).T).bfloat16()


def moe_layer(x_q: torch.Tensor, x_sf: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
              l1_q: torch.Tensor, l1_sf: torch.Tensor, l2_q: torch.Tensor, l2_sf: torch.Tensor,
              clamp: Optional[float] = None, return_intermediates: bool = False,
              shared_rows: Optional[torch.Tensor] = None):
    """Whole layer on one rank holding every expert.

    x_q e4m3 [T, H] with x_sf fp32 [T, H/32] (per-32 UE8M0, tests/test_mega_moe.py:53-59);
    l1_q int8 [E, 2I, H/2] rows [gate | up] with l1_sf fp32 [E, 2I, H/32]; l2_q int8 [E, H, I/2], l2_sf [E, H, I/32].
    Per expert: acc1 = deq(x) @ deq(W1).T (fp32) -> swiglu_requant -> acc2 = deq(a2) @ deq(W2).T -> bf16 row;
    y[t] = bf16(sum over valid slots k, ascending, of fp32(row(t, k))) (sm100_fp8_fp4_mega_moe.cuh:1378-1430);
    ``shared_rows`` (bf16 [T, H], see shared_expert_rows) is one more slot after the top-k ones (combine slot index
    num_topk, sm100_fp8_fp4_mega_moe.cuh:1275-1278)."""
    tokens, hidden = x_q.shape
    num_experts, topk = l1_q.shape[0], topk_idx.shape[1]
    x = dequantize_fp8(x_q, x_sf, 32)
    slot_rows = torch.zeros((tokens, topk, hidden), dtype=torch.bfloat16)
    inter = {}
    for e in range(num_experts):
        tok, slot = torch.nonzero(topk_idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        w1 = dequantize_fp4(l1_q[e], l1_sf[e], 32)
        acc1 = x[tok] @ w1.T
        a2_q, a2_sf = swiglu_requant(acc1, topk_weights[tok, slot], clamp)
        w2 = dequantize_fp4(l2_q[e], l2_sf[e], 32)
        acc2 = dequantize_fp8(a2_q, a2_sf, 32) @ w2.T
        slot_rows[tok, slot] = acc2.bfloat16()
        if return_intermediates:
            inter[e] = (tok, slot, acc1, a2_q, a2_sf, acc2)
    valid = (topk_idx >= 0) & (topk_idx < num_experts)
    y = torch.zeros((tokens, hidden), dtype=torch.float32)
    for k in range(topk):
        y += torch.where(valid[:, k, None], slot_rows[:, k].float(), torch.zeros(()))
    if shared_rows is not None:
        y += shared_rows.float()
    y = y.bfloat16()
    return (y, inter) if return_intermediates else y


def swiglu_bf16(gate_up: torch.Tensor, weight: torch.Tensor, clamp: Optional[float]) -> torch.Tensor:
    """L1 epilogue of the BF16 layer on fp32 accumulators [rows, 2I] laid out [gate | up]: round to bf16 -> clamp ->
    silu(gate) * up * weight in fp32 -> bf16 (sm100_bf16_mega_moe.cuh:927-955). Returns bf16 [rows, I]."""
    half = gate_up.shape[1] // 2
    gate = gate_up[:, :half].bfloat16().float()
    up = gate_up[:, half:].bfloat16().float()
    if clamp is not None:
        gate = gate.clamp(max=clamp)
        up = up.clamp(min=-clamp, max=clamp)
    return (gate / (1.0 + torch.exp(-gate)) * up * weight.float().unsqueeze(1)).bfloat16()


def shared_expert_rows_bf16(x: torch.Tensor, s1: torch.Tensor, s2: torch.Tensor, clamp: Optional[float] = None) -> torch.Tensor:
    """Shared experts of the BF16 layer: dense MLP over every token with routing weight 1, s1 [2 SI, H] rows [gate | up],
    s2 [H, SI] (shared_l1_weights / shared_l2_weights of bf16_mega_moe, csrc/apis/mega.hpp:288-400). Returns bf16 [T, H]."""
    a2 = swiglu_bf16(x.float() @ s1.float().T, torch.ones(x.shape[0]), clamp)
    return (a2.float() @ s2.float().T).bfloat16()


def moe_layer_bf16(x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                   clamp: Optional[float] = None, shared_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The layer of moe_layer with bfloat16 activations and weights (bf16_mega_moe, csrc/apis/mega.hpp:288-400):
    x [T, H], w1 [E, 2I, H] rows [gate | up], w2 [E, H, I]; FP32 accumulation, BF16 rows between the stages, the same
    combine."""
    tokens, hidden = x.shape
    num_experts, topk = w1.shape[0], topk_idx.shape[1]
    slot_rows = torch.zeros((tokens, topk, hidden), dtype=torch.bfloat16)
    for e in range(num_experts):
        tok, slot = torch.nonzero(topk_idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        a2 = swiglu_bf16(x[tok].float() @ w1[e].float().T, topk_weights[tok, slot], clamp)
        slot_rows[tok, slot] = (a2.float() @ w2[e].float().T).bfloat16()
    valid = (topk_idx >= 0) & (topk_idx < num_experts)
    y = torch.zeros((tokens, hidden), dtype=torch.float32)
    for k in range(topk):
        y += torch.where(valid[:, k, None], slot_rows[:, k].float(), torch.zeros(()))
    if shared_rows is not None:
        y += shared_rows.float()
    return y.bfloat16()


def ep_counts(topk_idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Entries of one rank per (global) expert, masked slots (-1) excluded: the vector each rank publishes."""
    flat = topk_idx.reshape(-1)
    return torch.bincount(flat[(flat >= 0) & (flat < num_experts)], minlength=num_experts)


def ep_plan(all_counts: torch.Tensor, rank: int, alignment: int):
    """Expert-parallel dispatch plan, computed identically by every rank from all_counts [ranks, experts].

    Expert e lives on rank e // (experts / ranks) (sm100_fp8_fp4_mega_moe.cuh:372,389). On its owner, the rows of
    expert e are ordered by (source rank, entry) and the experts' segments are padded to ``alignment``.
    Returns (my_base int64 [experts]: first row on the owner of this rank's entries for e,
             expert_start, expert_end int64 [experts_per_rank] of this rank's own experts)."""
    ranks, experts = all_counts.shape
    per_rank = experts // ranks
    total = all_counts.sum(dim=0)
    before_me = all_counts[:rank].sum(dim=0)
    owner_start = torch.zeros(experts, dtype=torch.int64)
    for owner in range(ranks):
        cursor = 0
        for e in range(owner * per_rank, (owner + 1) * per_rank):
            owner_start[e] = cursor
            cursor = align(cursor + int(total[e]), alignment)
    mine = slice(rank * per_rank, (rank + 1) * per_rank)
    return owner_start + before_me, owner_start[mine].clone(), (owner_start + total)[mine].clone()


def ep_dest_rows(topk_idx: torch.Tensor, my_base: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Row, on the owner rank, of each of this rank's (token, k) entries: my_base[e] + the number of earlier entries
    of this rank with the same expert; -1 for masked slots."""
    flat = topk_idx.reshape(-1)
    dest = torch.full_like(flat, -1)
    seen = torch.zeros(num_experts, dtype=torch.int64)
    for i, e in enumerate(flat.tolist()):
        if 0 <= e < num_experts:
            dest[i] = int(my_base[e]) + int(seen[e])
            seen[e] += 1
    return dest


def ep_spill_table(all_counts: torch.Tensor, guest_slots: int):
    """Which rank computes the rows that source rank s routes to expert e, when hot experts may spill rows to other ranks.

    No reference counterpart (the reference keeps every expert's rows on its owner, sm100_fp8_fp4_mega_moe.cuh:372,389).
    Every rank has ``guest_slots`` spare expert slots after its own experts. From the same all_counts [ranks, experts]
    every rank derives the same table with integer arithmetic only:

      load[r] = rows of the experts r owns; repeat at most ranks * guest_slots times:
        hi = the most loaded rank, lo = the least loaded rank other than hi that still has a free guest slot (ties: lower rank);
        gap = load[hi] - load[lo]; stop when gap < max(256, total rows / (32 * ranks));
        e  = the expert owned by hi with the most rows still on hi (ties: lower e); stop when it has none;
        walk the source ranks from the last to the first: the rows (s, e) still on hi move to lo while
        2 * moved + count[s][e] < gap (each move must shrink the gap); stop when nothing moved;
        lo hosts e in a guest slot (the one it already has for e, else its next free one).

    Returns (dest int64 [experts, ranks]: the computing rank of (e, s); slot int64 [experts, ranks]: the expert slot on
    that rank (own experts 0..per_rank-1, guests per_rank..per_rank+guest_slots-1); guest int64 [ranks, guest_slots]:
    the expert each guest slot hosts, -1 = unused)."""
    ranks, experts = all_counts.shape
    per_rank = experts // ranks
    counts = all_counts.to(torch.int64)
    dest = (torch.arange(experts) // per_rank).unsqueeze(1).repeat(1, ranks)
    slot = (torch.arange(experts) % per_rank).unsqueeze(1).repeat(1, ranks)
    guest = torch.full((ranks, max(guest_slots, 1)), -1, dtype=torch.int64)[:, :guest_slots]
    used = [0] * ranks
    load = [int(counts[:, r * per_rank:(r + 1) * per_rank].sum()) for r in range(ranks)]
    min_gap = max(256, int(counts.sum()) // (32 * ranks))
    for _ in range(ranks * guest_slots):
        hi = max(range(ranks), key=lambda r: (load[r], -r))
        free = [r for r in range(ranks) if r != hi and used[r] < guest_slots]
        if not free:
            break
        lo = min(free, key=lambda r: (load[r], r))
        gap = load[hi] - load[lo]
        if gap < min_gap:
            break
        on_hi = lambda e: sum(int(counts[s, e]) for s in range(ranks) if int(dest[e, s]) == hi)
        e = max(range(hi * per_rank, (hi + 1) * per_rank), key=lambda e: (on_hi(e), -e))
        if on_hi(e) == 0:
            break
        hosted = [g for g in range(used[lo]) if int(guest[lo, g]) == e]
        g = hosted[0] if hosted else used[lo]
        moved = 0
        for s in reversed(range(ranks)):
            c = int(counts[s, e])
            if c > 0 and int(dest[e, s]) == hi and 2 * moved + c < gap:
                dest[e, s] = lo
                slot[e, s] = per_rank + g
                moved += c
        if moved == 0:
            break
        if not hosted:
            guest[lo, g] = e
            used[lo] += 1
        load[hi] -= moved
        load[lo] += moved
    return dest, slot, guest


def ep_plan_with_spill(all_counts: torch.Tensor, rank: int, alignment: int, guest_slots: int):
    """The expert-parallel dispatch plan of one rank under ep_spill_table. On every rank the expert slots (own experts,
    then guest slots) are laid out one after the other, each padded to ``alignment``; inside a slot the rows are ordered
    by (source rank, entry).

    Returns (my_base int64 [experts]: first row, on the computing rank, of this rank's entries for e;
             my_dest, my_slot int64 [experts]: that rank and the expert slot there;
             slot_start, slot_end int64 [per_rank + guest_slots] of this rank's own slots;
             guest int64 [guest_slots]: the experts this rank hosts as a guest, -1 = unused)."""
    ranks, experts = all_counts.shape
    per_rank = experts // ranks
    slots = per_rank + guest_slots
    dest, slot, guest = ep_spill_table(all_counts, guest_slots)
    rows = torch.zeros(ranks, slots, dtype=torch.int64)
    before_me = torch.zeros(experts, dtype=torch.int64)
    for e in range(experts):
        for s in range(ranks):
            d, v = int(dest[e, s]), int(slot[e, s])
            if s < rank and d == int(dest[e, rank]):
                before_me[e] += int(all_counts[s, e])
            rows[d, v] += int(all_counts[s, e])
    start = torch.zeros(ranks, slots, dtype=torch.int64)
    for d in range(ranks):
        cursor = 0
        for v in range(slots):
            start[d, v] = cursor
            cursor = align(cursor + int(rows[d, v]), alignment)
    my_dest, my_slot = dest[:, rank].clone(), slot[:, rank].clone()
    my_base = start[my_dest, my_slot] + before_me
    return my_base, my_dest, my_slot, start[rank].clone(), (start[rank] + rows[rank]).clone(), guest[rank].clone()
