"""CPU tests of the oracle's own logic (dispatch plan, layer composition, layouts) on small seeded cases."""
import torch

from oracle import gemm as ogemm
from oracle import moe as omoe
from oracle import quant
from tests.helpers import contiguous_case, moe_case


def test_dispatch_plan_is_a_stable_sort_by_expert():
    torch.manual_seed(0)
    idx = torch.randint(-1, 6, (50, 3))
    dest, src, start, end = omoe.dispatch_plan(idx, 6, 16)
    flat = idx.reshape(-1)
    assert (dest[flat < 0] == -1).all()
    valid = torch.nonzero(flat >= 0).reshape(-1)
    assert len(set(dest[valid].tolist())) == valid.numel()
    for e in range(6):
        entries = torch.nonzero(flat == e).reshape(-1)
        rows = dest[entries]
        assert rows.tolist() == list(range(int(start[e]), int(end[e])))  # stable: entry order preserved
        assert int(start[e]) % 16 == 0
    assert torch.equal(src[dest[valid].long()].long(), valid)
    assert (src[src >= 0].numel()) == valid.numel()


def test_dispatch_plan_expert_window():
    idx = torch.tensor([[0, 5], [4, 7], [6, 1]])
    dest, src, start, end = omoe.dispatch_plan(idx, 4, 4, expert_lo=4)
    assert dest.tolist() == [-1, 4, 0, 12, 8, -1]
    assert (end - start).tolist() == [1, 1, 1, 1]


def test_layer_equals_per_token_evaluation():
    c = moe_case(12, 256, 128, 4, 2, seed=3)
    y = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
    x = quant.dequantize_fp8(c['x_q'], c['x_sf'], 32)
    for t in range(12):
        acc = torch.zeros(256)
        for k in range(2):
            e = int(c['topk_idx'][t, k])
            a1 = x[t:t + 1] @ quant.dequantize_fp4(c['l1_q'][e], c['l1_sf'][e], 32).T
            q, sf = omoe.swiglu_requant(a1, c['topk_weights'][t:t + 1, k], None)
            a2 = quant.dequantize_fp8(q, sf, 32) @ quant.dequantize_fp4(c['l2_q'][e], c['l2_sf'][e], 32).T
            acc += a2.bfloat16().float()[0]
        assert quant.calc_diff(y[t], acc.bfloat16()) < 1e-6


def test_swiglu_requant_scale_rule():
    acc = torch.zeros(2, 128)
    acc[0, :64] = 3.0      # gate
    acc[0, 64:] = 2.0      # up
    q, sf = omoe.swiglu_requant(acc, torch.tensor([0.5, 1.0]), None)
    value = 3.0 / (1 + torch.exp(torch.tensor(-3.0))) * 2.0 * 0.5
    expect_sf = quant.ue8m0_ceil(value * torch.tensor(1.0 / 448.0))
    assert torch.equal(sf[0], expect_sf.expand(2))
    assert float(sf[1, 0]) == 2.0 ** -126  # all-zero group: smallest UE8M0 scale, no 1e-4 clamp
    clamped, _ = omoe.swiglu_requant(acc * 100, torch.ones(2), 1.0)
    assert torch.isfinite(clamped.float()).all()


def test_router_renormalises_and_breaks_ties_low():
    logits = torch.tensor([[0.0, 1.0, 1.0, -2.0], [3.0, 3.0, 3.0, 3.0]])
    idx, w = omoe.route_sigmoid_topk(logits, 2)
    assert idx.tolist() == [[1, 2], [0, 1]]
    assert torch.allclose(w.sum(dim=1), torch.ones(2))


def test_contiguous_and_psum_oracles_agree():
    c = contiguous_case(3, 128, 256, 5, 40, seed=1)
    d1, m1 = ogemm.grouped_gemm_contiguous(c['a_q'], c['a_sf'], c['b_q'], c['b_sf'], c['row_ids'])
    d2, m2 = ogemm.grouped_gemm_contiguous(c['a_q'], c['a_sf'], c['b_q'], c['b_sf'], c['psum'], use_psum_layout=True)
    assert torch.equal(m1, m2) and torch.equal(d1[m1], d2[m2])
    assert int(m1.sum()) == sum(c['ms'])


def test_shared_expert_rows_add_after_the_topk_slots():
    c = moe_case(9, 256, 128, 4, 2, seed=8)
    torch.manual_seed(8)
    s1_q, s1_sf = quant.quantize_fp8_per_token((torch.randn(2 * 128, 256) * 0.05).bfloat16(), 32)
    s2_q, s2_sf = quant.quantize_fp8_per_token((torch.randn(256, 128) * 0.05).bfloat16(), 32)
    shared = omoe.shared_expert_rows(c['x_q'], c['x_sf'], s1_q, s1_sf, s2_q, s2_sf)
    assert shared.shape == (9, 256) and shared.dtype == torch.bfloat16
    y0, inter = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'],
                               c['l2_sf'], return_intermediates=True)
    y1 = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'],
                        shared_rows=shared)
    # rebuild token 0 by hand: fp32 sum of its two slot rows, then the shared row, then one rounding
    acc = torch.zeros(256)
    for k in range(2):
        e = int(c['topk_idx'][0, k])
        tok, slot, _, _, _, acc2 = inter[e]
        i = int(torch.nonzero((tok == 0) & (slot == k))[0])
        acc += acc2[i].bfloat16().float()
    assert torch.equal(y1[0], (acc + shared[0].float()).bfloat16())
    assert not torch.equal(y0, y1)


def test_bf16_layer_oracle_against_a_dense_evaluation():
    """moe_layer_bf16 (per-expert gather form) against evaluating every expert on every token and selecting."""
    import torch
    from oracle import moe as omoe
    torch.manual_seed(11)
    tokens, hidden, inter, experts, topk = 37, 64, 32, 5, 2
    x = torch.randn(tokens, hidden).bfloat16()
    w1 = (torch.randn(experts, 2 * inter, hidden) * 0.1).bfloat16()
    w2 = (torch.randn(experts, hidden, inter) * 0.1).bfloat16()
    idx, w = omoe.route_sigmoid_topk(torch.randn(tokens, experts), topk)
    idx[3, 1] = -1  # a masked slot
    s1 = (torch.randn(2 * inter, hidden) * 0.1).bfloat16()
    s2 = (torch.randn(hidden, inter) * 0.1).bfloat16()
    shared = omoe.shared_expert_rows_bf16(x, s1, s2)
    got = omoe.moe_layer_bf16(x, idx, w, w1, w2, clamp=1.0, shared_rows=shared)
    y = torch.zeros(tokens, hidden)
    for k in range(topk):
        for t in range(tokens):
            e = int(idx[t, k])
            if e < 0:
                continue
            a2 = omoe.swiglu_bf16(x[t:t + 1].float() @ w1[e].float().T, w[t:t + 1, k], 1.0)
            y[t] += (a2.float() @ w2[e].float().T).bfloat16().float()[0]
    y += shared.float()
    assert torch.equal(got, y.bfloat16())


def test_k_grouped_oracle_layouts_agree():
    """Plain K extents and the psum layout describe the same split when every extent is a multiple of the alignment."""
    import torch
    from oracle import gemm as ogemm
    from oracle import quant
    torch.manual_seed(5)
    ks, m, n = [256, 0, 128], 24, 16
    a, b = torch.randn(sum(ks), m).bfloat16(), torch.randn(sum(ks), n).bfloat16()
    a_q, a_sf = quant.quantize_fp8_per_channel(a, 128)
    b_q, b_sf = quant.quantize_fp8_per_channel(b, 128)
    c = torch.randn(len(ks), m, n)
    d1 = ogemm.k_grouped_gemm(a_q, a_sf, b_q, b_sf, c, ks)
    d2 = ogemm.k_grouped_gemm_psum(a_q, a_sf, b_q, b_sf, c, [256, 256, 384], 128)
    assert torch.equal(d1, d2) and torch.equal(d1[1], c[1])
    assert not torch.equal(d1[0], c[0])


def test_spill_plan_conserves_rows_and_balances():
    """ep_plan_with_spill over Zipf-skewed counts of 8 ranks: every (expert, source) pair lands in exactly one slot of
    one rank, the ranks agree on every segment, guests only host other ranks' experts, and the loads end up closer."""
    from oracle import moe as omoe
    ranks, experts, guests = 8, 64, 4
    per_rank = experts // ranks
    g = torch.Generator().manual_seed(5)
    popularity = 1.0 / torch.arange(1, experts + 1, dtype=torch.float32)[torch.randperm(experts, generator=g)]
    counts = torch.stack([torch.poisson(4000 * popularity / popularity.sum() * torch.ones(experts), generator=g).long()
                          for _ in range(ranks)])
    dest, slot, guest = omoe.ep_spill_table(counts, guests)
    plans = [omoe.ep_plan_with_spill(counts, r, 128, guests) for r in range(ranks)]
    rows_seen = torch.zeros(ranks, per_rank + guests, dtype=torch.long)
    for e in range(experts):
        for s in range(ranks):
            d, v = int(dest[e, s]), int(slot[e, s])
            assert int(plans[s][1][e]) == d and int(plans[s][2][e]) == v
            assert (v < per_rank and d == e // per_rank and v == e % per_rank) or \
                (v >= per_rank and d != e // per_rank and int(guest[d, v - per_rank]) == e)
            # this source's rows lie inside the segment the computing rank holds for the slot, after the earlier sources'
            start, end = int(plans[d][3][v]), int(plans[d][4][v])
            base = int(plans[s][0][e])
            assert start <= base and base + int(counts[s, e]) <= end
            rows_seen[d, v] += int(counts[s, e])
    for r in range(ranks):
        assert torch.equal(rows_seen[r], plans[r][4] - plans[r][3])
        assert all(int(plans[r][3][v]) % 128 == 0 for v in range(per_rank + guests))
        assert all(int(plans[r][3][v + 1]) >= int(plans[r][4][v]) for v in range(per_rank + guests - 1))
    before = torch.stack([counts[:, r * per_rank:(r + 1) * per_rank].sum() for r in range(ranks)])
    after = rows_seen.sum(dim=1)
    assert int(after.sum()) == int(counts.sum())
    assert int(after.max()) < int(before.max()) and int(after.max() - after.min()) < int(before.max() - before.min()) // 4
    # no guest slots: the plain plan
    my_base, my_dest, my_slot, start, end, none = omoe.ep_plan_with_spill(counts, 3, 128, 0)
    plain_base, plain_start, plain_end = omoe.ep_plan(counts, 3, 128)
    assert torch.equal(my_base, plain_base) and torch.equal(start, plain_start) and torch.equal(end, plain_end) and none.numel() == 0
