"""Shared input builders for the parity tests: seeded CPU tensors quantised by the oracle."""
import random

import torch

from oracle import quant


def quantize_groups(t: torch.Tensor, gran_k: int, fp4: bool):
    """[G, R, K] bf16 -> (stacked q, stacked fp32 sf) with the oracle's quantisers."""
    qs, sfs = [], []
    for g in range(t.shape[0]):
        q, sf = (quant.quantize_fp4_per_token if fp4 else quant.quantize_fp8_per_token)(t[g], gran_k)
        qs.append(q)
        sfs.append(sf)
    return torch.stack(qs), torch.stack(sfs)


def contiguous_case(num_groups, n, k, m_lo, m_hi, seed, alignment=128, gran_a=128, gran_b=32, b_fp4=True):
    """BASELINE-style m-grouped contiguous inputs: rows per group uniform in [m_lo, m_hi], segments padded to
    `alignment` with zero rows; A ~ N(0,1), B ~ N(0,0.02)."""
    rng = random.Random(seed)
    torch.manual_seed(seed)
    ms = [rng.randint(m_lo, m_hi) for _ in range(num_groups)]
    aligned = [-(-x // alignment) * alignment for x in ms]
    m = sum(aligned)
    a = torch.randn(m, k).bfloat16()
    b = (torch.randn(num_groups, n, k) * 0.02).bfloat16()
    row_ids = torch.full((m,), -1, dtype=torch.int32)
    ends, start = [], 0
    for g in range(num_groups):
        row_ids[start:start + ms[g]] = g
        a[start + ms[g]:start + aligned[g]] = 0
        ends.append(start + ms[g])
        start += aligned[g]
    a_q, a_sf = quant.quantize_fp8_per_token(a, gran_a)
    b_q, b_sf = quantize_groups(b, gran_b, b_fp4)
    return dict(m=m, ms=ms, a_q=a_q, a_sf=a_sf, b_q=b_q, b_sf=b_sf, row_ids=row_ids,
                psum=torch.tensor(ends, dtype=torch.int32))


def moe_case(tokens, hidden, inter, experts, topk, seed, masked_ratio=0.0, empty_experts=()):
    """Small MoE layer inputs: x ~ N(0,1) -> FP8 per-32, weights ~ N(0,0.02) -> MXFP4 per-32, sigmoid/top-k router."""
    from oracle import moe as omoe
    torch.manual_seed(seed)
    x = torch.randn(tokens, hidden).bfloat16()
    x_q, x_sf = quant.quantize_fp8_per_token(x, 32)
    w1 = (torch.randn(experts, 2 * inter, hidden) * 0.02).bfloat16()
    w2 = (torch.randn(experts, hidden, inter) * 0.02).bfloat16()
    l1_q, l1_sf = quantize_groups(w1, 32, True)
    l2_q, l2_sf = quantize_groups(w2, 32, True)
    logits = torch.randn(tokens, experts)
    for e in empty_experts:
        logits[:, e] = -1e9
    idx, w = omoe.route_sigmoid_topk(logits, topk)
    if masked_ratio > 0:
        mask = torch.rand(idx.shape) < masked_ratio
        idx = idx.masked_fill(mask, -1)
        w = w.masked_fill(mask, 0.0)
    return dict(x=x, x_q=x_q, x_sf=x_sf, l1_q=l1_q, l1_sf=l1_sf, l2_q=l2_q, l2_sf=l2_sf, logits=logits,
                topk_idx=idx, topk_weights=w)


def moe_case_nvfp4(tokens, hidden, inter, experts, topk, seed, masked_ratio=0.0, empty_experts=()):
    """moe_case with NVFP4 tensors: x and the weights quantised by the NVFP4 oracle (per-16 UE4M3 + tensor scale)."""
    from oracle import moe as omoe
    from oracle import nvfp4 as onv
    torch.manual_seed(seed)
    x = torch.randn(tokens, hidden).bfloat16()
    x_q, x_sf, x_scale = onv.quantize_nvfp4(x)
    w1 = (torch.randn(experts, 2 * inter, hidden) * 0.02).bfloat16()
    w2 = (torch.randn(experts, hidden, inter) * 0.02).bfloat16()
    l1 = [onv.quantize_nvfp4(w1[e]) for e in range(experts)]
    l2 = [onv.quantize_nvfp4(w2[e]) for e in range(experts)]
    stack = lambda parts, i: torch.stack([p[i] for p in parts])
    logits = torch.randn(tokens, experts)
    for e in empty_experts:
        logits[:, e] = -1e9
    idx, w = omoe.route_sigmoid_topk(logits, topk)
    if masked_ratio > 0:
        mask = torch.rand(idx.shape) < masked_ratio
        idx = idx.masked_fill(mask, -1)
        w = w.masked_fill(mask, 0.0)
    return dict(x=x, x_q=x_q, x_sf=x_sf, x_scale=x_scale, l1_q=stack(l1, 0), l1_sf=stack(l1, 1), l1_scales=stack(l1, 2),
                l2_q=stack(l2, 0), l2_sf=stack(l2, 1), l2_scales=stack(l2, 2), topk_idx=idx, topk_weights=w)


def pick_sampled_tokens(topk_idx: torch.Tensor, num: int, seed: int):
    """Tokens for the value checks of the full-size layers: a quarter each routed to some expert that received at most
    128 rows, 129..160 rows and more than 160 rows (the sizes at which the layer's GEMMs change their tiling), where such
    experts exist, the rest drawn uniformly. Returns a sorted list of distinct token indices."""
    g = torch.Generator().manual_seed(seed)
    flat = topk_idx.reshape(-1)
    counts = torch.bincount(flat[flat >= 0])
    rows_of = torch.where(topk_idx >= 0, counts[topk_idx.clamp(min=0)], torch.zeros((), dtype=counts.dtype))
    chosen = set()
    for lo, hi in ((1, 128), (129, 160), (161, 1 << 30)):
        hits = torch.nonzero(((rows_of >= lo) & (rows_of <= hi)).any(dim=1)).reshape(-1)
        if hits.numel():
            chosen.update(hits[torch.randperm(hits.numel(), generator=g)[:num // 4]].tolist())
    while len(chosen) < num:
        chosen.add(int(torch.randint(0, topk_idx.shape[0], (1,), generator=g)))
    return sorted(chosen)


def oracle_rows_of_sampled_tokens(tokens, topk_idx, topk_weights, x_rows, l1_weight, l2_weight, requant, hidden):
    """y of the sampled tokens from the oracle's arithmetic, each expert's weights dequantised once:
    x_rows(token list) -> fp32 [n, H]; l1_weight(e) / l2_weight(e) -> fp32 [2I, H] / [H, I];
    requant(acc1, weights) -> fp32 [n, I] (the dequantised post-SwiGLU activations). The slots of a token are summed
    in ascending order in fp32 from their bf16 rows, as the layer's combine does. Returns {token: bf16 [H]}."""
    by_expert = {}
    for t in tokens:
        for k in range(topk_idx.shape[1]):
            e = int(topk_idx[t, k])
            if e >= 0:
                by_expert.setdefault(e, []).append((t, k))
    rows = {}
    for e, pairs in by_expert.items():
        toks = [t for t, _ in pairs]
        w = torch.stack([topk_weights[t, k] for t, k in pairs])
        acc1 = x_rows(toks) @ l1_weight(e).T
        acc2 = requant(acc1, w) @ l2_weight(e).T
        for i, pair in enumerate(pairs):
            rows[pair] = acc2[i].bfloat16().float()
    out = {}
    for t in tokens:
        acc = torch.zeros(hidden)
        for k in range(topk_idx.shape[1]):
            if (t, k) in rows:
                acc += rows[(t, k)]
        out[t] = acc.bfloat16()
    return out
