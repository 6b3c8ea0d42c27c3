"""Parity of the BF16 x BF16 GEMMs (CUDA, through the C ABI) against the CPU oracle. The reference's bound for this
family is calc_diff < 1e-5 (tests/test_bf16.py:41,83,89,144); the same bound is used here."""
import random

import pytest
import torch

from oracle import gemm as ogemm
from oracle import quant

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-5


@pytest.fixture(scope='module')
def dg():
    import deepgemm_b200
    return deepgemm_b200


def _finish():
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0


def _contiguous(num_groups, n, k, m_lo, m_hi, seed, alignment=128):
    rng = random.Random(seed)
    torch.manual_seed(seed)
    ms = [rng.randint(m_lo, m_hi) for _ in range(num_groups)]
    aligned = [-(-x // alignment) * alignment for x in ms]
    m = sum(aligned)
    a = torch.randn(m, k).bfloat16()
    b = (torch.randn(num_groups, n, k) * 0.05).bfloat16()
    row_ids = torch.full((m,), -1, dtype=torch.int32)
    ends, start = [], 0
    for g in range(num_groups):
        row_ids[start:start + ms[g]] = g
        a[start + ms[g]:start + aligned[g]] = 0
        ends.append(start + ms[g])
        start += aligned[g]
    return m, a, b, row_ids, torch.tensor(ends, dtype=torch.int32)


@pytest.mark.parametrize('use_psum', [False, True])
@pytest.mark.parametrize('n,k', [(512, 1024), (384, 192)])
def test_m_grouped_contiguous(dg, use_psum, n, k):
    m, a, b, row_ids, psum = _contiguous(4, n, k, 0 if use_psum else 64, 256, seed=1)
    layout = psum if use_psum else row_ids
    want, mask = ogemm.bf16_grouped_gemm_contiguous(a, b, layout, use_psum_layout=use_psum)
    d = torch.full((m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_bf16_gemm_nt_contiguous(a.cuda(), b.cuda(), d, layout.cuda(), use_psum_layout=use_psum,
                                         ensure_zero_padding=False)
    _finish()
    got = d.cpu()
    assert not torch.isnan(got[mask].float()).any()
    assert quant.calc_diff(got[mask], want[mask]) < BF16_TOL
    if use_psum:
        assert torch.isnan(got[~mask].float()).all(), 'rows outside the groups must not be written'
    # the [G, K, N] view of the same weights goes through the NN name
    d2 = torch.zeros_like(d)
    dg.m_grouped_bf16_gemm_nn_contiguous(a.cuda(), b.cuda().transpose(1, 2), d2, layout.cuda(), use_psum_layout=use_psum)
    _finish()
    assert torch.equal(d2.cpu()[mask], got[mask])
    # ... and genuinely [G, K, N] storage (an MN-major operand) gives the same bits
    d3 = torch.zeros_like(d)
    b_kn = b.cuda().transpose(1, 2).contiguous()
    dg.m_grouped_bf16_gemm_nn_contiguous(a.cuda(), b_kn, d3, layout.cuda(), use_psum_layout=use_psum)
    dg.m_grouped_bf16_gemm_nt_contiguous(a.cuda(), b_kn.transpose(1, 2), d2, layout.cuda(), use_psum_layout=use_psum)
    _finish()
    assert torch.equal(d3.cpu()[mask], got[mask]) and torch.equal(d2.cpu()[mask], got[mask])


def test_psum_zero_padding(dg):
    m, a, b, _, psum = _contiguous(3, 256, 256, 40, 200, seed=3)
    d = torch.full((m, 256), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_bf16_gemm_nt_contiguous(a.cuda(), b.cuda(), d, psum.cuda(), use_psum_layout=True, ensure_zero_padding=True)
    _finish()
    got = d.cpu()
    want, mask = ogemm.bf16_grouped_gemm_contiguous(a, b, psum, use_psum_layout=True)
    assert quant.calc_diff(got[mask], want[mask]) < BF16_TOL
    assert (got[~mask] == 0).all()


@pytest.mark.parametrize('max_m', [256, 200])
def test_masked(dg, max_m):
    torch.manual_seed(5)
    g, n, k = 6, 512, 448
    a = torch.randn(g, max_m, k).bfloat16()
    b = (torch.randn(g, n, k) * 0.05).bfloat16()
    masked_m = torch.tensor([0, 1, 127, 128, 129, max_m], dtype=torch.int32)
    want, mask = ogemm.bf16_grouped_gemm_masked(a, b, masked_m)
    d = torch.full((g, max_m, n), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_bf16_gemm_nt_masked(a.cuda(), b.cuda(), d, masked_m.cuda(), 64)
    _finish()
    got = d.cpu()
    assert quant.calc_diff(got[mask], want[mask]) < BF16_TOL
    assert torch.isnan(got[~mask].float()).all(), 'rows at or past masked_m[g] must not be written'


@pytest.mark.parametrize('m,n,k,out', [(1, 128, 64, torch.bfloat16), (300, 768, 1024, torch.bfloat16),
                                       (200, 384, 320, torch.bfloat16), (72, 256, 128, torch.float32),
                                       (4096, 4096, 4096, torch.bfloat16), (130, 256, 512, torch.float32)])
def test_dense(dg, m, n, k, out):
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k).bfloat16().cuda()
    b = (torch.randn(n, k) * 0.05).bfloat16().cuda()
    d = torch.full((m, n), float('nan'), dtype=out, device='cuda')
    dg.bf16_gemm_nt(a, b, d)
    _finish()
    want = (a.float() @ b.float().T).to(out)  # FP32 product of the same tensors, as the reference's test builds it
    assert quant.calc_diff(d.cpu(), want.cpu()) < BF16_TOL
    d2 = torch.zeros_like(d)
    dg.bf16_gemm_nn(a, b.transpose(0, 1), d2)
    _finish()
    assert torch.equal(d2, d)
    d2.zero_()
    dg.bf16_gemm_nn(a, b.transpose(0, 1).contiguous(), d2)  # row-major [K, N] storage: an MN-major operand
    _finish()
    assert torch.equal(d2, d)
    if m % 8 == 0:  # a given as [K, M] storage: MN-major A
        a_km = a.transpose(0, 1).contiguous()
        d2.zero_()
        dg.bf16_gemm_tt(a_km, b, d2)
        _finish()
        assert torch.equal(d2, d)
        d2.zero_()
        dg.bf16_gemm_tn(a_km, b.transpose(0, 1).contiguous(), d2)
        _finish()
        assert torch.equal(d2, d)
    if out == torch.float32:  # the accumulator input: d = c + a @ b.T
        c = torch.randn(m, n, device='cuda') * 3
        d3 = torch.full_like(d, float('nan'))
        dg.bf16_gemm_nt(a, b, d3, c=c)
        _finish()
        assert torch.equal(d3, c + d)


def test_rejected_inputs(dg):
    a = torch.zeros(128, 96, dtype=torch.bfloat16, device='cuda')  # k not a multiple of 64
    b = torch.zeros(128, 96, dtype=torch.bfloat16, device='cuda')
    d = torch.zeros(128, 128, dtype=torch.bfloat16, device='cuda')
    with pytest.raises(RuntimeError):
        dg.bf16_gemm_nt(a, b, d)
    with pytest.raises(RuntimeError):
        dg.bf16_gemm_nt(a.float(), b, d)
    with pytest.raises(RuntimeError):
        dg.bf16_gemm_nt(a, b, d, c=d)  # accumulation needs a float32 d


# ----------------------------------------------------------------------------------------------------------------
# the BF16 layer
# ----------------------------------------------------------------------------------------------------------------
def _layer_case(tokens, hidden, inter, experts, topk, seed, masked_ratio=0.0):
    from oracle import moe as omoe
    torch.manual_seed(seed)
    x = torch.randn(tokens, hidden).bfloat16()
    w1 = (torch.randn(experts, 2 * inter, hidden) * 0.05).bfloat16()
    w2 = (torch.randn(experts, hidden, inter) * 0.05).bfloat16()
    idx, w = omoe.route_sigmoid_topk(torch.randn(tokens, experts), topk)
    if masked_ratio > 0:
        mask = torch.rand(idx.shape) < masked_ratio
        idx = idx.masked_fill(mask, -1)
        w = w.masked_fill(mask, 0.0)
    return x, w1, w2, idx, w


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk,clamp,masked', [
    (200, 512, 256, 8, 2, None, 0.0),
    (77, 1024, 128, 16, 4, 0.5, 0.2),
    (1, 256, 128, 4, 1, None, 0.0),
    (1000, 256, 384, 5, 3, None, 0.0),
])
def test_bf16_layer_matches_oracle(dg, tokens, hidden, inter, experts, topk, clamp, masked):
    from oracle import moe as omoe
    x, w1, w2, idx, w = _layer_case(tokens, hidden, inter, experts, topk, seed=tokens, masked_ratio=masked)
    want = omoe.moe_layer_bf16(x, idx, w, w1, w2, clamp)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, mma_type='bf16xbf16')
    buf.x[:tokens].copy_(x.cuda())
    buf.topk_idx[:tokens].copy_(idx.cuda())
    buf.topk_weights[:tokens].copy_(w.cuda())
    l1, l2 = dg.transform_weights_for_mega_moe(w1.cuda(), w2.cuda())
    stats = torch.zeros(experts, dtype=torch.int32, device='cuda')
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    for _ in range(2):  # the buffer is reusable
        dg.bf16_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=clamp)
    _finish()
    got = y.cpu()
    assert not torch.isnan(got.float()).any()
    # BF16 rows between the stages round differently where the FP32 sums differ in their last bits (summation order),
    # so the reference's 1e-5 bound of a single GEMM does not carry over to two chained GEMMs with a BF16 rounding between
    assert quant.calc_diff(got, want) < 1e-4
    counts = torch.bincount(idx[idx >= 0].reshape(-1), minlength=experts).int()
    assert torch.equal(stats.cpu(), 2 * counts)


@pytest.mark.parametrize('tokens,num_shared', [(256, 1), (100, 2)])
def test_bf16_layer_with_shared_experts(dg, tokens, num_shared):
    from oracle import moe as omoe
    hidden, inter, experts, topk = 512, 128, 8, 2
    x, w1, w2, idx, w = _layer_case(tokens, hidden, inter, experts, topk, seed=tokens + 7, masked_ratio=0.1)
    si = inter * num_shared
    s1 = (torch.randn(2 * si, hidden) * 0.05).bfloat16()
    s2 = (torch.randn(hidden, si) * 0.05).bfloat16()
    want = omoe.moe_layer_bf16(x, idx, w, w1, w2, shared_rows=omoe.shared_expert_rows_bf16(x, s1, s2))
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, num_shared_experts=num_shared,
                                          mma_type='bf16xbf16')
    buf.x[:tokens].copy_(x.cuda())
    buf.topk_idx[:tokens].copy_(idx.cuda())
    buf.topk_weights[:tokens].copy_(w.cuda())
    l1, l2 = dg.transform_weights_for_mega_moe(w1.cuda(), w2.cuda())
    sl1, sl2 = dg.transform_weights_for_mega_moe(s1.cuda(), s2.cuda())
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.bf16_mega_moe(y, l1, l2, buf, shared_l1_weights=sl1, shared_l2_weights=sl2)
    _finish()
    got = y.cpu()
    assert not torch.isnan(got.float()).any()
    assert quant.calc_diff(got, want) < 1e-4
    # the same buffer without the shared experts
    y2 = torch.full_like(y, float('nan'))
    dg.bf16_mega_moe(y2, l1, l2, buf)
    _finish()
    assert quant.calc_diff(y2.cpu(), omoe.moe_layer_bf16(x, idx, w, w1, w2)) < 1e-4
