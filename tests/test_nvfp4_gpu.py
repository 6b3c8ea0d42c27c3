"""Parity of the NVFP4 x NVFP4 path (quantiser, grouped GEMM, MoE layer) against the CPU oracle, through the
package's public operators (each one a call into libdgb200.so). The quantiser must be bit-exact; GEMM and layer
outputs within calc_diff <= 2e-3, the tolerance of the FP4 paths. The oracle for this format is authored from the
published NVFP4 definition (the reference has no NVFP4 code), see oracle/nvfp4.py."""
import random

import pytest
import torch

from oracle import moe as omoe
from oracle import nvfp4 as onv
from oracle import quant
from tests.helpers import moe_case_nvfp4, oracle_rows_of_sampled_tokens, pick_sampled_tokens

pytestmark = pytest.mark.gpu
FP4_TOL = 2e-3
SEGMENT = 128  # rows each expert's segment is padded to (dgb200_get_segment_alignment_for_mega_moe)


@pytest.fixture(scope='module')
def dg():
    import deepgemm_b200
    return deepgemm_b200


def _status_ok():
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0


@pytest.mark.parametrize('rows,k', [(1, 64), (70, 512), (33, 7168), (257, 2048)])
def test_cast_is_bit_exact(dg, rows, k):
    torch.manual_seed(rows)
    x = torch.randn(rows, k).bfloat16()
    x[0, :16] = 0
    if rows > 2:
        x[2] = 0
    want_q, want_sf, want_scale = onv.quantize_nvfp4(x)
    q, sf, scale = dg.per_token_cast_to_nvfp4(x.cuda())
    assert float(scale.cpu()) == float(want_scale)
    assert torch.equal(q.cpu(), want_q)
    assert torch.equal(sf.cpu().view(torch.uint8), want_sf.view(torch.uint8))
    # MN-major packed form, as the GEMM reads it
    _, sf_mn, _ = dg.per_token_cast_to_nvfp4(x.cuda(), sf_layout='mn')
    want_mn = onv.pack_sf_bytes_mn_major(want_sf.unsqueeze(0))[0]
    assert sf_mn.stride(0) == 1 and torch.equal(sf_mn.cpu().t().contiguous(), want_mn[:, :rows])
    assert torch.equal(dg.pack_nvfp4_sf_mn_major(want_sf.cuda()).cpu().t().contiguous(), want_mn[:, :rows])


def test_cast_with_calibrated_scale_saturates(dg):
    torch.manual_seed(3)
    x = (torch.randn(40, 256) * 5).bfloat16()
    fixed = torch.tensor(2e-4)
    want_q, want_sf, _ = onv.quantize_nvfp4(x, fixed)
    q, sf, _ = dg.per_token_cast_to_nvfp4(x.cuda(), fixed.cuda())
    assert float(want_sf.float().max()) == 448.0
    assert torch.equal(q.cpu(), want_q) and torch.equal(sf.cpu().view(torch.uint8), want_sf.view(torch.uint8))


def test_all_zero_tensor(dg):
    q, sf, scale = dg.per_token_cast_to_nvfp4(torch.zeros(8, 128, dtype=torch.bfloat16, device='cuda'))
    assert float(scale.cpu()) == 1.0 and (q == 0).all() and (sf.view(torch.uint8) == 0).all()


def _gemm_case(num_groups, n, k, m_lo, m_hi, seed, alignment):
    rng = random.Random(seed)
    torch.manual_seed(seed)
    ms = [rng.randint(m_lo, m_hi) for _ in range(num_groups)]
    ends, cur = [], 0
    row_ids = []
    for g, v in enumerate(ms):
        ends.append(cur + v)
        nxt = -(-(cur + v) // alignment) * alignment
        row_ids += [g] * v + [-1] * (nxt - cur - v)
        cur = nxt
    m = -(-max(cur, 1) // 128) * 128
    row_ids += [-1] * (m - len(row_ids))
    a = torch.randn(m, k).bfloat16()
    b = (torch.randn(num_groups, n, k) * 0.02).bfloat16()
    a_q, a_sf, a_s = onv.quantize_nvfp4(a)
    parts = [onv.quantize_nvfp4(b[g]) for g in range(num_groups)]
    b_q, b_sf, b_s = (torch.stack([p[i] for p in parts]) for i in range(3))
    return dict(m=m, a=(a_q, a_sf, a_s), b=(b_q, b_sf, b_s), psum=torch.tensor(ends, dtype=torch.int32),
                row_ids=torch.tensor(row_ids, dtype=torch.int32))


@pytest.mark.parametrize('num_groups,n,k,m_lo,m_hi,alignment,out', [
    (1, 128, 256, 128, 128, 128, torch.float32),
    (3, 512, 1024, 1, 200, 16, torch.bfloat16),
    (4, 256, 2048, 0, 90, 4, torch.bfloat16),      # empty groups possible, N = 256 tile
    (2, 384, 512, 100, 300, 128, torch.float32),   # N = 384 -> 128-wide tiles
])
def test_grouped_gemm_psum(dg, num_groups, n, k, m_lo, m_hi, alignment, out):
    c = _gemm_case(num_groups, n, k, m_lo, m_hi, seed=n + k, alignment=alignment)
    want, mask = onv.grouped_gemm_contiguous(*c['a'], *c['b'], c['psum'], alignment, out)
    d = torch.full((c['m'], n), float('nan'), dtype=out, device='cuda')
    dg.set_mk_alignment_for_contiguous_layout(alignment)
    try:
        dg.m_grouped_nvfp4_gemm_nt_contiguous(tuple(t.cuda() for t in c['a']), tuple(t.cuda() for t in c['b']), d,
                                              c['psum'].cuda(), use_psum_layout=True)
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)
    _status_ok()
    got = d.cpu()
    if mask.any():
        assert not torch.isnan(got[mask].float()).any()
        assert quant.calc_diff(got[mask].float(), want[mask].float()) <= FP4_TOL
    assert torch.isnan(got[~mask].float()).all(), 'rows outside every group must stay untouched'


def test_grouped_gemm_row_ids(dg):
    c = _gemm_case(3, 256, 512, 60, 250, seed=11, alignment=128)
    want, mask = onv.grouped_gemm_contiguous(*c['a'], *c['b'], c['psum'], 128)
    d = torch.zeros((c['m'], 256), dtype=torch.bfloat16, device='cuda')
    dg.m_grouped_nvfp4_gemm_nt_contiguous(tuple(t.cuda() for t in c['a']), tuple(t.cuda() for t in c['b']), d,
                                          c['row_ids'].cuda())
    _status_ok()
    assert quant.calc_diff(d.cpu()[mask].float(), want[mask].float()) <= FP4_TOL


def test_gemm_linearity_in_tensor_scales(dg):
    """Size-independent property: doubling a per-tensor scale doubles D exactly (power of two, FP32 epilogue)."""
    c = _gemm_case(2, 256, 512, 100, 128, seed=4, alignment=128)
    a = tuple(t.cuda() for t in c['a'])
    b = tuple(t.cuda() for t in c['b'])
    d1 = torch.zeros((c['m'], 256), dtype=torch.float32, device='cuda')
    d2 = torch.zeros_like(d1)
    dg.m_grouped_nvfp4_gemm_nt_contiguous(a, b, d1, c['psum'].cuda(), use_psum_layout=True)
    dg.m_grouped_nvfp4_gemm_nt_contiguous((a[0], a[1], a[2] * 2), (b[0], b[1], b[2] * 4), d2, c['psum'].cuda(),
                                          use_psum_layout=True)
    _status_ok()
    assert torch.equal(d1 * 8, d2)


def test_rejects_bad_shapes(dg):
    c = _gemm_case(1, 128, 256, 128, 128, seed=1, alignment=128)
    a = tuple(t.cuda() for t in c['a'])
    b = tuple(t.cuda() for t in c['b'])
    d = torch.zeros((128, 128), dtype=torch.bfloat16, device='cuda')
    with pytest.raises(RuntimeError):
        dg.m_grouped_nvfp4_gemm_nt_contiguous((a[0][:, :64].contiguous(), a[1][:, :8].contiguous(), a[2]), b, d,
                                              c['psum'].cuda(), use_psum_layout=True)  # K mismatch
    with pytest.raises(RuntimeError):
        dg.per_token_cast_to_nvfp4(torch.zeros(4, 48, dtype=torch.bfloat16, device='cuda'))  # k % 64 != 0
    with pytest.raises(RuntimeError):
        dg.get_symm_buffer_for_mega_moe(None, 4, 128, 2, 384, 256, mma_type='nvfp4xnvfp4')  # hidden % 256 != 0


def _run_layer(dg, c, tokens, hidden, inter, experts, topk, act_scale, clamp=None, buf=None):
    buf = buf or dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, mma_type='nvfp4xnvfp4')
    buf.x[:tokens].copy_(c['x_q'].cuda())
    buf.x_sf[:tokens].copy_(c['x_sf'].view(torch.uint8).contiguous().view(torch.int32).cuda())
    buf.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
    buf.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
    l1 = (c['l1_q'].cuda(), dg.pack_nvfp4_sf_mn_major(c['l1_sf'].cuda()), c['l1_scales'].cuda())
    l2 = (c['l2_q'].cuda(), dg.pack_nvfp4_sf_mn_major(c['l2_sf'].cuda()), c['l2_scales'].cuda())
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.nvfp4_mega_moe(y, l1, l2, buf, c['x_scale'].cuda(), act_scale.cuda(), activation_clamp=clamp, fast_math=False)
    _status_ok()
    return y.cpu(), buf


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk,masked', [
    (200, 512, 256, 8, 2, 0.0),
    (77, 1024, 256, 16, 4, 0.0),
    (1, 256, 256, 4, 1, 0.0),
    (150, 512, 512, 6, 3, 0.3),
])
def test_layer_matches_oracle(dg, tokens, hidden, inter, experts, topk, masked):
    c = moe_case_nvfp4(tokens, hidden, inter, experts, topk, seed=tokens, masked_ratio=masked,
                       empty_experts=(1,) if masked else ())
    act_scale = onv.calibrate_act_scale(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'],
                                        c['l1_sf'], c['l1_scales'])
    want = onv.moe_layer_nvfp4(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'],
                               c['l1_scales'], c['l2_q'], c['l2_sf'], c['l2_scales'], act_scale)
    got, buf = _run_layer(dg, c, tokens, hidden, inter, experts, topk, act_scale)
    lay = buf.layout
    dest = buf.buffer[lay['dest_row']:lay['dest_row'] + tokens * topk * 4].view(torch.int32).cpu()
    want_dest, _, _, _ = omoe.dispatch_plan(c['topk_idx'], experts, SEGMENT)
    assert torch.equal(dest, want_dest), 'dispatch permutation must be bit-exact'
    assert not torch.isnan(got.float()).any()
    assert quant.calc_diff(got, want) <= FP4_TOL
    fully_masked = (c['topk_idx'] < 0).all(dim=1)
    assert (got[fully_masked] == 0).all()


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk,use_logits', [
    (200, 512, 256, 8, 2, False),
    (333, 1024, 256, 16, 4, True),
    (1, 256, 256, 4, 1, True),
])
def test_fused_prologue_gives_the_same_bits(dg, tokens, hidden, inter, experts, topk, use_logits):
    """nvfp4_mega_moe_bf16_input (BF16 rows quantised to NVFP4 while they are dispatched, router inside the call) against the
    separate steps per_token_cast_to_nvfp4_into + route_sigmoid_topk + nvfp4_mega_moe: same plan, same output bits."""
    c = moe_case_nvfp4(tokens, hidden, inter, experts, topk, seed=900 + tokens)
    torch.manual_seed(tokens)
    logits = torch.randn(tokens, experts).cuda()
    x = c['x'].cuda()
    x_scale, act_scale = c['x_scale'].cuda(), torch.tensor(2e-4).cuda()
    l1 = (c['l1_q'].cuda(), dg.pack_nvfp4_sf_mn_major(c['l1_sf'].cuda()), c['l1_scales'].cuda())
    l2 = (c['l2_q'].cuda(), dg.pack_nvfp4_sf_mn_major(c['l2_sf'].cuda()), c['l2_scales'].cuda())
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    outs, plans = [], []
    for fused in (False, True):
        buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, mma_type='nvfp4xnvfp4')
        if use_logits and not fused:
            dg.route_sigmoid_topk(logits, topk, buf.topk_idx[:tokens], buf.topk_weights[:tokens])
        elif not use_logits:
            buf.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
            buf.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
        y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
        if fused:
            dg.nvfp4_mega_moe_bf16_input(y, x, l1, l2, buf, x_scale, act_scale, logits=logits if use_logits else None,
                                         fast_math=False)
        else:
            dg.per_token_cast_to_nvfp4_into(x, x_scale, buf.x, buf.x_sf)
            dg.nvfp4_mega_moe(y, l1, l2, buf, x_scale, act_scale, fast_math=False)
        _status_ok()
        lay = buf.layout
        outs.append(y.cpu())
        plans.append(buf.buffer[lay['dest_row']:lay['dest_row'] + tokens * topk * 4].view(torch.int32).cpu())
    assert not torch.isnan(outs[0].float()).any()
    assert torch.equal(plans[0], plans[1]) and torch.equal(outs[0], outs[1])


def test_layer_with_clamp_and_saturating_act_scale(dg):
    """An activation scale 8x too small makes block scales saturate at 448; kernel and oracle must clip alike."""
    tokens, hidden, inter, experts, topk = 96, 512, 256, 4, 2
    c = moe_case_nvfp4(tokens, hidden, inter, experts, topk, seed=13)
    act_scale = onv.calibrate_act_scale(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'],
                                        c['l1_sf'], c['l1_scales'], clamp=0.5) / 8
    want = onv.moe_layer_nvfp4(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'],
                               c['l1_scales'], c['l2_q'], c['l2_sf'], c['l2_scales'], act_scale, clamp=0.5)
    got, _ = _run_layer(dg, c, tokens, hidden, inter, experts, topk, act_scale, clamp=0.5)
    assert quant.calc_diff(got, want) <= FP4_TOL


def test_layer_buffer_reuse_is_deterministic(dg):
    hidden, inter, experts, topk = 512, 256, 8, 2
    big = moe_case_nvfp4(256, hidden, inter, experts, topk, seed=21)
    small = moe_case_nvfp4(100, hidden, inter, experts, topk, seed=22)
    s = torch.tensor(1e-5)
    y_big, buf = _run_layer(dg, big, 256, hidden, inter, experts, topk, s)
    y_small_reused, _ = _run_layer(dg, small, 100, hidden, inter, experts, topk, s, buf=buf)
    y_small_fresh, _ = _run_layer(dg, small, 100, hidden, inter, experts, topk, s)
    assert torch.equal(y_small_reused, y_small_fresh)
    y_big_again, _ = _run_layer(dg, big, 256, hidden, inter, experts, topk, s, buf=buf)
    assert torch.equal(y_big, y_big_again)


def test_full_prefill_config_permutation_and_sampled_tokens(dg):
    """BASELINE NVFP4 prefill layer at full size: 16384 tokens, hidden 7168, 256 experts, top-8, inter 2048. Weights and
    activations are quantised on the GPU. Checked: routing and the permutation of all 131072 entries bit-exact against
    the oracle; y of sampled tokens against the oracle evaluated from the same quantised bits."""
    tokens, hidden, inter, experts, topk = 16384, 7168, 2048, 256, 8
    torch.manual_seed(0)
    x = torch.randn(tokens, hidden, device='cuda', dtype=torch.bfloat16)
    logits = torch.randn(tokens, experts, device='cuda')
    l1_q = torch.empty((experts, 2 * inter, hidden // 2), dtype=torch.int8, device='cuda')
    l1_sf = torch.empty((experts, 2 * inter, hidden // 16), dtype=torch.float8_e4m3fn, device='cuda')
    l2_q = torch.empty((experts, hidden, inter // 2), dtype=torch.int8, device='cuda')
    l2_sf = torch.empty((experts, hidden, inter // 16), dtype=torch.float8_e4m3fn, device='cuda')
    l1_s = torch.empty(experts, dtype=torch.float32, device='cuda')
    l2_s = torch.empty(experts, dtype=torch.float32, device='cuda')
    for e in range(experts):
        w = torch.randn(2 * inter, hidden, device='cuda', dtype=torch.bfloat16) * 0.02
        l1_q[e], l1_sf[e], l1_s[e] = dg.per_token_cast_to_nvfp4(w)
        w = torch.randn(hidden, inter, device='cuda', dtype=torch.bfloat16) * 0.02
        l2_q[e], l2_sf[e], l2_s[e] = dg.per_token_cast_to_nvfp4(w)
    l1, l2 = dg.transform_weights_for_mega_moe((l1_q, dg.pack_nvfp4_sf_mn_major(l1_sf), l1_s),
                                               (l2_q, dg.pack_nvfp4_sf_mn_major(l2_sf), l2_s))
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, mma_type='nvfp4xnvfp4')
    x_scale = torch.tensor(8.0 / (6 * 448), device='cuda')
    act_scale = torch.tensor(64.0 / (6 * 448), device='cuda')
    dg.per_token_cast_to_nvfp4_into(x, x_scale, buf.x, buf.x_sf)
    dg.route_sigmoid_topk(logits, topk, buf.topk_idx, buf.topk_weights)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
    dg.nvfp4_mega_moe(y, l1, l2, buf, x_scale, act_scale, fast_math=False)
    _status_ok()

    want_idx, _ = omoe.route_sigmoid_topk(logits.cpu(), topk)
    idx = buf.topk_idx.cpu()
    assert torch.equal(idx, want_idx)
    lay = buf.layout
    dest = buf.buffer[lay['dest_row']:lay['dest_row'] + tokens * topk * 4].view(torch.int32).cpu()
    want_dest, _, _, _ = omoe.dispatch_plan(idx, experts, SEGMENT)
    assert torch.equal(dest, want_dest)
    assert not torch.isnan(y.float()).any()

    w = buf.topk_weights.cpu()
    x_q_c = buf.x.cpu()
    x_sf_c = buf.x_sf.cpu().view(torch.uint8).view(torch.float8_e4m3fn).view(tokens, hidden // 16)
    xs, acs = x_scale.cpu(), act_scale.cpu()
    sample = sorted(set(pick_sampled_tokens(idx, 64, seed=4) + [0, 16383]))

    def requant(acc1, weights):
        a2_q, a2_sf = onv.swiglu_requant_nvfp4(acc1, weights, None, acs)
        return onv.dequantize_nvfp4(a2_q, a2_sf, acs)

    want_rows = oracle_rows_of_sampled_tokens(
        sample, idx, w, lambda toks: onv.dequantize_nvfp4(x_q_c[toks], x_sf_c[toks], xs),
        lambda e: onv.dequantize_nvfp4(l1_q[e].cpu(), l1_sf[e].cpu(), l1_s[e].cpu()),
        lambda e: onv.dequantize_nvfp4(l2_q[e].cpu(), l2_sf[e].cpu(), l2_s[e].cpu()), requant, hidden)
    y_c = y.cpu()
    for t in sample:
        assert quant.calc_diff(y_c[t], want_rows[t]) <= FP4_TOL, t
