"""Parity of the MoE layer (dispatch -> L1 + SwiGLU/requant -> L2 -> combine) against the CPU oracle.
Routing indices and the dispatch permutation must be bit-exact; y within calc_diff <= 2e-3 (FP4 weights)."""
import pytest
import torch

from oracle import layout as olay
from oracle import moe as omoe
from oracle import quant
from tests.helpers import moe_case, oracle_rows_of_sampled_tokens, pick_sampled_tokens

pytestmark = pytest.mark.gpu
FP4_TOL = 2e-3
SEGMENT = 128  # rows each expert's segment is padded to (dgb200_get_segment_alignment_for_mega_moe)


@pytest.fixture(scope='module')
def dg():
    import deepgemm_b200
    return deepgemm_b200


def _device_weights(dg, c):
    """oracle-quantised weights -> the packed layouts the public API takes -> transform_weights_for_mega_moe"""
    e, n1, h = c['l1_sf'].shape[0], c['l1_q'].shape[1], c['l1_q'].shape[2] * 2
    l1_sf = dg.transform_sf_into_required_layout(c['l1_sf'].cuda(), n1, h, (1, 32), e)
    l2_sf = dg.transform_sf_into_required_layout(c['l2_sf'].cuda(), c['l2_q'].shape[1], c['l2_q'].shape[2] * 2, (1, 32), e)
    return dg.transform_weights_for_mega_moe((c['l1_q'].cuda(), l1_sf), (c['l2_q'].cuda(), l2_sf))


def _run_layer(dg, c, tokens, hidden, inter, experts, topk, clamp=None, stats=None, buf=None):
    buf = buf or dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    buf.x[:tokens].copy_(c['x_q'].cuda())
    buf.x_sf[:tokens].copy_(quant.pack_ue8m0(c['x_sf']).cuda())
    buf.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
    buf.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
    l1, l2 = _device_weights(dg, c)
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.fp8_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=clamp)
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0
    return y.cpu(), buf


def _plan_views(buf, tokens, topk, experts):
    lay = buf.layout
    raw = buf.buffer
    dest = raw[lay['dest_row']:lay['dest_row'] + tokens * topk * 4].view(torch.int32).cpu()
    end = raw[lay['expert_end']:lay['expert_end'] + experts * 4].view(torch.int32).cpu()
    start = raw[lay['expert_start']:lay['expert_start'] + experts * 4].view(torch.int32).cpu()
    return dest, start, end


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk', [
    (200, 512, 256, 8, 2),
    (77, 1024, 128, 16, 4),
    (1, 256, 128, 4, 1),
    (300, 256, 384, 5, 3),
])
def test_small_layer_matches_oracle(dg, tokens, hidden, inter, experts, topk):
    c = moe_case(tokens, hidden, inter, experts, topk, seed=tokens)
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
    stats = torch.full((experts,), 5, dtype=torch.int32, device='cuda')
    got, buf = _run_layer(dg, c, tokens, hidden, inter, experts, topk, stats=stats)
    dest, start, end = _plan_views(buf, tokens, topk, experts)
    want_dest, _, want_start, want_end = omoe.dispatch_plan(c['topk_idx'], experts, SEGMENT)
    assert torch.equal(dest, want_dest), 'dispatch permutation must be bit-exact'
    assert torch.equal(start, want_start) and torch.equal(end, want_end)
    assert torch.equal(stats.cpu(), 5 + (want_end - want_start))
    assert not torch.isnan(got.float()).any()
    assert quant.calc_diff(got, want) <= FP4_TOL


def test_masked_slots_empty_experts_and_clamp(dg):
    """topk_idx = -1 slots are skipped (reference: tests/test_mega_moe.py:131-134), two experts get no token,
    and the activation clamp is applied before SwiGLU."""
    tokens, hidden, inter, experts, topk = 150, 512, 256, 8, 3
    c = moe_case(tokens, hidden, inter, experts, topk, seed=9, masked_ratio=0.3, empty_experts=(2, 5))
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'],
                          c['l2_sf'], clamp=0.05)
    got, buf = _run_layer(dg, c, tokens, hidden, inter, experts, topk, clamp=0.05)
    dest, _, end = _plan_views(buf, tokens, topk, experts)
    want_dest, _, _, want_end = omoe.dispatch_plan(c['topk_idx'], experts, SEGMENT)
    assert torch.equal(dest, want_dest) and torch.equal(end, want_end)
    assert (dest[c['topk_idx'].reshape(-1) < 0] == -1).all()
    assert quant.calc_diff(got, want) <= FP4_TOL
    fully_masked = (c['topk_idx'] < 0).all(dim=1)
    assert (got[fully_masked] == 0).all()


def test_buffer_is_reusable_and_deterministic(dg):
    """Two calls on one buffer (fewer tokens the second time) give the same bits as fresh buffers: nothing of a
    previous call leaks into the next (the reference cleans its workspace in-kernel, sm100_fp8_fp4_mega_moe.cuh:601-659)."""
    hidden, inter, experts, topk = 512, 256, 8, 2
    big = moe_case(256, hidden, inter, experts, topk, seed=21)
    small = moe_case(100, hidden, inter, experts, topk, seed=22)
    y_big, buf = _run_layer(dg, big, 256, hidden, inter, experts, topk)
    y_small_reused, _ = _run_layer(dg, small, 100, hidden, inter, experts, topk, buf=buf)
    y_small_fresh, _ = _run_layer(dg, small, 100, hidden, inter, experts, topk)
    assert torch.equal(y_small_reused, y_small_fresh)
    y_big_again, _ = _run_layer(dg, big, 256, hidden, inter, experts, topk, buf=buf)
    assert torch.equal(y_big, y_big_again)


def test_full_config_permutation_and_sampled_tokens(dg):
    """BASELINE single-GPU layer at full size: 4096 tokens, hidden 7168, 256 experts, top-8, inter 2048.
    Weights are drawn and quantised on the GPU expert by expert. Checked: routing + permutation bit-exact against
    the oracle for all 32768 entries; y of sampled tokens against the oracle computed from the same quantised bits."""
    tokens, hidden, inter, experts, topk = 4096, 7168, 2048, 256, 8
    torch.manual_seed(0)
    x = torch.randn(tokens, hidden, device='cuda', dtype=torch.bfloat16)
    logits = torch.randn(tokens, experts, device='cuda')
    l1_q = torch.empty((experts, 2 * inter, hidden // 2), dtype=torch.int8, device='cuda')
    l1_sf = torch.empty((experts, 2 * inter, hidden // 32), dtype=torch.float32, device='cuda')
    l2_q = torch.empty((experts, hidden, inter // 2), dtype=torch.int8, device='cuda')
    l2_sf = torch.empty((experts, hidden, inter // 32), dtype=torch.float32, device='cuda')
    for e in range(experts):
        w = torch.randn(2 * inter, hidden, device='cuda', dtype=torch.bfloat16) * 0.02
        l1_q[e], l1_sf[e] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
        w = torch.randn(hidden, inter, device='cuda', dtype=torch.bfloat16) * 0.02
        l2_q[e], l2_sf[e] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
    l1_sf_p = dg.transform_sf_into_required_layout(l1_sf, 2 * inter, hidden, (1, 32), experts)
    l2_sf_p = dg.transform_sf_into_required_layout(l2_sf, hidden, inter, (1, 32), experts)
    l1, l2 = dg.transform_weights_for_mega_moe((l1_q, l1_sf_p), (l2_q, l2_sf_p))
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    x_q, x_sf = dg.utils.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
    buf.x.copy_(x_q)
    buf.x_sf.copy_(x_sf)
    dg.route_sigmoid_topk(logits, topk, buf.topk_idx, buf.topk_weights)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
    dg.fp8_fp4_mega_moe(y, l1, l2, buf)
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0

    want_idx, want_w = omoe.route_sigmoid_topk(logits.cpu(), topk)
    idx = buf.topk_idx.cpu()
    assert torch.equal(idx, want_idx)
    dest, start, end = _plan_views(buf, tokens, topk, experts)
    want_dest, _, want_start, want_end = omoe.dispatch_plan(idx, experts, SEGMENT)
    assert torch.equal(dest, want_dest) and torch.equal(end, want_end)
    assert not torch.isnan(y.float()).any()

    # values: 64 tokens, among them tokens of experts with at most 128, 129..160 and more than 160 rows
    w = buf.topk_weights.cpu()
    x_q_c, x_sf_c = x_q.cpu(), quant.unpack_ue8m0(x_sf.cpu())
    sample = sorted(set(pick_sampled_tokens(idx, 64, seed=3) + [0, 4095]))
    sizes = (want_end - want_start)
    hit = sizes[idx[sample].reshape(-1)]
    assert (hit <= 128).any() and (hit > 128).any()

    def requant(acc1, weights):
        a2_q, a2_sf = omoe.swiglu_requant(acc1, weights, None)
        return quant.dequantize_fp8(a2_q, a2_sf, 32)

    want_rows = oracle_rows_of_sampled_tokens(
        sample, idx, w, lambda toks: quant.dequantize_fp8(x_q_c[toks], x_sf_c[toks], 32),
        lambda e: quant.dequantize_fp4(l1_q[e].cpu(), l1_sf[e].cpu(), 32),
        lambda e: quant.dequantize_fp4(l2_q[e].cpu(), l2_sf[e].cpu(), 32), requant, hidden)
    y_c = y.cpu()
    for t in sample:
        assert quant.calc_diff(y_c[t], want_rows[t]) <= FP4_TOL, t


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk,use_logits', [
    (200, 512, 256, 8, 2, True),
    (77, 1024, 128, 16, 4, False),
    (130, 640, 256, 4, 3, True),      # hidden not a multiple of 512: the last column block is partial
])
def test_fused_prologue_gives_the_same_bits(dg, tokens, hidden, inter, experts, topk, use_logits):
    """fp8_fp4_mega_moe_bf16_input (router + quantise-while-dispatching) must equal the separate steps bit for bit,
    and the separate steps are checked against the oracle."""
    c = moe_case(tokens, hidden, inter, experts, topk, seed=100 + tokens, masked_ratio=0.0 if use_logits else 0.2)
    l1, l2 = _device_weights(dg, c)
    x = c['x'].cuda()
    # separate steps: quantise into the buffer, route, layer
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    dg.utils.per_token_cast_to_fp8_into(x, buf.x, buf.x_sf, gran_k=32)
    buf.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
    buf.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
    y_ref = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.fp8_fp4_mega_moe(y_ref, l1, l2, buf, fast_math=False)
    # fused prologue on a fresh buffer
    buf2 = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    if not use_logits:
        buf2.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
        buf2.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    dg.fp8_fp4_mega_moe_bf16_input(y, x, l1, l2, buf2, logits=c['logits'].cuda() if use_logits else None, fast_math=False)
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0
    if use_logits:
        assert torch.equal(buf2.topk_idx[:tokens].cpu(), c['topk_idx'])
    assert torch.equal(y.cpu(), y_ref.cpu())
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
    assert quant.calc_diff(y.cpu(), want) <= FP4_TOL


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk,num_shared,fused', [
    (200, 512, 256, 8, 2, 1, False),
    (130, 512, 128, 4, 3, 2, True),
    (256, 256, 128, 4, 1, 1, True),
])
def test_shared_experts(dg, tokens, hidden, inter, experts, topk, num_shared, fused):
    """Shared experts (FP8 x FP8, recipe (1, 1, 32)) add one combine slot after the top-k ones
    (reference: shared_l1_weights / shared_l2_weights, csrc/apis/mega.hpp:161-232)."""
    c = moe_case(tokens, hidden, inter, experts, topk, seed=300 + tokens, masked_ratio=0.1)
    si = inter * num_shared
    torch.manual_seed(tokens)
    s1_q, s1_sf = quant.quantize_fp8_per_token((torch.randn(2 * si, hidden) * 0.02).bfloat16(), 32)
    s2_q, s2_sf = quant.quantize_fp8_per_token((torch.randn(hidden, si) * 0.02).bfloat16(), 32)
    shared = omoe.shared_expert_rows(c['x_q'], c['x_sf'], s1_q, s1_sf, s2_q, s2_sf, clamp=10.0)
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'],
                          clamp=10.0, shared_rows=shared)
    l1, l2 = _device_weights(dg, c)
    sl1, sl2 = dg.transform_weights_for_mega_moe(
        (s1_q.cuda(), dg.transform_sf_into_required_layout(s1_sf.cuda(), 2 * si, hidden, (1, 32))),
        (s2_q.cuda(), dg.transform_sf_into_required_layout(s2_sf.cuda(), hidden, si, (1, 32))))
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, num_shared_experts=num_shared)
    buf.topk_idx[:tokens].copy_(c['topk_idx'].cuda())
    buf.topk_weights[:tokens].copy_(c['topk_weights'].cuda())
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
    if fused:
        dg.fp8_fp4_mega_moe_bf16_input(y, c['x'].cuda(), l1, l2, buf, shared_l1_weights=sl1, shared_l2_weights=sl2,
                                       activation_clamp=10.0, fast_math=False)
    else:
        buf.x[:tokens].copy_(c['x_q'].cuda())
        buf.x_sf[:tokens].copy_(quant.pack_ue8m0(c['x_sf']).cuda())
        dg.fp8_fp4_mega_moe(y, l1, l2, buf, shared_l1_weights=sl1, shared_l2_weights=sl2, activation_clamp=10.0,
                            fast_math=False)
    from deepgemm_b200 import _lib
    assert _lib.device_status()[0] == 0
    assert not torch.isnan(y.float()).any()
    assert quant.calc_diff(y.cpu(), want) <= FP4_TOL
    # the shared slot alone: y minus the routed part must match the shared rows
    routed = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'],
                            clamp=10.0)
    assert quant.calc_diff(y.cpu().float() - routed.float(), shared.float()) <= 5e-3
    with pytest.raises(RuntimeError):
        dg.fp8_fp4_mega_moe(y, l1, l2, dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter),
                            shared_l1_weights=sl1, shared_l2_weights=sl2)


@pytest.mark.parametrize('tokens,hidden,inter,experts,topk', [
    (300, 512, 256, 4, 2),     # 150 rows per expert on average: one token tile of up to 160 rows
    (700, 256, 256, 4, 2),     # 350 rows per expert: cut into 128-row token tiles
    (40, 512, 128, 8, 3),      # few rows, UMMA N = 16 .. 32; inter 128 -> one 256-row weight block in L1
])
def test_swapped_operand_kernel_forced(dg, tokens, hidden, inter, experts, topk):
    """Both layer GEMMs through the swapped-operand kernel (weights on UMMA M, tokens on N), including its SwiGLU
    epilogue, which the layer does not select by default."""
    from deepgemm_b200 import _lib
    c = moe_case(tokens, hidden, inter, experts, topk, seed=700 + tokens, masked_ratio=0.1)
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'],
                          clamp=5.0)
    _lib.check(_lib.lib().dgb200_set_tuning(b'swap_ab', 1))
    try:
        got, _ = _run_layer(dg, c, tokens, hidden, inter, experts, topk, clamp=5.0)
    finally:
        _lib.check(_lib.lib().dgb200_set_tuning(b'swap_ab', -1))
    assert not torch.isnan(got.float()).any()
    assert quant.calc_diff(got, want) <= FP4_TOL
    _lib.check(_lib.lib().dgb200_set_tuning(b'swap_ab', 0))
    try:
        ref, _ = _run_layer(dg, c, tokens, hidden, inter, experts, topk, clamp=5.0)
    finally:
        _lib.check(_lib.lib().dgb200_set_tuning(b'swap_ab', -1))
    assert quant.calc_diff(got, ref) <= 1e-5  # same arithmetic, only the FP32 accumulation order inside the MMA may differ


def test_down_gemm_split_by_group_size(dg):
    """Default dispatch: experts of 129..160 rows take the swapped kernel in the down GEMM, the others the tokens-on-M
    kernel. Router logits are shaped so that both kinds (and an empty expert) occur."""
    tokens, hidden, inter, experts, topk = 520, 256, 128, 5, 1
    c = moe_case(tokens, hidden, inter, experts, topk, seed=77, empty_experts=(4,))
    counts = torch.bincount(c['topk_idx'].reshape(-1), minlength=experts)
    assert ((counts >= 129) & (counts <= 160)).any() and (counts[:4] <= 128).any(), 'the seed no longer gives both kinds'
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
    got, _ = _run_layer(dg, c, tokens, hidden, inter, experts, topk)
    assert quant.calc_diff(got, want) <= FP4_TOL


def test_programmatic_dependent_launch_on_and_off(dg):
    """set_pdl (reference: csrc/apis/runtime.hpp:24-28): the layer's kernels launched with programmatic stream
    serialization (the default) and with plain launches must give the same plan and the same bits, call after call."""
    tokens, hidden, inter, experts, topk = 333, 512, 256, 16, 4
    c = moe_case(tokens, hidden, inter, experts, topk, seed=61, masked_ratio=0.1)
    assert dg.get_pdl() is True
    outs, plans = [], []
    try:
        for enabled in (True, False, True):
            dg.set_pdl(enabled)
            assert dg.get_pdl() is enabled
            for _ in range(3):  # back-to-back calls: a kernel may start before its predecessor has finished
                y, buf = _run_layer(dg, c, tokens, hidden, inter, experts, topk)
            outs.append(y)
            plans.append(_plan_views(buf, tokens, topk, experts))
    finally:
        dg.set_pdl(True)
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
    assert quant.calc_diff(outs[0], want) <= FP4_TOL
    for y, plan in zip(outs[1:], plans[1:]):
        assert torch.equal(y, outs[0])
        assert all(torch.equal(a, b) for a, b in zip(plan, plans[0]))


def test_layer_inside_a_cuda_graph(dg):
    """The single-rank layer captured into a CUDA graph (after one eager call, which creates the library's side stream and
    sets the kernels' attributes) and replayed on new inputs: the fork / join of the split GEMMs, the memset of the plan and
    the programmatic dependent launches must all be capturable, and a replay must give the bits of an eager call."""
    tokens, hidden, inter, experts, topk = 300, 512, 256, 4, 2  # about 150 rows per expert: the GEMMs split by expert size
    c = moe_case(tokens, hidden, inter, experts, topk, seed=71)
    c2 = moe_case(tokens, hidden, inter, experts, topk, seed=72)
    for k in ('l1_q', 'l1_sf', 'l2_q', 'l2_sf'):
        c2[k] = c[k]
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    l1, l2 = _device_weights(dg, c)
    y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')

    def load(case):
        buf.x[:tokens].copy_(case['x_q'].cuda())
        buf.x_sf[:tokens].copy_(quant.pack_ue8m0(case['x_sf']).cuda())
        buf.topk_idx[:tokens].copy_(case['topk_idx'].cuda())
        buf.topk_weights[:tokens].copy_(case['topk_weights'].cuda())

    from deepgemm_b200 import _lib
    load(c)
    dg.fp8_fp4_mega_moe(y, l1, l2, buf)
    assert _lib.device_status()[0] == 0
    eager = y.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dg.fp8_fp4_mega_moe(y, l1, l2, buf)
    y.fill_(float('nan'))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, eager), 'a replay on the same inputs gives the eager bits'
    load(c2)
    y.fill_(float('nan'))
    graph.replay()
    assert _lib.device_status()[0] == 0
    want = omoe.moe_layer(c2['x_q'], c2['x_sf'], c2['topk_idx'], c2['topk_weights'], c2['l1_q'], c2['l1_sf'], c2['l2_q'], c2['l2_sf'])
    assert quant.calc_diff(y.cpu(), want) <= FP4_TOL


def test_peer_wait_runs_out_and_the_library_stays_usable(dg):
    """Failure detection of the expert-parallel barrier, on one GPU and without faulting it: the layer is called as rank 0
    of 2 with both entries of the peer table pointing at this process's own buffer, so the flag "rank 1" should write
    never changes. With a 2 ms budget every wait on such a flag gives up, records the peer-timeout status (code 7, detail = the rank
    that did not answer) and the call returns; reading the status clears it. All tokens are routed to experts of rank 0,
    so the output is still the oracle's. After the test writes the missing flags itself the same call passes cleanly."""
    import ctypes
    from deepgemm_b200 import _lib, mega
    tokens, hidden, inter, experts, topk = 96, 512, 256, 8, 2
    local = experts // 2
    c = moe_case(tokens, hidden, inter, experts, topk, seed=31, empty_experts=tuple(range(local, experts)))
    assert int(c['topk_idx'].max()) < local
    want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
    lay = mega._buffer_layout(2, experts, 128, topk, hidden, inter)
    raw = torch.zeros(lay['total'], dtype=torch.int8, device='cuda')
    view = lambda key, nbytes, dtype: raw[lay[key]:lay[key] + nbytes].view(dtype)
    view('x', tokens * hidden, torch.float8_e4m3fn).view(tokens, hidden).copy_(c['x_q'].cuda())
    view('x_sf', tokens * (hidden // 128) * 4, torch.int32).view(tokens, hidden // 128).copy_(quant.pack_ue8m0(c['x_sf']).cuda())
    view('topk_idx', tokens * topk * 8, torch.int64).view(tokens, topk).copy_(c['topk_idx'].cuda())
    view('topk_weights', tokens * topk * 4, torch.float32).view(tokens, topk).copy_(c['topk_weights'].cuda())
    mine = {k: c[k][:local] for k in ('l1_q', 'l1_sf', 'l2_q', 'l2_sf')}
    l1, l2 = _device_weights(dg, mine)
    ptrs = (ctypes.c_uint64 * 2)(raw.data_ptr(), raw.data_ptr())
    lib = _lib.lib()

    def call():
        y = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
        _lib.check(lib.dgb200_fp8_fp4_mega_moe(
            y.data_ptr(), l1[0].data_ptr(), l1[1].data_ptr(), l2[0].data_ptr(), l2[1].data_ptr(), None, raw.data_ptr(),
            ctypes.cast(ptrs, ctypes.c_void_p), 0, 2, tokens, 128, experts, topk, hidden, inter, 0.0, 1, _lib.current_stream_ptr()))
        return y

    _lib.check(lib.dgb200_set_tuning(b'peer_wait_us', 2000))
    try:
        y = call()
        status = _lib.device_status(raise_on_error=False)
        assert status[0] == 7 and status[2] == 1, status  # peer timeout, waiting for rank 1
        assert _lib.device_status()[0] == 0, 'reading the status block clears it'
        assert quant.calc_diff(y.cpu(), want) <= FP4_TOL
        # play the missing rank: its flags, far ahead of any epoch this test reaches
        flags = view('flags', 13 * 8 * 4, torch.int32).view(13, 8)
        flags[:9, 1] = 1 << 20
        torch.cuda.synchronize()
        y = call()
        assert _lib.device_status()[0] == 0
        assert quant.calc_diff(y.cpu(), want) <= FP4_TOL
    finally:
        _lib.check(lib.dgb200_set_tuning(b'peer_wait_us', 10_000_000))
