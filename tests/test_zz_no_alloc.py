"""The allocation-free dispatch-plan entry point (dgb200_moe_dispatch_plan_noalloc) against the plan the layer call
builds in its caller-provided buffer.

Who needs it: hosts that may not call cudaMalloc where they invoke the library (a fixed memory pool owned by another
allocator, a callback that must not synchronise, a no-allocation-after-start-up policy). The scratch lives in a
static device array inside the library, shared by all calls, so the test makes two calls in a row with different
inputs (the second smaller): nothing of the first call may leak into the second. This file sorts last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan_from_layer(dg, case, tokens, hidden, inter, experts, topk):
    from deepgemm_b200 import _lib
    from oracle import quant
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    buf.x[:tokens].copy_(case['x_q'].cuda())
    buf.x_sf[:tokens].copy_(quant.pack_ue8m0(case['x_sf']).cuda())
    buf.topk_idx[:tokens].copy_(case['topk_idx'].cuda())
    buf.topk_weights[:tokens].copy_(case['topk_weights'].cuda())
    l1_sf = dg.transform_sf_into_required_layout(case['l1_sf'].cuda(), 2 * inter, hidden, (1, 32), experts)
    l2_sf = dg.transform_sf_into_required_layout(case['l2_sf'].cuda(), hidden, inter, (1, 32), experts)
    l1, l2 = dg.transform_weights_for_mega_moe((case['l1_q'].cuda(), l1_sf), (case['l2_q'].cuda(), l2_sf))
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
    dg.fp8_fp4_mega_moe(y, l1, l2, buf)
    assert _lib.device_status()[0] == 0
    lay, raw = buf.layout, buf.buffer
    take = lambda key, n: raw[lay[key]:lay[key] + n * 4].view(torch.int32).clone()
    return take('dest_row', tokens * topk), take('expert_start', experts), take('expert_end', experts)


def _plan_noalloc(topk_idx, experts, alignment, tokens=None):
    from deepgemm_b200 import _lib
    lib = _lib.lib()
    topk = topk_idx.shape[1]
    tokens = topk_idx.shape[0] if tokens is None else tokens  # fewer than the tensor holds: only the first rows are read
    idx = topk_idx.cuda().contiguous()
    dest = torch.full((max(tokens * topk, 1),), -7, dtype=torch.int32, device='cuda')
    start = torch.full((experts,), -7, dtype=torch.int32, device='cuda')
    end = torch.full((experts,), -7, dtype=torch.int32, device='cuda')
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(lib.dgb200_moe_dispatch_plan_noalloc(p(idx), tokens, topk, experts, alignment, p(dest), p(start), p(end),
                                                    _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    return dest, start, end


def test_noalloc_plan_matches_layer_plan_twice_in_a_row():
    import deepgemm_b200 as dg
    from tests.helpers import moe_case
    hidden, inter, experts, topk = 256, 128, 16, 4
    for tokens, seed in ((700, 41), (90, 42)):  # 2800 entries = 3 chunks, then a single partial chunk
        case = moe_case(tokens, hidden, inter, experts, topk, seed=seed, masked_ratio=0.2)
        want = _plan_from_layer(dg, case, tokens, hidden, inter, experts, topk)
        got = _plan_noalloc(case['topk_idx'], experts, dg.get_segment_alignment_for_mega_moe())
        for g, w, name in zip(got, want, ('dest_row', 'expert_start', 'expert_end')):
            assert torch.equal(g, w), f'{name} differs from the layer call ({tokens} tokens)'


def test_noalloc_plan_rejects_oversized_problems():
    from deepgemm_b200 import _lib
    lib = _lib.lib()
    one = ctypes.c_void_p(16)
    assert lib.dgb200_moe_dispatch_plan_noalloc(one, 65536, 2, 8, 16, one, one, one, None) == 1
    assert 'exceeds the built-in scratch' in lib.dgb200_last_error().decode()
    assert lib.dgb200_moe_dispatch_plan_noalloc(one, 16, 2, 513, 16, one, one, one, None) == 1
    assert 'exceeds the built-in scratch' in lib.dgb200_last_error().decode()


def test_noalloc_plan_at_the_documented_limit_and_with_no_tokens():
    """Exactly 65536 entries over 512 experts fill the built-in scratch to its last word (64 chunks x 512 counters) and
    need the assign kernel's largest shared-memory footprint; checked against a stable argsort on the host. A call with
    no tokens must leave every expert's segment empty."""
    from oracle import moe as omoe
    tokens, topk, experts, alignment = 8192, 8, 512, 16
    g = torch.Generator().manual_seed(77)
    idx = torch.stack([torch.randperm(experts, generator=g)[:topk] for _ in range(tokens)])
    idx = idx.masked_fill(torch.rand(idx.shape, generator=g) < 0.1, -1)
    dest, start, end = _plan_noalloc(idx, experts, alignment)
    want_dest, _, want_start, want_end = omoe.dispatch_plan(idx, experts, alignment)
    assert torch.equal(dest.cpu(), want_dest) and torch.equal(start.cpu(), want_start) and torch.equal(end.cpu(), want_end)
    _, start, end = _plan_noalloc(idx[:1], experts, alignment, tokens=0)
    assert torch.equal(start, end) and int(end.max()) == 0
