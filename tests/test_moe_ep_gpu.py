"""Expert-parallel MoE layer on 2 GPUs (one process per GPU, NCCL for the rendezvous, P2P stores for the data):
every rank's output must match the single-rank CPU oracle evaluated on that rank's tokens, and the rows each rank
received must be the ones the oracle's rank-major plan predicts. Skipped when fewer than 2 GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

EXPERTS, TOPK, HIDDEN, INTER = 8, 3, 512, 256
TOKENS = (150, 97)


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _rank_inputs(rank):
    from tests.helpers import moe_case
    c = moe_case(TOKENS[rank], HIDDEN, INTER, EXPERTS, TOPK, seed=500 + rank, masked_ratio=0.15)
    w = moe_case(4, HIDDEN, INTER, EXPERTS, TOPK, seed=77)  # the same weights on every rank
    for k in ('l1_q', 'l1_sf', 'l2_q', 'l2_sf'):
        c[k] = w[k]
    return c


def _shared_weights():
    from oracle import quant
    torch.manual_seed(4242)
    s1_q, s1_sf = quant.quantize_fp8_per_token((torch.randn(2 * INTER, HIDDEN) * 0.02).bfloat16(), 32)
    s2_q, s2_sf = quant.quantize_fp8_per_token((torch.randn(HIDDEN, INTER) * 0.02).bfloat16(), 32)
    return s1_q, s1_sf, s2_q, s2_sf


def _worker(rank, world, port, results):
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    from oracle import quant
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        c = _rank_inputs(rank)
        per_rank = EXPERTS // world
        mine = slice(rank * per_rank, (rank + 1) * per_rank)
        buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, EXPERTS, max(TOKENS), TOPK, HIDDEN, INTER, num_shared_experts=1)
        l1_sf = dg.transform_sf_into_required_layout(c['l1_sf'][mine].cuda(), 2 * INTER, HIDDEN, (1, 32), per_rank)
        l2_sf = dg.transform_sf_into_required_layout(c['l2_sf'][mine].cuda(), HIDDEN, INTER, (1, 32), per_rank)
        l1, l2 = dg.transform_weights_for_mega_moe((c['l1_q'][mine].cuda(), l1_sf), (c['l2_q'][mine].cuda(), l2_sf))
        t = TOKENS[rank]
        stats = torch.zeros(per_rank, dtype=torch.int32, device='cuda')
        ys = []
        for _ in range(2):  # two calls: the barrier epochs and the buffers must survive reuse
            buf.x[:t].copy_(c['x_q'].cuda())
            buf.x_sf[:t].copy_(quant.pack_ue8m0(c['x_sf']).cuda())
            buf.topk_idx[:t].copy_(c['topk_idx'].cuda())
            buf.topk_weights[:t].copy_(c['topk_weights'].cuda())
            y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
            dg.fp8_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats)
            status = _lib.device_status()
            assert status[0] == 0, status
            ys.append(y.cpu())
        # third call: BF16 rows quantised while they are pushed to their owners must give the same bits
        y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe_bf16_input(y, c['x'].cuda(), l1, l2, buf, cumulative_local_expert_recv_stats=None)
        assert _lib.device_status()[0] == 0
        ys.append(y.cpu())
        # fourth call: shared experts (rank-local FP8 x FP8 MLP) as an extra combine slot
        s1_q, s1_sf, s2_q, s2_sf = _shared_weights()
        sl1, sl2 = dg.transform_weights_for_mega_moe(
            (s1_q.cuda(), dg.transform_sf_into_required_layout(s1_sf.cuda(), 2 * INTER, HIDDEN, (1, 32))),
            (s2_q.cuda(), dg.transform_sf_into_required_layout(s2_sf.cuda(), HIDDEN, INTER, (1, 32))))
        y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe(y, l1, l2, buf, shared_l1_weights=sl1, shared_l2_weights=sl2, fast_math=False)
        assert _lib.device_status()[0] == 0
        ys.append(y.cpu())
        lay = buf.layout
        end = buf.buffer[lay['expert_end']:lay['expert_end'] + per_rank * 4].view(torch.int32).cpu()
        start = buf.buffer[lay['expert_start']:lay['expert_start'] + per_rank * 4].view(torch.int32).cpu()
        dest = buf.buffer[lay['dest_row']:lay['dest_row'] + t * TOPK * 4].view(torch.int32).cpu()
        results[rank] = dict(y0=ys[0], y1=ys[1], y_fused=ys[2], y_shared=ys[3], start=start, end=end, dest=dest, stats=stats.cpu())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_two_rank_layer_matches_oracle():
    import torch.multiprocessing as mp
    from oracle import moe as omoe
    from oracle import quant
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    cases = [_rank_inputs(r) for r in range(world)]
    all_counts = torch.stack([omoe.ep_counts(c['topk_idx'], EXPERTS) for c in cases])
    for rank in range(world):
        c, got = cases[rank], results[rank]
        want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
        assert torch.equal(got['y0'], got['y1']), 'two calls on the same buffer must give the same bits'
        assert torch.equal(got['y0'], got['y_fused']), 'the fused prologue must give the same bits'
        assert not torch.isnan(got['y0'].float()).any()
        assert quant.calc_diff(got['y0'], want) <= 2e-3
        my_base, want_start, want_end = omoe.ep_plan(all_counts, rank, 128)
        assert torch.equal(got['start'].long(), want_start) and torch.equal(got['end'].long(), want_end)
        assert torch.equal(got['dest'].long(), omoe.ep_dest_rows(c['topk_idx'], my_base, EXPERTS))
        assert torch.equal(got['stats'].long(), 2 * (want_end - want_start))
        shared = omoe.shared_expert_rows(c['x_q'], c['x_sf'], *_shared_weights())
        want_shared = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'],
                                     c['l2_sf'], shared_rows=shared)
        assert quant.calc_diff(got['y_shared'], want_shared) <= 2e-3


# ---- NVFP4 form of the same layer: rows cross ranks as packed E2M1 + UE4M3 scales, one input scale for all ranks
NV_HIDDEN, NV_INTER = 512, 256
NV_X_SCALE = 6.0 / (6.0 * 448.0)


def _rank_inputs_nvfp4(rank):
    from oracle import nvfp4 as onv
    from tests.helpers import moe_case_nvfp4
    c = moe_case_nvfp4(TOKENS[rank], NV_HIDDEN, NV_INTER, EXPERTS, TOPK, seed=600 + rank, masked_ratio=0.15)
    c['x_scale'] = torch.tensor(NV_X_SCALE)
    c['x_q'], c['x_sf'], _ = onv.quantize_nvfp4(c['x'], c['x_scale'])
    w = moe_case_nvfp4(4, NV_HIDDEN, NV_INTER, EXPERTS, TOPK, seed=78)  # the same weights on every rank
    for k in ('l1_q', 'l1_sf', 'l1_scales', 'l2_q', 'l2_sf', 'l2_scales'):
        c[k] = w[k]
    return c


def _worker_nvfp4(rank, world, port, act_scale, results):
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        c = _rank_inputs_nvfp4(rank)
        per_rank = EXPERTS // world
        mine = slice(rank * per_rank, (rank + 1) * per_rank)
        buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, EXPERTS, max(TOKENS), TOPK, NV_HIDDEN, NV_INTER,
                                              mma_type='nvfp4xnvfp4')
        l1 = (c['l1_q'][mine].cuda(), dg.pack_nvfp4_sf_mn_major(c['l1_sf'][mine].cuda()), c['l1_scales'][mine].cuda())
        l2 = (c['l2_q'][mine].cuda(), dg.pack_nvfp4_sf_mn_major(c['l2_sf'][mine].cuda()), c['l2_scales'][mine].cuda())
        l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
        t = TOKENS[rank]
        ys = []
        for _ in range(2):
            buf.x[:t].copy_(c['x_q'].cuda())
            buf.x_sf[:t].copy_(c['x_sf'].view(torch.uint8).contiguous().view(torch.int32).cuda())
            buf.topk_idx[:t].copy_(c['topk_idx'].cuda())
            buf.topk_weights[:t].copy_(c['topk_weights'].cuda())
            y = torch.full((t, NV_HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
            dg.nvfp4_mega_moe(y, l1, l2, buf, c['x_scale'].cuda(), torch.tensor(act_scale).cuda(), fast_math=False)
            status = _lib.device_status()
            assert status[0] == 0, status
            ys.append(y.cpu())
        results[rank] = dict(y0=ys[0], y1=ys[1])
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_two_rank_nvfp4_layer_matches_oracle():
    import torch.multiprocessing as mp
    from oracle import nvfp4 as onv
    from oracle import quant
    world = 2
    cases = [_rank_inputs_nvfp4(r) for r in range(world)]
    act_scale = max(float(onv.calibrate_act_scale(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'],
                                                  c['l1_q'], c['l1_sf'], c['l1_scales'])) for c in cases)
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker_nvfp4, args=(world, _free_port(), act_scale, results), nprocs=world, join=True)
    for rank in range(world):
        c, got = cases[rank], results[rank]
        want = onv.moe_layer_nvfp4(c['x_q'], c['x_sf'], c['x_scale'], c['topk_idx'], c['topk_weights'], c['l1_q'],
                                   c['l1_sf'], c['l1_scales'], c['l2_q'], c['l2_sf'], c['l2_scales'], torch.tensor(act_scale))
        assert torch.equal(got['y0'], got['y1'])
        assert not torch.isnan(got['y0'].float()).any()
        assert quant.calc_diff(got['y0'], want) <= 2e-3
