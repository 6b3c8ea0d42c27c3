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
        buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, EXPERTS, max(TOKENS), TOPK, HIDDEN, INTER)
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
        lay = buf.layout
        end = buf.buffer[lay['expert_end']:lay['expert_end'] + per_rank * 4].view(torch.int32).cpu()
        start = buf.buffer[lay['expert_start']:lay['expert_start'] + per_rank * 4].view(torch.int32).cpu()
        dest = buf.buffer[lay['dest_row']:lay['dest_row'] + t * TOPK * 4].view(torch.int32).cpu()
        results[rank] = dict(y0=ys[0], y1=ys[1], start=start, end=end, dest=dest, stats=stats.cpu())
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
        assert not torch.isnan(got['y0'].float()).any()
        assert quant.calc_diff(got['y0'], want) <= 2e-3
        my_base, want_start, want_end = omoe.ep_plan(all_counts, rank, 16)
        assert torch.equal(got['start'].long(), want_start) and torch.equal(got['end'].long(), want_end)
        assert torch.equal(got['dest'].long(), omoe.ep_dest_rows(c['topk_idx'], my_base, EXPERTS))
        assert torch.equal(got['stats'].long(), 2 * (want_end - want_start))
