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
        # the same layer with both GEMMs through the swapped-operand kernel (tokens on UMMA N)
        _lib.check(_lib.lib().dgb200_set_tuning(b'swap_ab', 1))
        try:
            y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
            dg.fp8_fp4_mega_moe_bf16_input(y, c['x'].cuda(), l1, l2, buf)
            assert _lib.device_status()[0] == 0
        finally:
            _lib.check(_lib.lib().dgb200_set_tuning(b'swap_ab', -1))
        y_swapped = y.cpu()
        # fourth call: shared experts (rank-local FP8 x FP8 MLP) as an extra combine slot
        s1_q, s1_sf, s2_q, s2_sf = _shared_weights()
        sl1, sl2 = dg.transform_weights_for_mega_moe(
            (s1_q.cuda(), dg.transform_sf_into_required_layout(s1_sf.cuda(), 2 * INTER, HIDDEN, (1, 32))),
            (s2_q.cuda(), dg.transform_sf_into_required_layout(s2_sf.cuda(), HIDDEN, INTER, (1, 32))))
        y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe(y, l1, l2, buf, shared_l1_weights=sl1, shared_l2_weights=sl2, fast_math=False)
        assert _lib.device_status()[0] == 0
        ys.append(y.cpu())
        # a second buffer whose allocation history differs between the ranks (rank 0 allocates something else first, rank
        # 1 frees its first buffer before): the flag epochs live in the buffer, so a new buffer starts from zero on every
        # rank no matter where the allocator placed it
        if rank == 0:
            filler = torch.empty(37 << 20, dtype=torch.int8, device='cuda')
        else:
            buf.destroy()
        buf2 = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, EXPERTS, max(TOKENS), TOPK, HIDDEN, INTER, num_shared_experts=1)
        buf2.x[:t].copy_(c['x_q'].cuda())
        buf2.x_sf[:t].copy_(quant.pack_ue8m0(c['x_sf']).cuda())
        buf2.topk_idx[:t].copy_(c['topk_idx'].cuda())
        buf2.topk_weights[:t].copy_(c['topk_weights'].cuda())
        y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe(y, l1, l2, buf2)
        assert _lib.device_status()[0] == 0
        y_second_buffer = y.cpu()
        lay = buf2.layout
        buf = buf2
        end = buf.buffer[lay['expert_end']:lay['expert_end'] + per_rank * 4].view(torch.int32).cpu()
        start = buf.buffer[lay['expert_start']:lay['expert_start'] + per_rank * 4].view(torch.int32).cpu()
        dest = buf.buffer[lay['dest_row']:lay['dest_row'] + t * TOPK * 4].view(torch.int32).cpu()
        results[rank] = dict(y0=ys[0], y1=ys[1], y_fused=ys[2], y_shared=ys[3], y_swapped=y_swapped, y_second_buffer=y_second_buffer, start=start, end=end, dest=dest,
                             stats=stats.cpu())
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
        assert torch.equal(got['y0'], got['y_second_buffer']), 'a second buffer (new flag epochs) must give the same bits'
        assert quant.calc_diff(got['y_swapped'], got['y0']) <= 1e-5, 'tile orientation must not change the result'
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


# ---- hot-expert row spill: skewed routing, rows of hot experts computed by the other rank in a guest slot
SP_EXPERTS, SP_TOPK, SP_TOKENS, SP_GUESTS = 16, 4, (600, 420), 2


def _rank_inputs_spill(rank):
    from oracle import moe as omoe
    from tests.helpers import moe_case
    c = moe_case(SP_TOKENS[rank], HIDDEN, INTER, SP_EXPERTS, SP_TOPK, seed=700 + rank)
    # experts 0..2 (all owned by rank 0) are chosen by almost every token
    logits = c['logits'].clone()
    logits[:, :3] += 4.0
    c['topk_idx'], c['topk_weights'] = omoe.route_sigmoid_topk(logits, SP_TOPK)
    mask = torch.rand(c['topk_idx'].shape, generator=torch.Generator().manual_seed(710 + rank)) < 0.1  # masked slots
    c['topk_idx'] = c['topk_idx'].masked_fill(mask, -1)
    c['topk_weights'] = c['topk_weights'].masked_fill(mask, 0.0)
    w = moe_case(4, HIDDEN, INTER, SP_EXPERTS, SP_TOPK, seed=79)  # the same weights on every rank
    for k in ('l1_q', 'l1_sf', 'l2_q', 'l2_sf'):
        c[k] = w[k]
    return c


def _worker_spill(rank, world, port, results):
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    from oracle import quant
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        c = _rank_inputs_spill(rank)
        per_rank = SP_EXPERTS // world
        mine = slice(rank * per_rank, (rank + 1) * per_rank)
        buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, SP_EXPERTS, max(SP_TOKENS), SP_TOPK, HIDDEN, INTER)
        l1_sf = dg.transform_sf_into_required_layout(c['l1_sf'][mine].cuda(), 2 * INTER, HIDDEN, (1, 32), per_rank)
        l2_sf = dg.transform_sf_into_required_layout(c['l2_sf'][mine].cuda(), HIDDEN, INTER, (1, 32), per_rank)
        l1, l2 = dg.transform_weights_for_mega_moe((c['l1_q'][mine].cuda(), l1_sf), (c['l2_q'][mine].cuda(), l2_sf))
        l1s, l2s = dg.share_weights_for_mega_moe(dist.group.WORLD, l1, l2, num_guest_experts=SP_GUESTS)
        t = SP_TOKENS[rank]
        out = {}
        for name, (w1, w2) in (('plain', (l1, l2)), ('spill', (l1s, l2s)), ('spill_again', (l1s, l2s))):
            buf.x[:t].copy_(c['x_q'].cuda())
            buf.x_sf[:t].copy_(quant.pack_ue8m0(c['x_sf']).cuda())
            buf.topk_idx[:t].copy_(c['topk_idx'].cuda())
            buf.topk_weights[:t].copy_(c['topk_weights'].cuda())
            stats = torch.zeros(per_rank, dtype=torch.int32, device='cuda')
            y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
            dg.fp8_fp4_mega_moe(y, w1, w2, buf, cumulative_local_expert_recv_stats=stats)
            status = _lib.device_status()
            assert status[0] == 0, status
            out['y_' + name] = y.cpu()
            out['stats_' + name] = stats.cpu()
        # the down GEMM writes its rows locally and a separate kernel sends them back (the default sends them from the GEMM's
        # epilogue): same rows, same local combine, same bits
        _lib.check(_lib.lib().dgb200_set_tuning(b'fused_return', 0))
        try:
            y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
            dg.fp8_fp4_mega_moe(y, l1s, l2s, buf)
            assert _lib.device_status()[0] == 0
            out['y_separate_return'] = y.cpu()
        finally:
            _lib.check(_lib.lib().dgb200_set_tuning(b'fused_return', 1))
        # four expert phases on one stream, the dispatch rows of phase q + 1 pushed by the epilogue warps of the gate/up GEMM of
        # phase q: the same rows land in the same places
        _lib.check(_lib.lib().dgb200_set_tuning(b'fused_dispatch', 1))
        try:
            for name in ('y_riding_dispatch', 'y_riding_dispatch_again'):
                y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
                dg.fp8_fp4_mega_moe(y, l1s, l2s, buf)
                assert _lib.device_status()[0] == 0
                out[name] = y.cpu()
        finally:
            _lib.check(_lib.lib().dgb200_set_tuning(b'fused_dispatch', 0))
        # the same calls with the row-moving kernels on the library's second stream, beside the GEMMs of four expert phases
        _lib.check(_lib.lib().dgb200_set_tuning(b'ep_comm_sms', 16))
        try:
            for name, (w1, w2) in (('two_streams', (l1s, l2s)), ('two_streams_plain', (l1, l2)), ('two_streams_again', (l1s, l2s))):
                y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
                dg.fp8_fp4_mega_moe(y, w1, w2, buf)
                assert _lib.device_status()[0] == 0
                out['y_' + name] = y.cpu()
        finally:
            _lib.check(_lib.lib().dgb200_set_tuning(b'ep_comm_sms', 0))
        buf.x[:t].copy_(c['x_q'].cuda())
        y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe(y, l1s, l2s, buf)  # leaves the plan of a spilled, overlapped call in the buffer
        assert _lib.device_status()[0] == 0
        assert torch.equal(y.cpu(), out['y_spill'])
        lay, raw = buf.layout, buf.buffer
        take = lambda key, n: raw[lay[key]:lay[key] + n * 4].view(torch.int32).cpu().clone()
        slots = per_rank + SP_GUESTS
        out.update(start=take('expert_start', slots), end=take('expert_end', slots), dest=take('dest_row', t * SP_TOPK),
                   my_base=take('my_base', SP_EXPERTS), my_dest=take('my_dest', SP_EXPERTS), my_slot=take('my_slot', SP_EXPERTS),
                   guest=take('guest_expert', SP_GUESTS), rank_rows=take('rank_rows', 2 * world))
        results[rank] = out
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_two_rank_hot_expert_spill_matches_oracle():
    """Routing that sends most rows to rank 0's experts: with guest slots the plan moves rows of hot experts to rank 1,
    which computes them with weights fetched from rank 0. Every plan array must equal the oracle's (ep_plan_with_spill),
    the output must match the layer oracle, and must not depend on whether rows were spilled beyond the order of the
    combine's FP32 additions."""
    import torch.multiprocessing as mp
    from oracle import moe as omoe
    from oracle import quant
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker_spill, args=(world, _free_port(), results), nprocs=world, join=True)
    cases = [_rank_inputs_spill(r) for r in range(world)]
    all_counts = torch.stack([omoe.ep_counts(c['topk_idx'], SP_EXPERTS) for c in cases])
    per_rank = SP_EXPERTS // world
    rows_before = [int(all_counts[:, r * per_rank:(r + 1) * per_rank].sum()) for r in range(world)]
    hosted = 0
    for rank in range(world):
        c, got = cases[rank], results[rank]
        want = omoe.moe_layer(c['x_q'], c['x_sf'], c['topk_idx'], c['topk_weights'], c['l1_q'], c['l1_sf'], c['l2_q'], c['l2_sf'])
        assert not torch.isnan(got['y_spill'].float()).any()
        assert quant.calc_diff(got['y_spill'], want) <= 2e-3
        # a row's arithmetic does not depend on the rank that computes it; the tile orientation the layer picks for an
        # expert by its row count may, in the last bits of the FP32 sums
        assert quant.calc_diff(got['y_spill'], got['y_plain']) <= 1e-6
        assert torch.equal(got['y_separate_return'], got['y_spill']), 'returning rows from the GEMM epilogue must not change them'
        assert torch.equal(got['y_riding_dispatch'], got['y_spill']), 'rows pushed by the gate/up GEMM must give the same bits'
        assert torch.equal(got['y_riding_dispatch'], got['y_riding_dispatch_again'])
        assert quant.calc_diff(got['y_two_streams'], got['y_spill']) <= 1e-6
        assert quant.calc_diff(got['y_two_streams_plain'], got['y_spill']) <= 1e-6
        assert torch.equal(got['y_two_streams'], got['y_two_streams_again'])
        assert torch.equal(got['y_spill'], got['y_spill_again']), 'two calls must give the same bits'
        my_base, my_dest, my_slot, start, end, guest = omoe.ep_plan_with_spill(all_counts, rank, 128, SP_GUESTS)
        assert torch.equal(got['my_base'].long(), my_base) and torch.equal(got['my_dest'].long(), my_dest)
        assert torch.equal(got['my_slot'].long(), my_slot) and torch.equal(got['guest'].long(), guest)
        assert torch.equal(got['start'].long(), start) and torch.equal(got['end'].long(), end)
        assert torch.equal(got['dest'].long(), omoe.ep_dest_rows(c['topk_idx'], my_base, SP_EXPERTS))
        owned = all_counts[:, rank * per_rank:(rank + 1) * per_rank].sum(dim=0)
        assert torch.equal(got['stats_spill'].long(), owned) and torch.equal(got['stats_plain'].long(), owned)
        assert got['rank_rows'][:world].tolist() == rows_before
        assert int(got['rank_rows'][world + rank]) == int((end - start).sum())
        hosted += int((guest >= 0).sum())
    assert hosted > 0, 'the case must make at least one expert spill'
    after = results[0]['rank_rows'][world:].tolist()
    assert max(after) - min(after) < max(rows_before) - min(rows_before)


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


# ---- BASELINE expert-parallel configuration at full size on 2 GPUs: 8192 tokens per rank, hidden 7168, 256 experts
# sharded over the ranks, top-8, intermediate 2048, Zipf-biased routing. Weights and activations are drawn and quantised
# on each GPU (the same seed for the weights of an expert on whatever rank owns it).
def _worker_full(rank, world, port, results):
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        tokens, hidden, inter, experts, topk = 8192, 7168, 2048, 256, 8
        per_rank = experts // world
        l1_q = torch.empty((per_rank, 2 * inter, hidden // 2), dtype=torch.int8, device='cuda')
        l1_sf = torch.empty((per_rank, 2 * inter, hidden // 32), dtype=torch.float32, device='cuda')
        l2_q = torch.empty((per_rank, hidden, inter // 2), dtype=torch.int8, device='cuda')
        l2_sf = torch.empty((per_rank, hidden, inter // 32), dtype=torch.float32, device='cuda')
        for e in range(per_rank):
            g = torch.Generator(device='cuda').manual_seed(1000 + rank * per_rank + e)
            w = torch.randn(2 * inter, hidden, device='cuda', dtype=torch.bfloat16, generator=g) * 0.02
            l1_q[e], l1_sf[e] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
            w = torch.randn(hidden, inter, device='cuda', dtype=torch.bfloat16, generator=g) * 0.02
            l2_q[e], l2_sf[e] = dg.utils.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
        l1, l2 = dg.transform_weights_for_mega_moe(
            (l1_q, dg.transform_sf_into_required_layout(l1_sf, 2 * inter, hidden, (1, 32), per_rank)),
            (l2_q, dg.transform_sf_into_required_layout(l2_sf, hidden, inter, (1, 32), per_rank)))
        gen = torch.Generator().manual_seed(2024)
        popularity = torch.empty(experts)
        popularity[torch.randperm(experts, generator=gen)] = 1.0 / torch.arange(1, experts + 1, dtype=torch.float32)
        torch.manual_seed(50 + rank)
        x = torch.randn(tokens, hidden).bfloat16().cuda()
        logits = (torch.randn(tokens, experts) + torch.log(popularity / popularity.sum())).cuda()
        buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, experts, tokens, topk, hidden, inter)
        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe_bf16_input(y, x, l1, l2, buf, logits=logits, fast_math=False)
        assert _lib.device_status()[0] == 0
        idx = buf.topk_idx.cpu()
        # every rank needs every rank's routing for the plan: gather the index tensors over NCCL
        all_idx = [torch.empty_like(buf.topk_idx) for _ in range(world)]
        dist.all_gather(all_idx, buf.topk_idx.contiguous())
        lay = buf.layout
        dest = buf.buffer[lay['dest_row']:lay['dest_row'] + tokens * topk * 4].view(torch.int32).cpu()
        end = buf.buffer[lay['expert_end']:lay['expert_end'] + per_rank * 4].view(torch.int32).cpu()
        # sampled tokens: re-evaluate from the same quantised bits; the weights of remote experts are regenerated here
        x_q, x_sf = dg.utils.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32)
        samples = {}
        for t in (0, 4097, 8191):
            rows = []
            for k in range(topk):
                e = int(idx[t, k])
                g = torch.Generator(device='cuda').manual_seed(1000 + e)
                w1 = torch.randn(2 * inter, hidden, device='cuda', dtype=torch.bfloat16, generator=g) * 0.02
                w2 = torch.randn(hidden, inter, device='cuda', dtype=torch.bfloat16, generator=g) * 0.02
                q1, s1 = dg.utils.per_token_cast_to_fp4(w1, use_ue8m0=True, gran_k=32)
                q2, s2 = dg.utils.per_token_cast_to_fp4(w2, use_ue8m0=True, gran_k=32)
                rows.append((q1.cpu(), s1.cpu(), q2.cpu(), s2.cpu()))
            samples[t] = dict(x_q=x_q[t:t + 1].cpu(), x_sf=x_sf[t:t + 1].cpu(), rows=rows, w=buf.topk_weights[t].cpu(), y=y[t].cpu())
        # the same batch with guest experts: rows of hot experts move to the other rank, whose down GEMM (like everyone's)
        # sends its output rows back from its epilogue; compared with the run above over ALL tokens
        from oracle import quant
        l1s, l2s = dg.share_weights_for_mega_moe(dist.group.WORLD, l1, l2, num_guest_experts=4)
        y_spill = torch.full((tokens, hidden), float('nan'), dtype=torch.bfloat16, device='cuda')
        dg.fp8_fp4_mega_moe_bf16_input(y_spill, x, l1s, l2s, buf, logits=logits, fast_math=False)
        assert _lib.device_status()[0] == 0
        take = lambda key, n: buf.buffer[lay[key]:lay[key] + n * 4].view(torch.int32).cpu().clone()
        spill = dict(diff=float(quant.calc_diff(y_spill.cpu(), y.cpu())), same_rows=int((y_spill == y).all(dim=1).sum()),
                     dest=take('dest_row', tokens * topk), start=take('expert_start', per_rank + 4), end=take('expert_end', per_rank + 4),
                     my_dest=take('my_dest', experts), my_slot=take('my_slot', experts), guest=take('guest_expert', 4))
        results[rank] = dict(idx=idx, all_idx=[a.cpu() for a in all_idx], dest=dest, end=end, logits=logits.cpu(), samples=samples,
                             spill=spill)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_two_rank_full_size_plan_and_sampled_tokens():
    import torch.multiprocessing as mp
    from oracle import moe as omoe
    from oracle import quant
    world, experts, topk, hidden = 2, 256, 8, 7168
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker_full, args=(world, _free_port(), results), nprocs=world, join=True)
    all_counts = torch.stack([omoe.ep_counts(results[r]['idx'], experts) for r in range(world)])
    for rank in range(world):
        got = results[rank]
        want_idx, _ = omoe.route_sigmoid_topk(got['logits'], topk)
        assert torch.equal(got['idx'], want_idx), 'routing must be bit-exact'
        my_base, _, want_end = omoe.ep_plan(all_counts, rank, 128)
        assert torch.equal(got['end'].long(), want_end)
        assert torch.equal(got['dest'].long(), omoe.ep_dest_rows(got['idx'], my_base, experts))
        for t, s in got['samples'].items():
            acc = torch.zeros(hidden)
            for k in range(topk):
                q1, s1, q2, s2 = s['rows'][k]
                a1 = quant.dequantize_fp8(s['x_q'], s['x_sf'], 32) @ quant.dequantize_fp4(q1, s1, 32).T
                # transform_weights_for_mega_moe reorders rows only: the untransformed [gate | up] order is what the oracle takes
                a2_q, a2_sf = omoe.swiglu_requant(a1, s['w'][k:k + 1], None)
                a2 = quant.dequantize_fp8(a2_q, a2_sf, 32) @ quant.dequantize_fp4(q2, s2, 32).T
                acc += a2.bfloat16().float()[0]
            assert quant.calc_diff(s['y'], acc.bfloat16()) <= 2e-3
        # guest experts at full size: the plan is the oracle's, rows were moved, and all 8192 outputs agree with the run
        # that kept every expert's rows on its owner (most of them bit for bit: only the tile orientation chosen for an
        # expert whose row count changed can alter the last bits of an FP32 sum)
        sp = got['spill']
        my_base, my_dest, my_slot, start, end, guest = omoe.ep_plan_with_spill(all_counts, rank, 128, 4)
        assert torch.equal(sp['my_dest'].long(), my_dest) and torch.equal(sp['my_slot'].long(), my_slot)
        assert torch.equal(sp['guest'].long(), guest) and torch.equal(sp['start'].long(), start) and torch.equal(sp['end'].long(), end)
        assert torch.equal(sp['dest'].long(), omoe.ep_dest_rows(got['idx'], my_base, experts))
        assert sp['diff'] <= 1e-6 and sp['same_rows'] >= 8192 * 9 // 10, sp
    assert sum(int((results[r]['spill']['guest'] >= 0).sum()) for r in range(world)) > 0


# ---- the BF16 layer on 2 ranks: the same push / barrier / pull protocol with BF16 rows and no scale factors
def _rank_inputs_bf16(rank):
    from oracle import moe as omoe
    torch.manual_seed(700 + rank)
    t = TOKENS[rank]
    x = torch.randn(t, HIDDEN).bfloat16()
    idx, w = omoe.route_sigmoid_topk(torch.randn(t, EXPERTS), TOPK)
    mask = torch.rand(idx.shape) < 0.15
    idx, w = idx.masked_fill(mask, -1), w.masked_fill(mask, 0.0)
    torch.manual_seed(79)  # the same weights on every rank
    w1 = (torch.randn(EXPERTS, 2 * INTER, HIDDEN) * 0.05).bfloat16()
    w2 = (torch.randn(EXPERTS, HIDDEN, INTER) * 0.05).bfloat16()
    return dict(x=x, topk_idx=idx, topk_weights=w, w1=w1, w2=w2)


def _worker_bf16(rank, world, port, results):
    import torch.distributed as dist
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        c = _rank_inputs_bf16(rank)
        per_rank = EXPERTS // world
        mine = slice(rank * per_rank, (rank + 1) * per_rank)
        buf = dg.get_symm_buffer_for_mega_moe(dist.group.WORLD, EXPERTS, max(TOKENS), TOPK, HIDDEN, INTER,
                                              mma_type='bf16xbf16')
        l1, l2 = dg.transform_weights_for_mega_moe(c['w1'][mine].cuda(), c['w2'][mine].cuda())
        t = TOKENS[rank]
        ys = []
        for _ in range(2):
            buf.x[:t].copy_(c['x'].cuda())
            buf.topk_idx[:t].copy_(c['topk_idx'].cuda())
            buf.topk_weights[:t].copy_(c['topk_weights'].cuda())
            y = torch.full((t, HIDDEN), float('nan'), dtype=torch.bfloat16, device='cuda')
            dg.bf16_mega_moe(y, l1, l2, buf, fast_math=False)
            status = _lib.device_status()
            assert status[0] == 0, status
            ys.append(y.cpu())
        results[rank] = dict(y0=ys[0], y1=ys[1])
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs 2 GPUs')
def test_two_rank_bf16_layer_matches_oracle():
    import torch.multiprocessing as mp
    from oracle import moe as omoe
    from oracle import quant
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker_bf16, args=(world, _free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        c, got = _rank_inputs_bf16(rank), results[rank]
        want = omoe.moe_layer_bf16(c['x'], c['topk_idx'], c['topk_weights'], c['w1'], c['w2'])
        assert torch.equal(got['y0'], got['y1'])
        assert not torch.isnan(got['y0'].float()).any()
        assert quant.calc_diff(got['y0'], want) < 1e-4
