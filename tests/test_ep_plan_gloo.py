"""World-size-2 CPU test (gloo) of the expert-parallel dispatch protocol as restated in the oracle: ranks exchange
per-expert counts, derive the same plan, and the rows every rank would push land exactly where a global stable
sort of all entries (rank-major, then entry order) puts them."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as omoe

EXPERTS, TOPK, TOKENS, ALIGN = 8, 2, 23, 16


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        idx = torch.randint(-1, EXPERTS, (TOKENS + rank, TOPK))
        counts = omoe.ep_counts(idx, EXPERTS)
        gathered = [torch.zeros_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        all_counts = torch.stack(gathered)
        my_base, start, end = omoe.ep_plan(all_counts, rank, ALIGN)
        dest = omoe.ep_dest_rows(idx, my_base, EXPERTS)
        out[rank] = (idx, dest, start, end)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_plan_matches_global_stable_sort():
    world = 2
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    per_rank = EXPERTS // world
    # global reference: all entries concatenated in rank order, stably sorted by expert, per owner rank
    all_idx = torch.cat([out[r][0].reshape(-1) for r in range(world)])
    for owner in range(world):
        want_dest, _, want_start, want_end = omoe.dispatch_plan(all_idx.view(-1, 1), per_rank, ALIGN, expert_lo=owner * per_rank)
        got = torch.cat([torch.where((out[r][0].reshape(-1) // per_rank == owner) & (out[r][0].reshape(-1) >= 0),
                                     out[r][1], torch.full_like(out[r][1], -1)) for r in range(world)])
        assert torch.equal(got, want_dest.to(torch.int64))
        assert torch.equal(out[owner][2], want_start.to(torch.int64))
        assert torch.equal(out[owner][3], want_end.to(torch.int64))


SP_EXPERTS, SP_TOPK, SP_TOKENS, SP_GUESTS = 16, 4, 400, 2


def _worker_spill(rank, world, port, out):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        torch.manual_seed(300 + rank)
        logits = torch.randn(SP_TOKENS + 7 * rank, SP_EXPERTS)
        logits[:, :3] += 4.0  # three experts of rank 0 take most of the rows
        idx, _ = omoe.route_sigmoid_topk(logits, SP_TOPK)
        counts = omoe.ep_counts(idx, SP_EXPERTS)
        gathered = [torch.zeros_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        all_counts = torch.stack(gathered)
        my_base, my_dest, my_slot, start, end, guest = omoe.ep_plan_with_spill(all_counts, rank, ALIGN, SP_GUESTS)
        dest = omoe.ep_dest_rows(idx, my_base, SP_EXPERTS)
        out[rank] = dict(idx=idx, dest=dest, my_dest=my_dest, my_slot=my_slot, start=start, end=end, guest=guest, counts=all_counts)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_plan_with_guest_experts_places_every_row_once():
    """Hot-expert row spill over gloo: both ranks derive their plans from the exchanged counts alone. Every entry of every
    rank must land on a distinct row of the rank and slot its plan names, inside that slot's segment, ordered by (source
    rank, entry) within the slot; rows really move, and a guest slot hosts an expert of the other rank."""
    world = 2
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker_spill, args=(world, _free_port(), out), nprocs=world, join=True)
    per_rank = SP_EXPERTS // world
    assert torch.equal(out[0]['counts'], out[1]['counts'])
    landed = {r: {} for r in range(world)}  # computing rank -> row -> (slot, source rank, entry)
    for src in range(world):
        o = out[src]
        flat = o['idx'].reshape(-1)
        for entry, (e, row) in enumerate(zip(flat.tolist(), o['dest'].tolist())):
            d, v = int(o['my_dest'][e]), int(o['my_slot'][e])
            assert row not in landed[d], 'two entries on one row'
            assert int(out[d]['start'][v]) <= row < int(out[d]['end'][v]), 'row outside its slot'
            hosted = e if v < per_rank else int(out[d]['guest'][v - per_rank])
            assert hosted == e and (v >= per_rank) == (d != e // per_rank)
            landed[d][row] = (v, src, entry)
    moved = 0
    for d in range(world):
        rows = sorted(landed[d])
        assert len(rows) == int((out[d]['end'] - out[d]['start']).sum()), 'segments hold exactly the rows that landed'
        keys = [landed[d][r] for r in rows]
        assert keys == sorted(keys), 'rows of a slot are ordered by (source rank, entry)'
        moved += sum(1 for v, _, _ in keys if v >= per_rank)
        assert all(int(s) % ALIGN == 0 for s in out[d]['start'])
    assert moved > 0
    as_routed = [int(out[0]['counts'][:, r * per_rank:(r + 1) * per_rank].sum()) for r in range(world)]
    computed = [len(landed[r]) for r in range(world)]
    assert sum(as_routed) == sum(computed) and max(computed) < max(as_routed)
