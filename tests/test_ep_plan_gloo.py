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
