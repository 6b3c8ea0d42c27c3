"""The expert-parallel plan with guest experts (dgb200_ep_plan_with_guest_experts, the kernel the layer runs on every rank)
against the oracle's restatement (oracle.moe.ep_plan_with_spill), bit for bit, on one GPU: every rank's view of a
Zipf-skewed 8-rank, 256-expert exchange, of a 2-rank case, and of cases where nothing may move."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan(counts, rank, alignment, guests):
    from deepgemm_b200 import _lib
    ranks, experts = counts.shape
    slots = experts // ranks + guests
    dev = lambda n: torch.full((max(n, 1),), -7, dtype=torch.int32, device='cuda')
    out = dict(my_base=dev(experts), my_dest=dev(experts), my_slot=dev(experts), start=dev(slots), end=dev(slots),
               guest=dev(guests), rank_rows=dev(2 * ranks + 1))
    c = counts.to(torch.int32).cuda().contiguous()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(_lib.lib().dgb200_ep_plan_with_guest_experts(
        p(c), ranks, experts, rank, alignment, guests, p(out['my_base']), p(out['my_dest']), p(out['my_slot']), p(out['start']),
        p(out['end']), p(out['guest']), p(out['rank_rows']), _lib.current_stream_ptr()))
    torch.cuda.synchronize()
    return {k: v.cpu().long() for k, v in out.items()}


def _zipf_counts(ranks, experts, tokens, topk, seed):
    g = torch.Generator().manual_seed(seed)
    popularity = torch.empty(experts)
    popularity[torch.randperm(experts, generator=g)] = 1.0 / torch.arange(1, experts + 1, dtype=torch.float32)
    bias = torch.log(popularity / popularity.sum())
    rows = []
    for _ in range(ranks):
        idx = torch.topk(torch.randn(tokens, experts, generator=g) + bias, topk, dim=1).indices
        rows.append(torch.bincount(idx.reshape(-1), minlength=experts))
    return torch.stack(rows)


@pytest.mark.parametrize('ranks,experts,tokens,topk,guests', [
    (8, 256, 2048, 8, 4),   # the shape of the 8-GPU benchmark, fewer tokens
    (8, 256, 2048, 8, 8),
    (4, 64, 512, 4, 2),
    (2, 16, 600, 4, 2),
    (2, 256, 512, 8, 4),    # 128 experts per rank: slot indices beyond 127
])
def test_plan_matches_oracle_on_every_rank(ranks, experts, tokens, topk, guests):
    from oracle import moe as omoe
    counts = _zipf_counts(ranks, experts, tokens, topk, seed=ranks * 1000 + experts + guests)
    per_rank = experts // ranks
    as_routed = [int(counts[:, r * per_rank:(r + 1) * per_rank].sum()) for r in range(ranks)]
    hosted = 0
    for rank in range(ranks):
        got = _plan(counts, rank, 128, guests)
        my_base, my_dest, my_slot, start, end, guest = omoe.ep_plan_with_spill(counts, rank, 128, guests)
        assert torch.equal(got['my_dest'], my_dest) and torch.equal(got['my_slot'], my_slot), f'rank {rank}'
        assert torch.equal(got['my_base'], my_base) and torch.equal(got['guest'][:guests], guest), f'rank {rank}'
        assert torch.equal(got['start'], start) and torch.equal(got['end'], end), f'rank {rank}'
        assert got['rank_rows'][:ranks].tolist() == as_routed
        assert int(got['rank_rows'][ranks + rank]) == int((end - start).sum())
        assert int(got['rank_rows'][2 * ranks]) == -(-int(end[-1]) // 128) * 128
        hosted += int((guest >= 0).sum())
    assert hosted > 0
    computed = got['rank_rows'][ranks:2 * ranks]
    assert int(computed.sum()) == int(counts.sum()) and int(computed.max()) < max(as_routed)


def test_plan_without_guests_and_with_balanced_loads_moves_nothing():
    from oracle import moe as omoe
    counts = _zipf_counts(4, 32, 256, 4, seed=9)
    got = _plan(counts, 2, 128, 0)
    my_base, start, end = omoe.ep_plan(counts, 2, 128)
    assert torch.equal(got['my_base'], my_base) and torch.equal(got['start'], start) and torch.equal(got['end'], end)
    assert torch.equal(got['my_dest'], torch.arange(32) // 8) and torch.equal(got['my_slot'], torch.arange(32) % 8)
    flat = torch.full((4, 32), 40)  # every rank routes the same number of rows to every expert
    got = _plan(flat, 1, 128, 4)
    assert torch.equal(got['guest'][:4], torch.full((4,), -1)) and torch.equal(got['my_dest'], torch.arange(32) // 8)
    assert got['rank_rows'][:4].tolist() == got['rank_rows'][4:8].tolist()


def test_plan_rejects_oversized_problems():
    from deepgemm_b200 import _lib
    one = ctypes.c_void_p(16)
    lib = _lib.lib()
    assert lib.dgb200_ep_plan_with_guest_experts(one, 9, 72, 0, 128, 2, one, one, one, one, one, one, one, None) == 1
    assert lib.dgb200_ep_plan_with_guest_experts(one, 2, 16, 0, 128, 9, one, one, one, one, one, one, one, None) == 1
    assert lib.dgb200_ep_plan_with_guest_experts(one, 2, 512, 0, 128, 4, one, one, one, one, one, one, one, None) == 1
