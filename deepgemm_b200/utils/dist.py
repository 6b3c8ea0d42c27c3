"""Process-group helpers with the reference's names (deep_gemm/utils/dist.py:10-74), used by its multi-GPU test
drivers: one process per GPU, NCCL, rendezvous over TCP on MASTER_ADDR / MASTER_PORT (default 127.0.0.1:8361)."""
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

_LOCAL_RANK: Optional[int] = None


def init_dist(local_rank: int, num_local_ranks: int) -> Tuple[int, int, dist.ProcessGroup]:
    """Joins the job as rank ``RANK * num_local_ranks + local_rank`` of ``WORLD_SIZE * num_local_ranks`` (RANK and
    WORLD_SIZE count nodes, as in the reference), binds the process to its GPU and makes it the default device.
    Returns (rank, world size, a group over all ranks)."""
    global _LOCAL_RANK
    _LOCAL_RANK = local_rank
    nodes, node = int(os.getenv('WORLD_SIZE', 1)), int(os.getenv('RANK', 0))
    address = f"tcp://{os.getenv('MASTER_ADDR', '127.0.0.1')}:{int(os.getenv('MASTER_PORT', '8361'))}"
    torch.cuda.set_device(local_rank)
    dist.init_process_group('nccl', init_method=address, world_size=nodes * num_local_ranks,
                            rank=node * num_local_ranks + local_rank, device_id=torch.device('cuda', local_rank))
    torch.set_default_device('cuda')
    return dist.get_rank(), dist.get_world_size(), dist.new_group(list(range(nodes * num_local_ranks)))


def uneven_all_gather(tensor: torch.Tensor, dim: int = 0, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Concatenation along ``dim`` of every rank's tensor when the ranks' extents along ``dim`` differ: extents are
    exchanged first, the tensors padded to the largest, gathered, and the padding dropped."""
    world = dist.get_world_size(group)
    mine = torch.tensor([tensor.shape[dim]], dtype=torch.long, device=tensor.device)
    extents = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(extents, mine, group=group)
    extents = [int(e) for e in extents]
    pad = max(extents) - tensor.shape[dim]
    if pad > 0:
        shape = list(tensor.shape)
        shape[dim] = pad
        tensor = torch.cat([tensor, tensor.new_zeros(shape)], dim=dim)
    parts = [torch.empty_like(tensor) for _ in range(world)]
    dist.all_gather(parts, tensor.contiguous(), group=group)
    return torch.cat([part.narrow(dim, 0, extent) for part, extent in zip(parts, extents)], dim=dim)


def dist_print(s: str = '', once_in_node: bool = False) -> None:
    """Prints on every rank (or on local rank 0 only), then a barrier so the lines of one call stay together."""
    assert _LOCAL_RANK is not None, 'init_dist has not been called'
    if _LOCAL_RANK == 0 or not once_in_node:
        print(s, flush=True)
    dist.barrier()
