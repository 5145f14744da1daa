"""Process-group helpers with the names of the reference's deep_gemm/utils/dist.py:10-74, so that its multi-GPU
test and benchmark scripts import unchanged: one process per GPU, NCCL over 127.0.0.1 unless MASTER_ADDR says
otherwise.  Only the Mega MoE forward uses a process group here (for the symmetric-memory rendezvous)."""
from __future__ import annotations

import inspect
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

_local_rank: Optional[int] = None


def init_dist(local_rank: int, num_local_ranks: int) -> Tuple[int, int, dist.ProcessGroup]:
    """Join the job as local rank `local_rank` of `num_local_ranks` on this node; WORLD_SIZE / RANK count nodes,
    as in the reference.  Returns (rank, world size, a group of all ranks)."""
    global _local_rank
    _local_rank = local_rank
    nodes, node = int(os.getenv("WORLD_SIZE", 1)), int(os.getenv("RANK", 0))
    kwargs = dict(backend="nccl",
                  init_method=f"tcp://{os.getenv('MASTER_ADDR', '127.0.0.1')}:{os.getenv('MASTER_PORT', '8361')}",
                  world_size=nodes * num_local_ranks, rank=node * num_local_ranks + local_rank)
    if "device_id" in inspect.signature(dist.init_process_group).parameters:
        kwargs["device_id"] = torch.device("cuda", local_rank)
    torch.cuda.set_device(local_rank)
    dist.init_process_group(**kwargs)
    torch.set_default_device("cuda")
    return dist.get_rank(), dist.get_world_size(), dist.new_group(list(range(nodes * num_local_ranks)))


def uneven_all_gather(tensor: torch.Tensor, dim: int = 0, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Concatenation along `dim` of every rank's tensor; the extents along `dim` may differ between ranks."""
    world = dist.get_world_size(group)
    mine = torch.tensor([tensor.shape[dim]], dtype=torch.long, device=tensor.device)
    sizes = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(sizes, mine, group=group)
    sizes = [int(s.item()) for s in sizes]
    widest = max(sizes)
    padded = tensor.contiguous()
    if tensor.shape[dim] < widest:
        shape = list(tensor.shape)
        shape[dim] = widest - tensor.shape[dim]
        padded = torch.cat([tensor, tensor.new_zeros(shape)], dim=dim)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p.narrow(dim, 0, n) for p, n in zip(parts, sizes)], dim=dim)


def dist_print(s: str = "", once_in_node: bool = False) -> None:
    """Print on every rank (or on local rank 0 only), then meet at a barrier so that output stays in order."""
    assert _local_rank is not None, "call init_dist first"
    if not once_in_node or _local_rank == 0:
        print(s, flush=True)
    dist.barrier()
