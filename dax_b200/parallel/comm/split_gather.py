"""Sequence split at the DiT entry and gather at its exit
(``dax/parallel/comm/split_gather.py:5-36``)."""
import torch
import torch.distributed as dist


def _gather(inputs: torch.Tensor, dim: int = -1, group=None) -> torch.Tensor:
    P = dist.get_world_size(group)
    if P == 1:
        return inputs
    inputs = inputs.contiguous()
    parts = [torch.empty_like(inputs) for _ in range(P)]
    dist.all_gather(parts, inputs, group=group)
    return torch.cat(parts, dim=dim).contiguous()


def _split(inputs: torch.Tensor, dim: int = -1, group=None) -> torch.Tensor:
    P = dist.get_world_size(group)
    if P == 1:
        return inputs
    size = inputs.size(dim)
    assert size % P == 0, (f"The dimension to split ({size}) is not a multiple of world size ({P}), "
                           "cannot split tensor evenly")
    return inputs.narrow(dim, dist.get_rank(group) * (size // P), size // P).contiguous()
