"""Synchronous Ulysses exchange on ``[B, seq, heads, d]`` tensors (the ``overlap_comm=False`` switch;
counterpart of ``dax/parallel/comm/all_to_all.py:26-88``).

Both directions are one equal-split ``all_to_all_single`` between a send buffer ``[P, ...]`` and a
receive buffer ``[P, ...]``.  Unlike the reference there is no device-wide synchronise after the
collective: the collective is stream-ordered, and the consumer runs on the same stream."""
from __future__ import annotations

import torch
import torch.distributed as dist


def exchange(send: torch.Tensor, group=None, async_op: bool = False, recv: torch.Tensor | None = None):
    """Equal-split all-to-all over dim 0 of a contiguous ``[P, ...]`` buffer."""
    if recv is None:
        recv = torch.empty_like(send)
    work = dist.all_to_all_single(recv, send, group=group, async_op=async_op)
    return recv, work


def _all_to_all_4D(input: torch.Tensor, scatter_idx: int = 2, gather_idx: int = 1, group=None) -> torch.Tensor:
    assert input.dim() == 4, f"input must be 4D tensor, got {input.dim()} and shape {input.shape}"
    P = dist.get_world_size(group)
    if scatter_idx == 2 and gather_idx == 1:
        # (B, s, H, d) sharded over tokens -> (B, S, h, d) sharded over heads
        B, s, H, d = input.shape
        assert H % P == 0, f"Number of heads ({H}) must be divisible by the sequence parallel size ({P})!"
        h = H // P
        if P == 1:
            return input.contiguous()
        send = input.reshape(B, s, P, h, d).permute(2, 0, 1, 3, 4).contiguous()  # [P, B, s, h, d]
        recv, _ = exchange(send, group)
        if B == 1:
            return recv.view(1, P * s, h, d)
        return recv.permute(1, 0, 2, 3, 4).reshape(B, P * s, h, d)
    if scatter_idx == 1 and gather_idx == 2:
        # (B, S, h, d) sharded over heads -> (B, s, H, d) sharded over tokens
        B, S, h, d = input.shape
        assert S % P == 0, f"Sequence length ({S}) must be divisible by the sequence parallel size ({P})!"
        s = S // P
        if P == 1:
            return input.contiguous()
        send = input.reshape(B, P, s, h, d).transpose(0, 1).contiguous()  # [P, B, s, h, d]
        recv, _ = exchange(send, group)
        return recv.permute(1, 2, 0, 3, 4).reshape(B, s, P * h, d)
    raise RuntimeError("scatter_idx must be 1 or 2 and gather_idx must be 1 or 2")
