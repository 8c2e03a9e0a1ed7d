"""Asynchronous (overlappable) sequence-parallel primitives for Wan2.1 T2V
(counterpart of ``dax/parallel/patches/wanx2_1_t2v_opt``).

``collect_tokens`` / ``collect_heads`` keep the reference's handle protocol: with ``async_op=True``
the dict passed as ``handle`` receives ``work`` (wait on it before reading), ``output`` (the raw
receive buffer) and ``post_all2all_func`` (turns the receive buffer into the result layout)."""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ...comm.all_to_all import exchange
from ...dist import parallel_state


def _group():
    return parallel_state.get_sequence_parallel_group() if parallel_state.is_parallel_state_initialized() else None


def single_all_to_all(input, seq_world_size, scatter_idx, gather_idx, batch_dim_idx=0, async_op=False, handle=None):
    """One Ulysses exchange of a ``[B, seq, heads, d]`` tensor
    (``dax/parallel/patches/wanx2_1_t2v_opt/layer.py:181-222``, batch-first layouts)."""
    assert batch_dim_idx == 0, "only batch-first layouts are used by the Wan adapter"
    P = seq_world_size
    if scatter_idx >= 2:   # tokens sharded -> heads sharded
        B, s, H, d = input.shape
        assert H % P == 0, f"Number of heads ({H}) must be divisible by the sequence parallel size ({P})!"
        h = H // P
        send = input.reshape(B, s, P, h, d).permute(2, 0, 1, 3, 4).contiguous()
        res_shape = (B, P * s, h, d)

        def post(out):
            return out.view(res_shape) if B == 1 else out.permute(1, 0, 2, 3, 4).reshape(res_shape)
    else:                  # heads sharded -> tokens sharded
        B, S, h, d = input.shape
        assert S % P == 0, f"Sequence length ({S}) must be divisible by the sequence parallel size ({P})!"
        s = S // P
        send = input.reshape(B, P, s, h, d).transpose(0, 1).contiguous()
        res_shape = (B, s, P * h, d)

        def post(out):
            return out.permute(1, 2, 0, 3, 4).reshape(res_shape)
    if P == 1:
        recv, work = send, None
    else:
        recv, work = exchange(send, _group(), async_op=async_op)
    if async_op:
        handle["work"] = work if work is not None else _DoneWork()
        handle["output"] = recv
        handle["post_all2all_func"] = post
        return recv
    return post(recv)


class _DoneWork:
    def wait(self):
        return True


def collect_tokens(x, seq_world_size, async_op=False, handle=None):
    """(B, s, H, d) -> (B, S, H/P, d)"""
    return single_all_to_all(x, seq_world_size, 2, 1, 0, async_op=async_op, handle=handle)


def collect_heads(x, seq_world_size, async_op=False, handle=None):
    """(B, S, H/P, d) -> (B, s, H, d)"""
    return single_all_to_all(x, seq_world_size, 1, 2, 0, async_op=async_op, handle=handle)


def collect_tokens_packed_qkv(q, k, v, seq_world_size, async_op=False, handle=None):
    """Q, K and V in ONE collective (``.../wanx2_1_t2v_opt/all_to_all.py:4-18``)."""
    B = q.shape[0]
    res = single_all_to_all(torch.cat([q, k, v], dim=0), seq_world_size, 2, 1, 0, async_op=False)
    return res[:B], res[B:2 * B], res[2 * B:]


def micro_batch_bounds(s: int, m: int) -> List[int]:
    """Boundaries of ``m`` nearly equal micro-batches of a rank's ``s`` tokens (the first ``s % m``
    get one token more).  The reference requires ``S % (P*m) == 0`` and silently drops tokens
    otherwise; uneven sizes are handled here because 480p at 8 ranks gives s = 4095."""
    base, rem = divmod(s, m)
    b = [0]
    for i in range(m):
        b.append(b[-1] + base + (1 if i < rem else 0))
    return b


def micro_batch_project_O_strategy(tensor, micro_batch_times, gpu_nums):
    """Split ``[B, S, h, d]`` into micro-batches for the O path: micro-batch i holds, for every
    destination rank j, the i-th slice of that rank's token block
    (``.../wanx2_1_t2v_opt/micro_batch_layer.py:1-29``)."""
    b, S, n, d = tensor.shape
    P, m = gpu_nums, micro_batch_times
    s = S // P
    bounds = micro_batch_bounds(s, m)
    view = tensor[:, :P * s].reshape(b, P, s, n, d)
    return [view[:, :, bounds[i]:bounds[i + 1]].reshape(b, P * (bounds[i + 1] - bounds[i]), n, d) for i in range(m)]


def split(x, world_size, dim):
    """This rank's equal share of ``x`` along ``dim`` (``.../wanx2_1_t2v_opt/split.py``)."""
    if world_size == 1:
        return x
    size = x.size(dim)
    assert size % world_size == 0, (f"The dimension to split ({size}) is not a multiple of world size "
                                    f"({world_size}), cannot split tensor evenly")
    rank = dist.get_rank(_group())
    return x.narrow(dim, rank * (size // world_size), size // world_size).contiguous()
