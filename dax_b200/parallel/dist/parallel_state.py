"""Sequence-parallel / data-parallel process groups (counterpart of
``dax/parallel/dist/parallel_state.py``).  Ranks are laid out as a ``(dp, sp)`` grid with ``sp``
fastest, so the ranks of one sequence-parallel group are consecutive (and, with one node, share
NVSwitch)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import ParallelConfig
from .coordinator import get_local_rank, get_rank, get_world_size

PARALLEL_STATE = None


class ParallelState:
    def __init__(self, parallel_config: ParallelConfig):
        self.parallel_config = parallel_config
        self.world_size = get_world_size()
        sp, dp = parallel_config.sp_degree, parallel_config.dp_degree
        assert sp >= 1, sp
        assert sp <= self.world_size, f"Invalid parallel dims: sp({sp}) > WORLD_SIZE({self.world_size})"
        if dp == -1:
            parallel_config.dp_degree = dp = self.world_size // sp
        assert dp >= 1, dp
        assert dp * sp == self.world_size, f"Invalid parallel dims: dp({dp}) * sp({sp}) != WORLD_SIZE({self.world_size})"
        rank = get_rank()
        self.sp_group = self.dp_group = None
        self.sp_ranks = self.dp_ranks = None
        # every rank must create every group, in the same order
        for d in range(dp):
            ranks = list(range(d * sp, (d + 1) * sp))
            g = dist.new_group(ranks) if self.world_size > 1 else None
            if rank in ranks:
                self.sp_group, self.sp_ranks = g, ranks
        for s in range(sp):
            ranks = list(range(s, self.world_size, sp))
            g = dist.new_group(ranks) if self.world_size > 1 else None
            if rank in ranks:
                self.dp_group, self.dp_ranks = g, ranks
        self.sp_size, self.sp_rank = sp, rank % sp
        self.dp_size, self.dp_rank = dp, rank // sp


def is_parallel_state_initialized() -> bool:
    return PARALLEL_STATE is not None


def initialize_parallel_state(parallel_config: ParallelConfig) -> None:
    global PARALLEL_STATE
    if PARALLEL_STATE is None:
        PARALLEL_STATE = ParallelState(parallel_config)
        if torch.cuda.is_available():
            torch.cuda.set_device(get_local_rank())


def reset_parallel_state() -> None:
    global PARALLEL_STATE
    PARALLEL_STATE = None


def get_data_parallel_group():
    return PARALLEL_STATE.dp_group


def get_data_parallel_size() -> int:
    return PARALLEL_STATE.dp_size


def get_data_parallel_rank() -> int:
    return PARALLEL_STATE.dp_rank


def get_data_parallel_all_ranks():
    return PARALLEL_STATE.dp_ranks


def get_sequence_parallel_group():
    return PARALLEL_STATE.sp_group


def get_sequence_parallel_size() -> int:
    return PARALLEL_STATE.sp_size


def get_sequence_parallel_rank() -> int:
    return PARALLEL_STATE.sp_rank


def get_sequence_parallel_all_ranks():
    return PARALLEL_STATE.sp_ranks


def is_enable_sequence_parallel() -> bool:
    return is_parallel_state_initialized() and get_sequence_parallel_size() > 1
