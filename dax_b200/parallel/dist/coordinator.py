"""Rank bookkeeping and process-group start-up (counterpart of ``dax/parallel/dist/coordinator.py``).

One process per GPU, launched by torchrun: ranks come from ``RANK`` / ``WORLD_SIZE`` /
``LOCAL_RANK`` / ``LOCAL_WORLD_SIZE``.  The default process group is created here if the caller has
not done so: NCCL when CUDA is available, gloo otherwise (the CPU test-suite runs the same host
logic over gloo)."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def get_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else int(os.environ.get("RANK", 0))


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else int(os.environ.get("WORLD_SIZE", 1))


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", 0))


def get_local_world_size() -> int:
    return int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", 1)))


def is_main_process() -> bool:
    return get_rank() == 0


def is_dist_coordinator_initialized() -> bool:
    return dist.is_initialized()


def initialize_dist_coordinator(backend: str | None = None, timeout_s: float = 600.0) -> None:
    if dist.is_initialized():
        return
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if use_cuda:
        torch.cuda.set_device(get_local_rank())
    kwargs = {}
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", get_local_rank())
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)


def destroy() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
