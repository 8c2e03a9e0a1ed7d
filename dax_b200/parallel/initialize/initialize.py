"""``initialize()``: the one call that turns sequence parallelism on
(``dax/parallel/initialize/initialize.py:14-35``).  The sequence-parallel degree defaults to the
number of ranks on the node, as in the reference."""
import os

from .. import dist
from ..config import ParallelConfig

INITIALIZED = False


def is_launched_with_torchrun() -> bool:
    return "TORCHELASTIC_RUN_ID" in os.environ or ("RANK" in os.environ and "WORLD_SIZE" in os.environ)


def initialize(sp_parallel_size=None, backend=None) -> int:
    global INITIALIZED
    if not is_launched_with_torchrun():
        raise ValueError("Not launched with torchrun")
    if not sp_parallel_size:
        sp_parallel_size = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ["WORLD_SIZE"]))
    dist.initialize(parallel_config=ParallelConfig(sp_degree=sp_parallel_size), backend=backend)
    INITIALIZED = True
    return sp_parallel_size


def is_initialized() -> bool:
    return INITIALIZED
