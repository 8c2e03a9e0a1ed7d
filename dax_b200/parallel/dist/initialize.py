from ..config import ParallelConfig
from .coordinator import initialize_dist_coordinator, is_dist_coordinator_initialized
from .parallel_state import initialize_parallel_state, is_parallel_state_initialized


def initialize(parallel_config: ParallelConfig = None, backend: str = None) -> None:
    if parallel_config is None:
        parallel_config = ParallelConfig()
    initialize_dist_coordinator(backend)
    initialize_parallel_state(parallel_config)


def is_initialized() -> bool:
    return is_dist_coordinator_initialized() and is_parallel_state_initialized()
