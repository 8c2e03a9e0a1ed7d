from dataclasses import dataclass


@dataclass
class ParallelConfig:
    """Degrees of the two mesh dimensions (``dax/parallel/config/parallel_config.py:4-7``).
    ``dp_degree = -1`` means "whatever is left": world_size // sp_degree.  Data parallelism is
    replicas only: nothing in the hot path communicates across it."""
    dp_degree: int = -1
    sp_degree: int = 1
