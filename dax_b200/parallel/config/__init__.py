from .parallel_config import ParallelConfig
