from .initialize import initialize, is_initialized, is_launched_with_torchrun
