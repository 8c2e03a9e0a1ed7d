"""Ulysses sequence parallelism (counterpart of ``dax.parallel``)."""
from . import comm, config, dist, initialize, patches
