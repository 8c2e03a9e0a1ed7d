from .all_to_all import _all_to_all_4D, exchange
from .split_gather import _gather, _split
