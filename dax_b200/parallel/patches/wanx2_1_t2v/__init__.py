"""Synchronous sequence-parallel primitives for Wan2.1 T2V
(counterpart of ``dax/parallel/patches/wanx2_1_t2v``)."""
from ...comm.all_to_all import _all_to_all_4D
from ...comm.split_gather import _gather, _split
from ...dist import parallel_state


def collect_tokens(x):
    """(B, s, H, d) -> (B, S, H/P, d)"""
    return _all_to_all_4D(x, 2, 1, parallel_state.get_sequence_parallel_group())


def collect_heads(x):
    """(B, S, H/P, d) -> (B, s, H, d)"""
    return _all_to_all_4D(x, 1, 2, parallel_state.get_sequence_parallel_group())


def gather(x, dim):
    return _gather(x, dim, parallel_state.get_sequence_parallel_group())


def split(x, dim):
    return _split(x, dim, parallel_state.get_sequence_parallel_group())
