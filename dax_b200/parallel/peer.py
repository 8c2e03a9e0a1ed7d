"""Peer-mapped receive buffers for the sequence-parallel attention block.

With NVLink peer access every GPU of the node can store into every other GPU's memory, so the two exchanges of
the Ulysses block need no collective call at all: the kernels that PRODUCE Q, K, V (RMSNorm/RoPE pack, the V
GEMM epilogue) write each head group straight into the owning rank's receive buffer, and the attention kernel's
epilogue writes every query row straight into the receive buffer of the rank that owns that token
(``dax_*_scatter`` entry points).  The transfer rides inside the producing kernel, tile by tile, so nothing is
left to overlap, the projections need not be cut into row chunks and the attention runs as one launch.  What
remains of the exchange is a device-side barrier on the compute stream (a few microseconds): once after the
projections ("every rank's stores into my buffers are complete") and once after the attention.

The buffers are allocated with ``torch.distributed._symmetric_memory`` (peer mappings of one another's
allocations, exchanged once per shape); only this library's own kernels ever touch a peer pointer, with plain
stores.  Multicast objects are not needed and are switched off.  The reference does the same exchanges with
``all_to_all_single`` plus pack / unpack copies (``dax/parallel/patches/wanx2_1_t2v_opt/layer.py:181-222``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class PeerBuffers:
    """Symmetric buffers of one process group, cached by (name, shape, dtype)."""

    BARRIER_TIMEOUT_MS = 60_000  # a rank that never arrives ends the wait with an error instead of a hang

    def __init__(self, group, size: int, rank: int):
        self.group, self.P, self.rank = group, size, rank
        self._bufs: Dict[Tuple, Tuple[torch.Tensor, object]] = {}
        self._any_handle = None
        self.local_only = False  # diagnostic: every "peer" pointer is this rank's own buffer (no NVLink traffic)

    @staticmethod
    def supported() -> bool:
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
        except Exception:
            return False
        return torch.cuda.is_available()

    def get(self, name: str, shape, dtype, device) -> Tuple[torch.Tensor, List[int]]:
        """This rank's buffer and the addresses of every rank's buffer (index = rank in the group) as mapped into
        this process.  Collective on first use of a (name, shape, dtype): all ranks must ask in the same order."""
        import torch.distributed._symmetric_memory as symm
        key = (name, tuple(shape), dtype, str(device))
        hit = self._bufs.get(key)
        if hit is None:
            for k in [k for k in self._bufs if k[0] == name and k[3] == str(device)]:
                del self._bufs[k]  # a resolution change must not leak the old shape
            t = symm.empty(tuple(shape), dtype=dtype, device=device)
            handle = symm.rendezvous(t, self.group)
            hit = self._bufs[key] = (t, handle)
            self._any_handle = handle
        t, handle = hit
        ptrs = [int(p) for p in handle.buffer_ptrs]
        if self.local_only:
            ptrs = [t.data_ptr()] * self.P
        return t, ptrs

    def barrier(self, channel: int = 0) -> None:
        """Device-side barrier of the group on the current stream: returns (in stream order) when every rank has
        reached it, i.e. when every kernel the other ranks enqueued before it, and its stores into this rank's
        buffers, have completed."""
        assert self._any_handle is not None, "barrier before any buffer was allocated"
        self._any_handle.barrier(channel=channel, timeout_ms=self.BARRIER_TIMEOUT_MS)


_PEERS: Dict[int, Optional[PeerBuffers]] = {}


def shared_peer_buffers(group, size: int, rank: int) -> Optional[PeerBuffers]:
    """The peer buffers of a group, or None where they cannot be had.  The first call per group is collective: every
    rank tries a small symmetric allocation and the ranks agree (all-reduce of a flag) on whether ALL of them
    succeeded, so that no rank takes the peer path while another falls back to NCCL."""
    if id(group) in _PEERS:
        return _PEERS[id(group)]
    pb = None
    ok = 0
    if PeerBuffers.supported():
        try:
            pb = PeerBuffers(group, size, rank)
            pb.get("probe", (256,), torch.float32, torch.device("cuda", torch.cuda.current_device()))
            ok = 1
        except Exception:
            ok = 0
    import torch.distributed as dist
    flag = torch.tensor([ok], device="cuda" if torch.cuda.is_available() else "cpu", dtype=torch.int32)
    if group is not None and size > 1 and dist.is_initialized():
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    _PEERS[id(group)] = pb if int(flag.item()) == 1 else None
    return _PEERS[id(group)]
