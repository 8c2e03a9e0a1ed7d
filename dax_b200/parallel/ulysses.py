"""Zero-copy, chunkable Ulysses exchanges used by the attention processor.

The two exchanges of the block are written so that neither needs a pack or an unpack copy:

* tokens -> heads.  Every rank holds the projection of its ``s`` tokens for all heads, already
  stored by the producing kernel as ``send[P, s, h*d]`` (slab p = the heads owned by rank p).  Rank p
  must end with ``recv[S, h*d]`` (all tokens, its heads); the block sent by rank r lands at rows
  ``[r*s, (r+1)*s)``.  A chunk is a row range ``[c0, c1)`` of every slab, which is contiguous on
  both sides, so chunks of the same tensor can be exchanged independently while the next chunk is
  still being computed.
* heads -> tokens.  ``src[S, h*d]`` (all tokens, own heads) -> ``recv[P, n, h*d]`` where slab r holds
  the heads of rank r for this rank's token range ``[b0, b1)`` (n = b1 - b0).  The O projection's
  quantiser reads that slab layout in place.

Both are expressed as point-to-point sends and receives of contiguous views (NCCL groups them into
one launch on its own stream; gloo runs them on the CPU for the test-suite).  The equivalent
reference code is ``dax/parallel/patches/wanx2_1_t2v_opt/layer.py:181-222`` plus the micro-batch
loop at ``dax/adapters/wan/attn_adapter.py:241-300``."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class _Done:
    def wait(self):
        return True


class _Works:
    def __init__(self, works):
        self.works = works

    def wait(self):
        for w in self.works:
            w.wait()
        return True


class UlyssesExchange:
    """``skip_comm`` and ``recorded`` exist for measuring how much of the exchange time is hidden:
    with ``skip_comm`` the point-to-point operations are left out (local copies still happen; the results are
    then meaningless), and while ``recorded`` is a list every exchange call is appended to it as a closure that
    re-issues the same operations on the same buffers, so that a step's exchanges can be replayed alone."""

    def __init__(self, group, size: int, rank: int):
        self.group, self.P, self.rank = group, size, rank
        self.global_ranks = (dist.get_process_group_ranks(group) if group is not None and size > 1
                             else list(range(size)))
        self.skip_comm = False
        self.recorded: Optional[list] = None

    def _run(self, ops, async_op: bool):
        if self.recorded is not None and ops:
            kinds = [(o.op, o.tensor, o.peer) for o in ops]
            group = self.group
            self.recorded.append(lambda: _Works(dist.batch_isend_irecv([dist.P2POp(k, t, p, group) for k, t, p in kinds])))
        if not ops or self.skip_comm:
            return _Done()
        works = _Works(dist.batch_isend_irecv(ops))
        if not async_op:
            works.wait()
            return _Done()
        return works

    def tokens_to_heads(self, sends: Sequence[torch.Tensor], recvs: Sequence[torch.Tensor], c0: int, c1: int,
                        async_op: bool = False):
        """Exchange rows ``[c0, c1)`` of every slab of every ``send [P, s, hd]`` into ``recv [P*s, hd]``."""
        P, r = self.P, self.rank
        ops = []
        for send, recv in zip(sends, recvs):
            s = send.shape[1]
            for p in range(P):
                if p != r:
                    ops.append(dist.P2POp(dist.irecv, recv[p * s + c0:p * s + c1], self.global_ranks[p], self.group))
        for send, recv in zip(sends, recvs):
            s = send.shape[1]
            for p in range(P):
                if p != r:
                    ops.append(dist.P2POp(dist.isend, send[p, c0:c1], self.global_ranks[p], self.group))
            recv[r * s + c0:r * s + c1].copy_(send[r, c0:c1])
        return self._run(ops, async_op)

    def heads_to_tokens(self, src: torch.Tensor, recv: torch.Tensor, s: int, b0: int, b1: int,
                        async_op: bool = False):
        """``src [P*s, hd]`` -> ``recv [P, b1-b0, hd]``: slab p of ``recv`` = rank p's heads for this
        rank's tokens ``[b0, b1)``; this rank sends rows ``[p*s + b0, p*s + b1)`` to rank p."""
        P, r = self.P, self.rank
        ops = []
        for p in range(P):
            if p != r:
                ops.append(dist.P2POp(dist.irecv, recv[p], self.global_ranks[p], self.group))
        for p in range(P):
            if p != r:
                ops.append(dist.P2POp(dist.isend, src[p * s + b0:p * s + b1], self.global_ranks[p], self.group))
        recv[r].copy_(src[r * s + b0:r * s + b1])
        return self._run(ops, async_op)

    def heads_to_tokens_group(self, src: torch.Tensor, recv: torch.Tensor, s: int, dests, async_op: bool = False):
        """The same exchange restricted to a group of destination ranks: every rank sends its heads of the
        WHOLE token block of each rank in ``dests``; only the ranks in ``dests`` receive (into
        ``recv [P, s, hd]``, slab p = rank p's heads for this rank's tokens)."""
        P, r = self.P, self.rank
        dests = list(dests)
        ops = []
        if r in dests:
            for p in range(P):
                if p != r:
                    ops.append(dist.P2POp(dist.irecv, recv[p], self.global_ranks[p], self.group))
        for j in dests:
            if j != r:
                ops.append(dist.P2POp(dist.isend, src[j * s:(j + 1) * s], self.global_ranks[j], self.group))
        if r in dests:
            recv[r].copy_(src[r * s:(r + 1) * s])
        return self._run(ops, async_op)


def chunk_bounds(n: int, chunks: int, align: int = 128) -> List[int]:
    """Boundaries of at most ``chunks`` row ranges covering ``[0, n)``, each (but the last) a
    multiple of ``align`` rows so that GEMM tiles never straddle a chunk."""
    chunks = max(1, min(chunks, (n + align - 1) // align))
    per = ((n + chunks - 1) // chunks + align - 1) // align * align
    b = list(range(0, n, per)) + [n]
    return b
