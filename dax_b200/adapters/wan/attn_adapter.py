"""Attention processor for Wan2.1-style DiT blocks: the per-layer hot path.

``DAXWanAttnProcessor2_0`` keeps the plugin protocol of the reference's processor
(``dax/adapters/wan/attn_adapter.py:53-69``): it is installed with ``Attention.set_processor`` and
called as ``processor(attn, hidden_states, encoder_hidden_states=None, attention_mask=None,
rotary_emb=None)``.  What runs underneath is different.  Installing the processor IS the backend
choice (there is no ``ATTENTION_BACKEND`` dispatch): every step is a kernel of ``libdax_b200``:

  hidden_states [s, D]
    -> per-token quantiser (once for Q, K and V)                           dax_quant_rowwise
    -> INT8/FP8 GEMM + de-quantisation (+ per-row sum of squares)          dax_gemm_dequant
    -> RMSNorm + RoPE + write into the exchange layout [P, s, h*d]         dax_rmsnorm_rope_pack
       (V: the GEMM epilogue writes the exchange layout directly)
    -> tokens->heads exchange, chunk by chunk while the next chunk is projected   (NCCL p2p group)
    -> K smoothing + INT8/FP8 operand preparation, flash attention         dax_attn_prepare/forward
    -> heads->tokens exchange per micro-batch while the next one is attended      (NCCL p2p group)
    -> O projection reading the receive slabs in place                     dax_quant_rowwise + GEMM

RoPE is applied before the exchange with this rank's slice of the rotary table; it is a per-token,
per-head operation, so this equals the reference's rotation after the exchange
(``attn_adapter.py:162-173``).  There is no CPU or eager fallback: non-CUDA input raises."""
from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ... import ops
from ...parallel import dist as para_dist
from ...parallel.patches.wanx2_1_t2v_opt import micro_batch_bounds
from ...parallel.peer import PeerBuffers, shared_peer_buffers
from ...parallel.ulysses import UlyssesExchange, _Done, chunk_bounds
from ...quant.nn.dynamic import Linear as QLinear

HEAD_DIM = 128


class _Buffers:
    """Per-(device, shape) scratch tensors shared by every layer (allocated by torch, once)."""

    def __init__(self):
        self.store: Dict[Tuple, torch.Tensor] = {}

    def get(self, name: str, shape, dtype, device) -> torch.Tensor:
        key = (name, tuple(shape), dtype, str(device))
        t = self.store.get(key)
        if t is None:
            # drop same-name buffers of other shapes so that a resolution change does not leak
            for k in [k for k in self.store if k[0] == name and k[3] == str(device)]:
                del self.store[k]
            t = torch.empty(shape, dtype=dtype, device=device)
            self.store[key] = t
        return t


_BUFFERS = _Buffers()
_ROPE_CACHE: Dict[Tuple, Tuple[torch.Tensor, int, torch.Tensor, torch.Tensor]] = {}


def _rope_tables(rotary_emb: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Complex ``[1, 1, S, 64]`` table -> fp32 cos / sin ``[S, 64]``, cached per table.

    An entry keeps its source tensor alive, so the allocator cannot hand the same address to a later table
    of the same shape with different content (pipelines build a fresh table every forward), and it records
    the tensor's version counter, so an in-place update of the table is noticed too."""
    key = (rotary_emb.data_ptr(), tuple(rotary_emb.shape), str(rotary_emb.device), rotary_emb.dtype)
    hit = _ROPE_CACHE.get(key)
    if hit is not None and hit[1] == rotary_emb._version:
        return hit[2], hit[3]
    if len(_ROPE_CACHE) >= 4:
        _ROPE_CACHE.clear()
    r = torch.view_as_real(rotary_emb.reshape(-1, rotary_emb.shape[-1]))
    cos, sin = r[..., 0].to(torch.float32).contiguous(), r[..., 1].to(torch.float32).contiguous()
    _ROPE_CACHE[key] = (rotary_emb, rotary_emb._version, cos, sin)
    return cos, sin


_SIDE_STREAMS: Dict[Tuple, torch.cuda.Stream] = {}


def _side_stream(device, k: int = 0) -> torch.cuda.Stream:
    """Stream `k` of the copy engines' transfers (a few per device, so that slabs for different destinations travel
    at the same time)."""
    st = _SIDE_STREAMS.get((str(device), k))
    if st is None:
        st = _SIDE_STREAMS[(str(device), k)] = torch.cuda.Stream(device=device)
    return st


_EXCHANGES: Dict[int, UlyssesExchange] = {}


def shared_exchange() -> UlyssesExchange:
    """The one exchange object of the sequence-parallel group, shared by every processor of the process."""
    ps = para_dist.parallel_state
    group = ps.get_sequence_parallel_group()
    x = _EXCHANGES.get(id(group))
    if x is None:
        x = _EXCHANGES[id(group)] = UlyssesExchange(group, ps.get_sequence_parallel_size(), ps.get_sequence_parallel_rank())
    return x


class DAXWanAttnProcessor2_0:
    def __init__(self, sp_size: int = 1, overlap_comm: bool = False, attention_mode: str = "bf16",
                 qkv_chunks: int = 4, o_micro_batches: int = 2, o_split: str = "auto",
                 sequence_parallel: Optional[bool] = None, exchange: str = "auto"):
        """``sp_size`` / ``overlap_comm`` as in the reference.  ``attention_mode``: "bf16" (bf16 contractions: the
        mode within rel-L2 1e-2 of fp32 SDPA, default), "sage" (INT8 Q.K^T, FP8 P.V: the reference backend's
        arithmetic) or "int8_bf16".  ``qkv_chunks``: token chunks of the Q/K/V
        projections whose exchange overlaps the next chunk's GEMMs; ``o_micro_batches``: micro-batches of the O
        path (2 in the reference); ``o_split``: how the O path is cut, "rows" (the reference's scheme),
        "ranks" (by groups of destination ranks) or "auto" (whichever needs fewer rounds of attention CTAs).
        ``sequence_parallel``: None follows the process-wide parallel state (the reference's behaviour); False
        keeps this processor local even when the state is initialised (an un-sharded layer run next to a sharded
        one, e.g. to check the sharded result).
        ``exchange``: how the two sequence<->head exchanges travel when ``overlap_comm`` is on.  "peer": the producing
        kernels store straight into the other GPUs' receive buffers over NVLink (peer-mapped symmetric memory) and a
        device-side barrier replaces the collective: the transfer is part of the kernels, nothing is chunked;
        "nccl": chunked point-to-point groups on NCCL's stream overlapping the next chunk's kernels; "auto": "peer"
        where peer-mapped buffers are available, else "nccl".  ``overlap_comm=False`` always takes one synchronous
        NCCL exchange per direction, as the reference does."""
        if exchange not in ("auto", "peer", "nccl"):
            raise ValueError("exchange must be 'auto', 'peer' or 'nccl'")
        self.exchange = exchange
        self.sequence_parallel = sequence_parallel
        if o_split not in ("auto", "rows", "ranks"):
            raise ValueError("o_split must be 'auto', 'rows' or 'ranks'")
        self.o_split = o_split
        if attention_mode not in ops.ATTN_MODES:
            raise ValueError(f"attention_mode must be one of {sorted(ops.ATTN_MODES)}")
        self.sp_size = sp_size
        self.overlap_comm = overlap_comm
        self.attention_mode = attention_mode
        self.qkv_chunks = qkv_chunks
        self.o_micro_batches = o_micro_batches
        self._xchg: Optional[UlyssesExchange] = None

    # ------------------------------------------------------------------------------------------
    def _exchange(self) -> Optional[UlyssesExchange]:
        if self.sequence_parallel is False or not para_dist.parallel_state.is_enable_sequence_parallel():
            return None
        if self._xchg is None:
            self._xchg = shared_exchange()
        return self._xchg

    def _direct(self, dtype=torch.bfloat16, S: int = 128, Sk: int = 128) -> bool:
        """The 16-bit mode reads bf16 Q, K, V in place (one kernel, no prepare step) when there is at least one tile of
        queries and keys; the INT8-score modes, fp16 tensors and tiny sequences prepare first."""
        return (ops.ATTN_MODES[self.attention_mode] == ops.ATTN_MODES["bf16"] and dtype == torch.bfloat16
                and S >= 128 and Sk >= 128)

    def _attend(self, q, k, v, out, **ranges) -> None:
        """Attention of ``[1, h, S, 128]`` views into ``out`` (optionally for query ranges only)."""
        if self._direct(q.dtype, q.shape[2], k.shape[2]):
            ops.attention_direct(q, k, v, out, sm_scale=1.0 / math.sqrt(HEAD_DIM), **ranges)
        else:
            plan = ops.attn_prepare(q, k, v, self.attention_mode, 1.0 / math.sqrt(HEAD_DIM))
            ops.attn_forward(plan, out, **ranges)

    @staticmethod
    def _project(lin: nn.Module, x_rows: torch.Tensor, q_pair, *, out: torch.Tensor, ldo: int, col_group: int,
                 group_stride: int, row_sumsq: Optional[torch.Tensor], resid: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None, group_ptrs=None) -> None:
        """``out <- lin(x_rows)`` in the (grouped) layout given by ldo / col_group / group_stride; with
        ``resid`` the gated residual ``out <- resid + gate * lin(x_rows)`` (fused into the GEMM epilogue); with
        ``group_ptrs`` (quantised linears only) the column groups go to those addresses instead of ``out``."""
        if isinstance(lin, QLinear):
            lin._check_supported()
            qx, sx = q_pair
            if group_ptrs is not None:
                lin.forward_quantized(qx, sx, ldo=ldo, out_col_group=col_group, group_ptrs=group_ptrs)
                return
            lin.forward_quantized(qx, sx, out=out, ldo=ldo, out_col_group=col_group,
                                  out_group_stride=group_stride, row_sumsq=row_sumsq, resid=resid, gate=gate)
        else:  # float projection: library GEMM, then a strided copy into the layout
            y = F.linear(x_rows, lin.weight, lin.bias)
            if resid is not None:
                y = (resid.float() + (y.float() * gate if gate is not None else y.float())).to(y.dtype)
            rows, N = y.shape
            dst = torch.as_strided(out, (N // col_group, rows, col_group), (group_stride, ldo, 1))
            dst.copy_(y.view(rows, N // col_group, col_group).transpose(0, 1))

    @staticmethod
    def _quantize_for(lins, x_rows: torch.Tensor):
        """One quantisation shared by all quantised projections of ``x_rows`` with the same input dtype."""
        cache = {}
        pairs = []
        for lin in lins:
            if isinstance(lin, QLinear):
                if lin.input_dtype not in cache:
                    cache[lin.input_dtype] = lin.quantize_input(x_rows)
                pairs.append(cache[lin.input_dtype])
            else:
                pairs.append(None)
        return pairs

    # ------------------------------------------------------------------------------------------
    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None,
                 attention_mask: Optional[torch.Tensor] = None, rotary_emb: Optional[torch.Tensor] = None) -> torch.Tensor:
        if getattr(attn, "add_k_proj", None) is not None:
            raise NotImplementedError("Wan I2V SP pararrel is not supported yet")
        if attention_mask is not None:
            raise NotImplementedError("The quantised attention kernel does not support `attention_mask`")
        if not hidden_states.is_cuda:
            raise RuntimeError("DAXWanAttnProcessor2_0 runs on CUDA tensors only; there is no CPU fallback")
        if hidden_states.dtype not in (torch.bfloat16, torch.float16):
            raise NotImplementedError(f"hidden_states must be bf16 or fp16, got {hidden_states.dtype}")
        outs = []
        for b in range(hidden_states.shape[0]):
            ctx = None if encoder_hidden_states is None else encoder_hidden_states[b]
            if ctx is None:
                outs.append(self._self_attention(attn, hidden_states[b].contiguous(), rotary_emb))
            else:
                outs.append(self._cross_attention(attn, hidden_states[b].contiguous(), ctx.contiguous()))
        out = outs[0].unsqueeze(0) if len(outs) == 1 else torch.stack(outs, 0)
        return attn.to_out[1](out)  # dropout (identity at inference), as in the reference

    # ------------------------------------------------------------------------------------------
    def _self_attention(self, attn, x: torch.Tensor, rotary_emb: Optional[torch.Tensor], prequant=None,
                        resid: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x [s, D]`` -> ``[s, D]``.  ``prequant = (codes, scales)`` of ``x`` when the caller has already
        quantised it (the fused block does, inside its LayerNorm kernel); ``resid`` / ``gate``: the O projection
        writes ``resid + gate * o`` instead of ``o``."""
        s, D = x.shape
        H = attn.heads
        dev, dt = x.device, x.dtype
        xchg = self._exchange()
        P = xchg.P if xchg is not None else 1
        rank = xchg.rank if xchg is not None else 0
        assert H % P == 0, f"Number of heads ({H}) must be divisible by the sequence parallel size ({P})!"
        assert D == H * HEAD_DIM, f"hidden size {D} != heads {H} x {HEAD_DIM}"
        h = H // P
        hd = h * HEAD_DIM
        S = s * P
        overlap = self.overlap_comm and P > 1

        cos = sin = None
        if rotary_emb is not None:
            cos, sin = _rope_tables(rotary_emb)
            assert cos.shape[0] >= S, f"rotary table has {cos.shape[0]} rows, sequence has {S}"

        if overlap and self.exchange != "nccl":
            peers = shared_peer_buffers(xchg.group, P, rank)
            if peers is not None:
                return self._self_attention_peer(attn, x, cos, sin, prequant, resid, gate, peers)
            if self.exchange == "peer":
                raise RuntimeError("exchange='peer' needs torch.distributed._symmetric_memory on CUDA devices")

        # exchange layout [P, s, h*d]: slab p = heads of rank p; with P == 1 this is plain [s, D]
        send = [_BUFFERS.get(f"send{i}", (P, s, hd), dt, dev) for i in range(3)]
        recv = send if P == 1 else [_BUFFERS.get(f"recv{i}", (S, hd), dt, dev) for i in range(3)]
        n_tiles = 2 * ((D + 255) // 256)  # sum-of-squares partials: one per 128 columns

        bounds = chunk_bounds(s, self.qkv_chunks if overlap else 1)
        max_rows = max(bounds[i + 1] - bounds[i] for i in range(len(bounds) - 1))
        works = []
        lins = (attn.to_q, attn.to_k, attn.to_v)
        norms = (attn.norm_q, attn.norm_k, None)
        for c in range(len(bounds) - 1):
            c0, c1 = bounds[c], bounds[c + 1]
            rows = c1 - c0
            x_rows = x[c0:c1]
            if prequant is not None:
                pairs = [(prequant[0][c0:c1], prequant[1][c0:c1]) if isinstance(lin, QLinear) else None for lin in lins]
            else:
                pairs = self._quantize_for(lins, x_rows)
            for i, (lin, norm) in enumerate(zip(lins, norms)):
                dst = send[i].view(P * s, hd)[c0:]  # row c0 of slab 0; slabs are s*hd apart
                if i == 2 or (norm is None and cos is None):
                    # no per-row post-processing: the GEMM writes the exchange layout itself
                    self._project(lin, x_rows, pairs[i], out=dst, ldo=hd, col_group=hd, group_stride=s * hd,
                                  row_sumsq=None)
                    continue
                tmp = _BUFFERS.get("proj_tmp", (max_rows, D), dt, dev)[:rows]
                fused = isinstance(lin, QLinear) and norm is not None
                ss = _BUFFERS.get("row_sumsq", (max_rows, n_tiles), torch.float32, dev)[:rows] if fused else None
                self._project(lin, x_rows, pairs[i], out=tmp, ldo=D, col_group=D, group_stride=0, row_sumsq=ss)
                w = getattr(norm, "weight", None) if norm is not None else None
                ops.rmsnorm_rope_pack(tmp, norm_weight=w, do_norm=norm is not None,
                                      eps=getattr(norm, "eps", 1e-6) if norm is not None else 1e-6,
                                      rope_cos=cos, rope_sin=sin, token_offset=rank * s + c0, row_sumsq=ss,
                                      out=dst, ldo=hd, col_group=hd, group_stride=s * hd)
            if P > 1:
                works.append(xchg.tokens_to_heads(send, recv, c0, c1, async_op=overlap))
        for w in works:
            w.wait()

        # attention over the full sequence of the local heads: [S, h, d] viewed as [1, h, S, d]
        def bhsd(t):
            return t.view(1, S, h, HEAD_DIM).transpose(1, 2)

        attn_out = _BUFFERS.get("attn_out", (S, hd), dt, dev)
        if self._direct(dt, S, S):
            def attend(**ranges):
                ops.attention_direct(bhsd(recv[0]), bhsd(recv[1]), bhsd(recv[2]), bhsd(attn_out),
                                     sm_scale=1.0 / math.sqrt(HEAD_DIM), **ranges)
        else:
            plan = ops.attn_prepare(bhsd(recv[0]), bhsd(recv[1]), bhsd(recv[2]), self.attention_mode,
                                    1.0 / math.sqrt(HEAD_DIM))

            def attend(**ranges):
                ops.attn_forward(plan, bhsd(attn_out), **ranges)
        o_lin = attn.to_out[0]
        out = torch.empty((s, D), dtype=dt, device=dev)

        if P == 1:
            attend()
            pair = self._quantize_for((o_lin,), attn_out)[0]
            self._project(o_lin, attn_out, pair, out=out, ldo=D, col_group=D, group_stride=0, row_sumsq=None,
                          resid=resid, gate=gate)
            return out

        # O path.  Two ways to cut it into micro-batches whose exchange overlaps the next one's attention:
        #  "rows":  micro-batch i = the i-th slice of EVERY destination rank's token block (the reference's
        #           scheme): the O projection of slice i-1 overlaps too;
        #  "ranks": micro-batch g = the whole blocks of a GROUP of destination ranks: one contiguous query
        #           range per launch, no partly filled tail tile per range.
        # The attention launches dominate, and every CTA (256 query rows x all keys) takes the same time, so
        # the split that needs fewer rounds of SM-count CTAs wins; ties go to the reference's scheme.
        m = self.o_micro_batches if overlap else 1
        mb = micro_batch_bounds(s, m)
        strategy = "rows"
        gb = micro_batch_bounds(P, min(m, P))
        if overlap and m > 1 and self.o_split == "ranks":
            strategy = "ranks"
        elif overlap and m > 1 and P >= 2 * m and self.o_split == "auto":
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            tiles = lambda n: (n + 255) // 256
            rounds_rows = sum(-(-(P * tiles(mb[i + 1] - mb[i]) * h) // sms) for i in range(m))
            rounds_ranks = sum(-(-(tiles((gb[g + 1] - gb[g]) * s) * h) // sms) for g in range(m))
            if rounds_ranks < rounds_rows:
                strategy = "ranks"
        if strategy == "ranks":
            o_recv = _BUFFERS.get("o_recv_full", (P, s, hd), dt, dev)
            mine, sends = None, []
            for g in range(len(gb) - 1):
                g0, g1 = gb[g], gb[g + 1]
                attend(q_begin=g0 * s, q_end=g1 * s)
                work = xchg.heads_to_tokens_group(attn_out, o_recv, s, range(g0, g1), async_op=True)
                if g0 <= rank < g1:
                    mine = work
                else:
                    sends.append(work)
            self._o_project(o_lin, (mine, o_recv, 0, s), out, P, hd, D, resid, gate)
            for w in sends:
                w.wait()  # sends of the other groups: attn_out is rewritten by the next layer
            return out

        pending = []
        for i in range(m):
            b0, b1 = mb[i], mb[i + 1]
            if b1 == b0:
                continue
            attend(q_begin=b0, q_end=b1, n_ranges=P, range_stride=s)
            o_recv = _BUFFERS.get(f"o_recv{i}", (P, b1 - b0, hd), dt, dev)
            work = xchg.heads_to_tokens(attn_out, o_recv, s, b0, b1, async_op=overlap)
            pending.append((work, o_recv, b0, b1))
            if len(pending) > 1:
                self._o_project(o_lin, pending.pop(0), out, P, hd, D, resid, gate)
        while pending:
            self._o_project(o_lin, pending.pop(0), out, P, hd, D, resid, gate)
        return out

    def _self_attention_peer(self, attn, x: torch.Tensor, cos, sin, prequant, resid, gate, peers: PeerBuffers) -> torch.Tensor:
        """The sequence-parallel block over peer-mapped receive buffers, no collective call: the Q / K / V slabs travel
        by copy engine while the next projection runs, the attention kernel stores every result row straight into the
        buffer of the rank that owns the token (free inside a compute-bound kernel), two device-side barriers order
        the ranks.  Un-chunked projections, one attention launch.  Same results as the NCCL paths (the kernels and
        their order per token are the same).  Three phases (produce, attend, project) separated by the barriers; they
        are methods of their own so that a test can drive several emulated ranks through them on one GPU."""
        c = self._peer_produce(attn, x, cos, sin, prequant, peers)
        self._peer_attend(c, peers)
        return self._peer_project(attn, c, peers, resid, gate)

    def _peer_produce(self, attn, x: torch.Tensor, cos, sin, prequant, peers: PeerBuffers):
        """Phase 1: project Q, K, V of this rank's tokens and send every head group to the rank that owns it."""
        s, D = x.shape
        H = attn.heads
        dev, dt = x.device, x.dtype
        P, rank = peers.P, peers.rank
        h = H // P
        hd = h * HEAD_DIM
        S = s * P
        esz = x.element_size()
        recv, recv_ptrs = peers.get("qkv_recv", (3, S, hd), dt, dev)      # [tensor, all tokens, my heads]
        o_recv, o_ptrs = peers.get("o_recv", (P, s, hd), dt, dev)         # slab p = rank p's heads for my tokens
        n_tiles = 2 * ((D + 255) // 256)
        lins = (attn.to_q, attn.to_k, attn.to_v)
        norms = (attn.norm_q, attn.norm_k, None)
        pairs = ([prequant if isinstance(lin, QLinear) else None for lin in lins] if prequant is not None
                 else self._quantize_for(lins, x))
        # Q, K, V: the producing kernel writes the slab of every OTHER rank into a local send buffer and this rank's own
        # slab straight into its receive buffer; the copy engines then carry each slab to its owner on a side stream
        # while the next projection runs on the SMs (a kernel that stored to the peers itself would be held to the
        # NVLink rate: these kernels are memory-bound or write short row segments).  V goes first, then K, then Q.
        main = torch.cuda.current_stream()
        sides = [_side_stream(dev, k) for k in range(min(P - 1, 4))]
        side = sides[0]
        send = [_BUFFERS.get(f"send{i}", (P, s, hd), dt, dev) for i in range(3)]
        kv_sent = None
        # row chunks of the last projection: about five full waves of GEMM tiles each (128 x 256 tiles, one CTA per SM)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        rows_target = 128 * max(1, round(5 * sms / ((D + 255) // 256)))
        q_chunks = max(1, round(s / rows_target))
        for i in (2, 1, 0):
            lin, norm = lins[i], norms[i]
            plain = norm is None and (i == 2 or cos is None)
            # the last tensor (Q) is projected in row chunks, so that only the last chunk's transfer is still in flight
            # when the attention could start
            bounds = chunk_bounds(s, q_chunks) if (i == 0 and self._direct(dt, S, S)) else [0, s]
            for c0, c1 in zip(bounds[:-1], bounds[1:]):
                own = recv[i, rank * s + c0:rank * s + c1]
                groups = [own.data_ptr() if p == rank else send[i][p, c0:c1].data_ptr() for p in range(P)]
                pair = None if pairs[i] is None else (pairs[i][0][c0:c1], pairs[i][1][c0:c1])
                if plain and isinstance(lin, QLinear):
                    self._project(lin, x[c0:c1], pair, out=None, ldo=hd, col_group=hd, group_stride=0, row_sumsq=None,
                                  group_ptrs=groups)
                else:
                    tmp = _BUFFERS.get("proj_tmp", (s, D), dt, dev)[c0:c1]
                    fused = isinstance(lin, QLinear) and norm is not None
                    ss = _BUFFERS.get("row_sumsq", (s, n_tiles), torch.float32, dev)[c0:c1] if fused else None
                    self._project(lin, x[c0:c1], pair, out=tmp, ldo=D, col_group=D, group_stride=0, row_sumsq=ss)
                    rope = i != 2 and cos is not None
                    ops.rmsnorm_rope_pack(tmp, norm_weight=getattr(norm, "weight", None) if norm is not None else None,
                                          do_norm=norm is not None, eps=getattr(norm, "eps", 1e-6) if norm is not None else 1e-6,
                                          rope_cos=cos if rope else None, rope_sin=sin if rope else None,
                                          token_offset=rank * s + c0, row_sumsq=ss, ldo=hd, col_group=hd, group_ptrs=groups)
                for st in sides:
                    st.wait_stream(main)
                for dp in range(1, P):
                    p = (rank + dp) % P  # every rank starts with a different destination
                    # rank p owns head group p: my rows of tensor i land at rows [rank * s, (rank + 1) * s) of ITS buffer
                    ops.peer_copy(recv_ptrs[p] + ((i * S + rank * s + c0) * hd) * esz, send[i][p, c0:c1],
                                  stream=sides[(dp - 1) % len(sides)])
            if i == 1:
                for st in sides[1:]:
                    side.wait_stream(st)
                kv_sent = side.record_event()

        return SimpleNamespace(s=s, D=D, P=P, rank=rank, h=h, hd=hd, S=S, esz=esz, dt=dt, dev=dev, recv=recv, o_recv=o_recv,
                               o_ptrs=o_ptrs, main=main, side=side, sides=sides, kv_sent=kv_sent)

    def _peer_attend(self, c, peers: PeerBuffers) -> None:
        """Phase 2: once every rank's rows have landed, attention over the full sequence of this rank's heads; every
        result row is stored into the buffer of the rank that owns the token."""
        s, P, rank, h, hd, S, esz, dt = c.s, c.P, c.rank, c.h, c.hd, c.S, c.esz, c.dt
        recv, o_ptrs, main, side, kv_sent = c.recv, c.o_ptrs, c.main, c.side, c.kv_sent

        def wait_all_sent():
            for st in c.sides:
                main.wait_stream(st)

        def bhsd(t):
            return t.view(1, S, h, HEAD_DIM).transpose(1, 2)

        # query row q belongs to rank q // s: its result goes to slab `rank` of that rank's o_recv
        o_dests = [o_ptrs[d] + (rank * s * hd) * esz for d in range(P)]
        if self._direct(dt, S, S):
            # the 16-bit kernel reads Q, K, V where they landed: nothing to prepare
            wait_all_sent()
            peers.barrier(0)  # every rank's Q, K and V rows are in my buffers
            ops.attention_direct(bhsd(recv[0]), bhsd(recv[1]), bhsd(recv[2]), sm_scale=1.0 / math.sqrt(HEAD_DIM),
                                 dest_ptrs=o_dests, rows_per_dest=s, head_stride=HEAD_DIM, token_stride=hd)
        else:
            # K and V have landed everywhere well before the last Q rows have: their statistics and operand passes run
            # under the tail of the Q transfer
            main.wait_event(kv_sent)
            peers.barrier(0)  # every rank's K and V rows are in my buffers
            args = (bhsd(recv[0]), bhsd(recv[1]), bhsd(recv[2]), self.attention_mode, 1.0 / math.sqrt(HEAD_DIM))
            ops.attn_prepare(*args, parts="kv")
            wait_all_sent()
            peers.barrier(2)  # ... and every rank's Q rows
            plan = ops.attn_prepare(*args, parts="q")
            ops.attn_forward_scatter(plan, o_dests, rows_per_dest=s, head_stride=HEAD_DIM, token_stride=hd)

    def _peer_project(self, attn, c, peers: PeerBuffers, resid, gate) -> torch.Tensor:
        """Phase 3: once every rank's attention rows for this rank's tokens have landed, the O projection."""
        s, D, P, hd, dt, dev, o_recv = c.s, c.D, c.P, c.hd, c.dt, c.dev, c.o_recv
        peers.barrier(1)  # every rank's attention rows for my tokens have landed
        out = torch.empty((s, D), dtype=dt, device=dev)
        self._o_project(attn.to_out[0], (_Done(), o_recv, 0, s), out, P, hd, D, resid, gate)
        return out

    def _o_project(self, o_lin, item, out: torch.Tensor, P: int, hd: int, D: int, resid=None, gate=None) -> None:
        work, o_recv, b0, b1 = item
        work.wait()
        n = b1 - b0
        res = resid[b0:b1] if resid is not None else None
        if isinstance(o_lin, QLinear):
            o_lin._check_supported()
            # the quantiser reads the receive slabs [P, n, h*d] in place as a [n, D] matrix
            qx, sx = ops.quant_rowwise(o_recv, o_lin.input_dtype, col_group=hd, group_stride=n * hd, rows=n, cols=D,
                                       ldx=hd)
            o_lin.forward_quantized(qx, sx, out=out[b0:b1], ldo=D, resid=res, gate=gate)
        else:
            xm = o_recv.permute(1, 0, 2).reshape(n, D)
            y = F.linear(xm, o_lin.weight, o_lin.bias)
            if res is not None:
                y = (res.float() + (y.float() * gate if gate is not None else y.float())).to(y.dtype)
            out[b0:b1] = y

    # ------------------------------------------------------------------------------------------
    def _cross_attention(self, attn, x: torch.Tensor, ctx: torch.Tensor, prequant=None,
                         resid: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Cross-attention (``attn2``): queries are this rank's tokens, keys/values the replicated text
        context.  Every query row attends to the whole context locally, so nothing is exchanged; the
        reference exchanges Q/K/V/O here too and attends over P identical copies of the context,
        which gives the same softmax (``attn_adapter.py:96-101,125-141``)."""
        s, D = x.shape
        H = attn.heads
        dev, dt = x.device, x.dtype
        Sk = ctx.shape[0]
        q = _BUFFERS.get("xq", (s, D), dt, dev)
        k = _BUFFERS.get("xk", (Sk, D), dt, dev)
        v = _BUFFERS.get("xv", (Sk, D), dt, dev)
        n_tiles = 2 * ((D + 255) // 256)  # sum-of-squares partials: one per 128 columns
        for lin, norm, src, dst in ((attn.to_q, attn.norm_q, x, q), (attn.to_k, attn.norm_k, ctx, k),
                                    (attn.to_v, None, ctx, v)):
            pair = prequant if (prequant is not None and src is x and isinstance(lin, QLinear)) else \
                self._quantize_for((lin,), src)[0]
            if norm is None:
                self._project(lin, src, pair, out=dst, ldo=D, col_group=D, group_stride=0, row_sumsq=None)
                continue
            rows = src.shape[0]
            tmp = _BUFFERS.get("xproj_tmp", (rows, D), dt, dev)
            fused = isinstance(lin, QLinear)
            ss = _BUFFERS.get("xrow_sumsq", (rows, n_tiles), torch.float32, dev) if fused else None
            self._project(lin, src, pair, out=tmp, ldo=D, col_group=D, group_stride=0, row_sumsq=ss)
            ops.rmsnorm_rope_pack(tmp, norm_weight=getattr(norm, "weight", None), do_norm=True,
                                  eps=getattr(norm, "eps", 1e-6), row_sumsq=ss, out=dst, ldo=D)

        def bhsd(t, n):
            return t.view(1, n, H, HEAD_DIM).transpose(1, 2)

        o = _BUFFERS.get("xo", (s, D), dt, dev)
        self._attend(bhsd(q, s), bhsd(k, Sk), bhsd(v, Sk), bhsd(o, s))
        o_lin = attn.to_out[0]
        out = torch.empty((s, D), dtype=dt, device=dev)
        pair = self._quantize_for((o_lin,), o)[0]
        self._project(o_lin, o, pair, out=out, ldo=D, col_group=D, group_stride=0, row_sumsq=None, resid=resid)
        return out


def _attention_classes():
    classes = []
    try:  # the real thing, when diffusers is installed
        from diffusers.models.attention_processor import Attention as DiffusersAttention
        classes.append(DiffusersAttention)
    except Exception:
        pass
    from .modules import Attention
    classes.append(Attention)
    return tuple(classes)


def replace_wan_attention(pipe, sp_size: int = 1, overlap_comm: bool = False, **processor_kwargs) -> None:
    """Install the processor on every attention module of ``pipe.transformer``
    (``dax/adapters/wan/attn_adapter.py:307-312``)."""
    classes = _attention_classes()
    for _, m in pipe.transformer.named_modules():
        if isinstance(m, classes):
            m.set_processor(DAXWanAttnProcessor2_0(sp_size=sp_size, overlap_comm=overlap_comm, **processor_kwargs))
