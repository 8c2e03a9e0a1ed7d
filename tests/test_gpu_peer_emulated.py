"""The peer-buffer exchange path of the sequence-parallel processor with P EMULATED ranks on one GPU.

Every "peer" buffer is a separate allocation of the same device (to a kernel, a peer mapping is just an unrelated
address), the device-side barrier is a synchronise, and the ranks are driven phase by phase (all produce, all attend,
all project).  This checks the addressing of the whole path — head-group slabs, copy-engine destinations, the two row
halves of Q, attention rows scattered to their owners, the O projection over the receive slabs — at 8 ranks with an
odd local length, against the same layer un-sharded.  The real multi-GPU run is tests/test_gpu_multi.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


class EmulatedPeers:
    def __init__(self, P):
        self.P, self.rank, self.store, self.local_only = P, 0, {}, False

    def get(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype)
        if key not in self.store:
            self.store[key] = [torch.zeros(tuple(shape), dtype=dtype, device=device) for _ in range(self.P)]
        bufs = self.store[key]
        return bufs[self.rank], [b.data_ptr() for b in bufs]

    def barrier(self, channel=0):
        torch.cuda.synchronize()


@pytest.mark.parametrize("P,s,mode,linear", [(8, 129, "bf16", "int8"), (8, 129, "sage", "fp8_e4m3"), (4, 300, "bf16", "fp8_e4m3"),
                                             (2, 1023, "int8_bf16", "int8")])
def test_peer_path_with_emulated_ranks(built_library, P, s, mode, linear):
    if not torch.cuda.is_available():
        pytest.fail("the gpu tests need a CUDA device")
    from dax_b200.adapters.wan.attn_adapter import DAXWanAttnProcessor2_0, _rope_tables
    from dax_b200.adapters.wan.modules import Attention, init_wan_weights_, wan_rope_table
    from dax_b200.adapters.wan.transformer_adapter import quantize_transformer
    from oracle import dax_oracle as O
    H, D, S = 8, 1024, P * s
    holder = torch.nn.Module()
    holder.attn = Attention(D, H)
    init_wan_weights_(holder, 0.02, 5)
    g = torch.Generator().manual_seed(6)
    with torch.no_grad():
        holder.attn.norm_q.weight.copy_(1 + 0.1 * torch.randn(D, generator=g))
        holder.attn.norm_k.weight.copy_(1 + 0.1 * torch.randn(D, generator=g))
        for lin in (holder.attn.to_q, holder.attn.to_k, holder.attn.to_v, holder.attn.to_out[0]):
            lin.bias.copy_(0.05 * torch.randn(D, generator=g))
    holder = holder.bfloat16().to(DEV)
    quantize_transformer(holder, linear)
    attn = holder.attn
    x = torch.randn(S, D, generator=g).bfloat16().to(DEV)
    rope = wan_rope_table((1, 1, S), device=DEV)
    with torch.no_grad():
        attn.set_processor(DAXWanAttnProcessor2_0(sequence_parallel=False, attention_mode=mode))
        ref = attn(x.unsqueeze(0), rotary_emb=rope)[0].float().cpu()
        proc = DAXWanAttnProcessor2_0(sp_size=P, overlap_comm=True, attention_mode=mode)
        cos, sin = _rope_tables(rope)
        peers = EmulatedPeers(P)
        ctx = []
        for r in range(P):
            peers.rank = r
            ctx.append(proc._peer_produce(attn, x[r * s:(r + 1) * s].contiguous(), cos, sin, None, peers))
            torch.cuda.synchronize()
        for r in range(P):
            peers.rank = r
            proc._peer_attend(ctx[r], peers)
            torch.cuda.synchronize()
        outs = []
        for r in range(P):
            peers.rank = r
            outs.append(proc._peer_project(attn, ctx[r], peers, None, None).float().cpu())
    got = torch.cat(outs, 0)
    from dax_b200 import _lib
    assert _lib.device_status() == 0
    # same kernels, same arithmetic per token: sharding must not change the numbers
    assert O.rel_l2(got, ref) <= 2e-3, O.rel_l2(got, ref)
