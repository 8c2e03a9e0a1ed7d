"""Sequence-parallel processor on 2 (and 4) GPUs against the single-GPU result with the same weights:
both `overlap_comm` settings and both O-path splits, an odd local token count (63: uneven chunks and
micro-batches), the 16-bit attention mode with INT8 linears and the INT8/FP8 mode with FP8 linears.  Skipped on a
one-GPU box.  Ranks are child processes over NCCL with NVLS off; no rank leaves with work in flight."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _build(D, H, seed):
    from dax_b200.adapters.wan.modules import Attention, init_wan_weights_
    attn = Attention(D, H)
    init_wan_weights_(attn, 0.02, seed)
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        attn.norm_q.weight.copy_(1 + 0.1 * torch.randn(D, generator=g))
        attn.norm_k.weight.copy_(1 + 0.1 * torch.randn(D, generator=g))
        for lin in (attn.to_q, attn.to_k, attn.to_v, attn.to_out[0]):
            lin.bias.copy_(0.05 * torch.randn(D, generator=g))
    return attn.bfloat16()


def _inputs(S, D, grid, seed=5):
    from dax_b200.adapters.wan.modules import wan_rope_table
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, S, D, generator=g).bfloat16(), wan_rope_table(grid)


def _worker(rank, world, port, S, D, H, grid, q, mode, linear):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    try:
        from dax_b200 import _lib
        from dax_b200.adapters.wan import optimize_pipe
        from dax_b200.adapters.wan.modules import _Pipe
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        x, rope = _inputs(S, D, grid)
        s = S // world
        outs = {}
        # no overlap (one synchronous NCCL exchange per direction); overlap with the producing kernels storing into the
        # peers' buffers; overlap over chunked NCCL groups with the O path cut by rows and by destination ranks
        for overlap in (False, "peer", "nccl_rows", "nccl_ranks"):
            holder = torch.nn.Module()
            holder.blocks = torch.nn.ModuleList([_build(D, H, 3)])
            pipe = _Pipe(holder.to(dev))
            optimize_pipe(pipe, sequence_parallel=True, compile=False, overlap_comm=bool(overlap),
                          int8_linear=linear == "int8", fp8_linear=linear == "fp8", attention_mode=mode)
            proc = holder.blocks[0].processor
            if overlap == "peer":
                proc.exchange = "peer"
            elif overlap:
                proc.exchange, proc.o_split = "nccl", overlap.split("_")[1]
            y = holder.blocks[0](x[:, rank * s:(rank + 1) * s].to(dev), rotary_emb=rope.to(dev))
            torch.cuda.synchronize()
            outs[overlap] = y.float().cpu()
        assert _lib.device_status() == 0
        dist.barrier()
        q.put((rank, outs, None))
    except Exception:
        import traceback
        q.put((rank, None, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


@pytest.mark.parametrize("mode,linear", [("f16", "int8"), ("sage", "fp8")])
@pytest.mark.parametrize("world", [2, 4])
def test_sequence_parallel_matches_single_gpu(built_library, world, mode, linear):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from dax_b200.adapters.wan import optimize_pipe
    from dax_b200.adapters.wan.modules import _Pipe
    from oracle import dax_oracle as O
    D, H = 1024, 8
    grid = (1, 7, world * 9)      # S = 63 * world tokens: odd local length 63
    S = grid[0] * grid[1] * grid[2]
    x, rope = _inputs(S, D, grid)
    holder = torch.nn.Module()
    holder.blocks = torch.nn.ModuleList([_build(D, H, 3)])
    pipe = _Pipe(holder.to("cuda:0"))
    optimize_pipe(pipe, sequence_parallel=False, compile=False, overlap_comm=False, int8_linear=linear == "int8",
                  fp8_linear=linear == "fp8", attention_mode=mode)
    ref = holder.blocks[0](x.to("cuda:0"), rotary_emb=rope.to("cuda:0")).float().cpu()

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, S, D, H, grid, q, mode, linear)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    errs = [e for _, _, e in results if e]
    assert not errs, "\n".join(errs)
    s = S // world
    for rank, outs, _ in results:
        for overlap, y in outs.items():
            want = ref[:, rank * s:(rank + 1) * s]
            # same kernels, same order of operations per token: sharding must not change the numbers
            assert O.rel_l2(y, want) <= 2e-3, (rank, overlap, O.rel_l2(y, want))
