"""The sequence-parallel host logic over gloo ranks on the CPU (world sizes 2 and 4)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dax_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world))
    try:
        from dax_b200.parallel.initialize import initialize
        sp = initialize(backend="gloo")
        assert sp == world
        globals()[fn_name](rank, world)
        dist.barrier()
        q.put((rank, None))
    except Exception as e:  # surfaced by the parent
        import traceback
        q.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run(fn_name, world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    errs = [e for _, e in results if e]
    assert not errs, "\n".join(errs)


def _shards(world, s, H, d=8, B=1):
    g = torch.Generator().manual_seed(7)
    return [torch.randn(B, s, H, d, generator=g) for _ in range(world)]


def case_state(rank, world):
    from dax_b200.parallel.dist import parallel_state as ps
    assert ps.is_enable_sequence_parallel() == (world > 1)
    assert ps.get_sequence_parallel_size() == world and ps.get_sequence_parallel_rank() == rank
    assert ps.get_data_parallel_size() == 1 and ps.get_sequence_parallel_all_ranks() == list(range(world))


def case_sync_exchange(rank, world):
    from dax_b200.parallel.patches import wanx2_1_t2v as sync
    for B in (1, 2):
        shards = _shards(world, 6, 8, B=B)
        tok = sync.collect_tokens(shards[rank])
        assert torch.equal(tok, O.collect_tokens_ref(shards, rank))
        full = [O.collect_tokens_ref(shards, r) for r in range(world)]
        back = sync.collect_heads(tok)
        assert torch.equal(back, O.collect_heads_ref(full, rank)) and torch.equal(back, shards[rank])
    x = torch.arange(4 * world * 3, dtype=torch.float32).reshape(1, 4 * world, 3)
    mine = sync.split(x, 1)
    assert torch.equal(mine, x[:, rank * 4:(rank + 1) * 4])
    assert torch.equal(sync.gather(mine, 1), x)
    with pytest.raises(AssertionError):
        sync.split(torch.zeros(1, 4 * world + 1, 3), 1)


def case_async_exchange(rank, world):
    from dax_b200.parallel.patches import wanx2_1_t2v_opt as opt
    shards = _shards(world, 6, 8)
    handle = {}
    opt.collect_tokens(shards[rank], world, async_op=True, handle=handle)
    handle["work"].wait()
    tok = handle["post_all2all_func"](handle["output"])
    assert torch.equal(tok, O.collect_tokens_ref(shards, rank))
    assert torch.equal(opt.collect_tokens(shards[rank], world), tok)
    # packed q, k, v in one collective
    q, k, v = opt.collect_tokens_packed_qkv(shards[rank], shards[rank] * 2, shards[rank] + 1, world)
    assert torch.equal(q, tok) and torch.equal(k, tok * 2) and torch.equal(v, tok + 1)
    # the O path: micro-batches, exchanged one by one, concatenate to this rank's block in order
    full = [O.collect_tokens_ref(shards, r) for r in range(world)]
    parts = []
    for mb in opt.micro_batch_project_O_strategy(full[rank], 2, world):
        h = {}
        opt.collect_heads(mb, world, async_op=True, handle=h)
        h["work"].wait()
        parts.append(h["post_all2all_func"](h["output"]))
    assert torch.equal(torch.cat(parts, dim=1), shards[rank])
    assert torch.equal(opt.split(torch.arange(2 * world).view(1, -1), world, 1),
                       torch.arange(2 * world).view(1, -1)[:, rank * 2:(rank + 1) * 2])
    with pytest.raises(AssertionError):
        opt.collect_tokens(torch.zeros(1, 4, world + 1, 8), world)


def case_zero_copy_chunks(rank, world):
    """The processor's exchange plan: chunked tokens->heads into [S, hd] and micro-batched
    heads->tokens into slabs, including an odd local length (uneven chunks and micro-batches)."""
    from dax_b200.parallel.dist import parallel_state as ps
    from dax_b200.parallel.patches.wanx2_1_t2v_opt import micro_batch_bounds
    from dax_b200.parallel.ulysses import UlyssesExchange, chunk_bounds
    xc = UlyssesExchange(ps.get_sequence_parallel_group(), world, rank)
    for s, align in ((7, 2), (12, 4)):
        H, d = 2 * world, 4
        h, hd = H // world, (H // world) * d
        shards = _shards(world, s, H, d)
        # what the projection kernels write: send[p] = heads of rank p for my tokens
        send = shards[rank][0].reshape(s, world, hd).transpose(0, 1).contiguous()
        recv = torch.zeros(world * s, hd)
        works = []
        b = chunk_bounds(s, 3, align)
        assert b[0] == 0 and b[-1] == s and all(x < y for x, y in zip(b, b[1:]))
        for c0, c1 in zip(b, b[1:]):
            works.append(xc.tokens_to_heads([send], [recv], c0, c1, async_op=True))
        for w in works:
            w.wait()
        want = O.collect_tokens_ref(shards, rank)[0].reshape(world * s, hd)
        assert torch.equal(recv, want)
        # heads -> tokens, micro-batched
        mb = micro_batch_bounds(s, 2)
        assert mb == [0, (s + 1) // 2, s]
        full = [O.collect_tokens_ref(shards, r) for r in range(world)]
        out = torch.zeros(s, world, hd)
        for b0, b1 in zip(mb, mb[1:]):
            slab = torch.zeros(world, b1 - b0, hd)
            xc.heads_to_tokens(recv, slab, s, b0, b1, async_op=False)
            out[b0:b1] = slab.transpose(0, 1)
        assert torch.equal(out.reshape(1, s, H, d), O.collect_heads_ref(full, rank))
        # heads -> tokens by groups of destination ranks
        slab = torch.zeros(world, s, hd)
        gb = micro_batch_bounds(world, 2)
        works = [xc.heads_to_tokens_group(recv, slab, s, range(g0, g1), async_op=True) for g0, g1 in zip(gb, gb[1:])]
        for w in works:
            w.wait()
        assert torch.equal(slab.transpose(0, 1).reshape(1, s, H, d), O.collect_heads_ref(full, rank))


def case_peer_probe_agrees(rank, world):
    """The peer-buffer probe is collective: where one rank cannot have peer-mapped buffers, no rank takes the peer
    path.  On CPU no rank can (the answer must still be the same everywhere); then rank 1 alone is made to 'succeed'
    and the minimum over the ranks still says no."""
    from dax_b200.parallel import peer
    from dax_b200.parallel.dist import parallel_state as ps
    group = ps.get_sequence_parallel_group()
    assert peer.shared_peer_buffers(group, world, rank) is None
    assert peer.shared_peer_buffers(group, world, rank) is None  # cached, no second collective
    peer._PEERS.clear()

    class FakeBuffers:
        def __init__(self, group, size, rank):
            self.P, self.rank = size, rank

        @staticmethod
        def supported():
            return rank == 1

        def get(self, *a, **k):
            return None

    real = peer.PeerBuffers
    peer.PeerBuffers = FakeBuffers
    try:
        assert peer.shared_peer_buffers(group, world, rank) is None
    finally:
        peer.PeerBuffers = real
        peer._PEERS.clear()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", ["case_state", "case_sync_exchange", "case_async_exchange", "case_zero_copy_chunks",
                                  "case_peer_probe_agrees"])
def test_gloo(case, world):
    run(case, world)


def test_initialize_requires_launcher(monkeypatch):
    from dax_b200.parallel.initialize import initialize
    for k in ("TORCHELASTIC_RUN_ID", "RANK", "WORLD_SIZE"):
        monkeypatch.delenv(k, raising=False)
    with pytest.raises(ValueError, match="torchrun"):
        initialize()


def test_parallel_config_validation():
    from dax_b200.parallel.config import ParallelConfig
    assert ParallelConfig().sp_degree == 1 and ParallelConfig().dp_degree == -1


def test_uneven_micro_batches_cover_everything():
    from dax_b200.parallel.patches.wanx2_1_t2v_opt import micro_batch_bounds, micro_batch_project_O_strategy
    # 480p at 8 ranks: 4095 local tokens, two micro-batches of 2048 and 2047
    assert micro_batch_bounds(4095, 2) == [0, 2048, 4095]
    t = torch.arange(3 * 7).view(1, 21, 1, 1)
    mbs = micro_batch_project_O_strategy(t, 2, 3)
    assert [m.shape[1] for m in mbs] == [12, 9]
    assert sorted(torch.cat(mbs, 1).flatten().tolist()) == list(range(21))
