"""Token data parallelism on CPU ranks (gloo, world_size 2): the flat gradient arena is
averaged by one all-reduce, replicas stay identical, and a rank that never joins makes the
collective fail with an error instead of hanging."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder
    from weightshared_torchtitan_b200.dp import GradArena, broadcast_parameters, shard_tokens
    torch.manual_seed(100 + rank)            # replicas start different on purpose
    m = WeightSharedDecoder(DecoderConfig(dim=32, hidden_dim=64, n_layers=4, n_unique=2, n_heads=2, n_kv_heads=1,
                                          head_dim=16, rank=8, vocab_size=64, embed_rank=16, max_seq_len=8))
    broadcast_parameters(m, src=0)
    arena = GradArena(m)
    # stand-in for backward: each rank writes rank-dependent gradients into its arena
    g = torch.Generator().manual_seed(7)
    base = torch.randn(arena.buffer.numel(), generator=g)
    arena.buffer.copy_(base * (rank + 1))
    arena.all_reduce_mean()
    want = base * (sum(range(1, world + 1)) / world)
    ok_avg = torch.allclose(arena.buffer, want, rtol=1e-6, atol=1e-6)
    psum = torch.stack([p.detach().double().sum() for p in m.parameters()]).sum()
    allp = [torch.zeros_like(psum) for _ in range(world)]
    dist.all_gather(allp, psum)
    ok_rep = all(torch.equal(allp[0], t) for t in allp)
    b, e = shard_tokens(8, rank, world)
    q.put((rank, ok_avg, ok_rep, (b, e)))
    dist.barrier()
    dist.destroy_process_group()


def test_arena_all_reduce_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [True, True]
    assert [r[2] for r in res] == [True, True]
    assert [r[3] for r in res] == [(0, 4), (4, 8)]


def _lonely(rank, world, port, q):
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
        q.put("joined")
    except Exception as e:  # noqa: BLE001 - any rendezvous failure is the expected outcome
        q.put("error:" + type(e).__name__)


def test_missing_rank_is_an_error_not_a_hang():
    """Failure made on the host: rank 1 never starts; rank 0's rendezvous ends with an error
    within its timeout."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely, args=(0, 2, _free_port(), q))
    p.start()
    out = q.get(timeout=60)
    p.join(timeout=30)
    assert out.startswith("error:")
