"""Token data parallelism on CPU ranks (gloo, world_size 2): the flat gradient arena is
averaged by one all-reduce or by buckets launched as the gradients become final, replicas
stay identical (also the bf16 compute copies of a model already bound to a training step),
and a rank that never joins makes the collective fail with an error instead of hanging."""
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
    # the same exchange in buckets, driven the way backward drives it: ranks become final in
    # ascending order; nothing may be sent before it is final, everything is averaged at the end
    arena.buffer.copy_(base * (rank + 1))
    sent = []
    arena.on_bucket = sent.append
    arena.begin_overlap(bucket_bytes=4 * 2000)
    for r, rb, re in arena.ready_bounds:
        arena.notify_ready(r)
        assert arena._ov_sent <= re
    arena.finish_overlap()
    ok_ov = torch.allclose(arena.buffer, want, rtol=1e-6, atol=1e-6) and len(sent) >= 2 \
        and sum(sent) == 4 * arena.buffer.numel()
    q.put((rank, ok_avg, ok_rep, (b, e), ok_ov))
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
    assert [r[4] for r in res] == [True, True]


def _bound_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder
    from weightshared_torchtitan_b200.dp import broadcast_parameters
    from weightshared_torchtitan_b200.train_step import TrainStep
    torch.manual_seed(200 + rank)
    m = WeightSharedDecoder(DecoderConfig(dim=32, hidden_dim=64, n_layers=2, n_unique=1, n_heads=2, n_kv_heads=1,
                                          head_dim=16, rank=8, vocab_size=64, embed_rank=16, max_seq_len=8))
    step = TrainStep(m)                       # binds the model's copy cache to the flat arena
    W = m.blocks[0].wq.weight
    stale = m._cache.get(torch.bfloat16, W).clone()     # creates the flat bf16 copy
    broadcast_parameters(m, src=0)            # rank 1 receives other values
    fresh = m._cache.get(torch.bfloat16, W)
    ok = torch.equal(fresh, W.detach().to(torch.bfloat16))
    changed = not torch.equal(fresh, stale)
    q.put((rank, ok, changed))
    dist.barrier()
    dist.destroy_process_group()


def test_broadcast_refreshes_copies_of_a_bound_model():
    """dp.broadcast_parameters after a TrainStep was built: the flat bf16 copy the kernels read
    follows the received values on every rank."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_bound_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [True, True]
    assert res[1][2] is True                  # rank 1's values really changed


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
