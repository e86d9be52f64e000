"""Token data parallelism on real GPUs (needs two; skipped on a single-GPU box): N ranks on their
shards + the gradient exchange give the gradients of one rank on the whole batch, with the
exchange as one all-reduce and as buckets overlapped with backward, and the replicas hold
bit-identical weights after several optimizer steps. Ranks are child processes, one GPU each,
NCCL with NVLS off; no rank leaves while a collective is in flight."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from weightshared_torchtitan_b200 import functional as Fn
    from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder
    from weightshared_torchtitan_b200.dp import broadcast_parameters
    from weightshared_torchtitan_b200.train_step import TrainStep
    c = DecoderConfig(dim=256, hidden_dim=512, n_layers=4, n_unique=2, n_heads=4, n_kv_heads=2, head_dim=64, rank=16,
                      vocab_size=1024, embed_rank=64, max_seq_len=128, loss_chunk=128)
    m = WeightSharedDecoder(c).cuda()
    m.init_weights(seed=7 + rank)                 # replicas start different on purpose
    broadcast_parameters(m, src=0)
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, c.vocab_size, (2 * world, 128), generator=g).cuda()
    labels = torch.randint(0, c.vocab_size, (2 * world, 128), generator=g).cuda()
    out = {}
    Fn.DERIVED_ADAPTER_GRADS = False              # per-token roundings only: shards and whole batch agree to fp32 order
    step = TrainStep(m, lr=1e-3, overlap=True, bucket_bytes=1 << 20, status_every=0)
    for mode, overlap in (("blocking", False), ("overlap", True)):
        step.overlap = overlap
        loss_full = step.gradients(tokens, labels, exchange=False)
        full = step.arena.buffer.clone()
        mine = slice(2 * rank, 2 * rank + 2)
        loss_shard = step.gradients(tokens[mine], labels[mine], exchange=True)
        dist.all_reduce(loss_shard, op=dist.ReduceOp.AVG)
        err = float((step.arena.buffer - full).abs().max() / full.abs().max())
        out[mode] = (err, abs(float(loss_full) - float(loss_shard)))
    for i in range(3):
        mine = slice(2 * rank, 2 * rank + 2)
        step(tokens[mine], labels[mine])
    chk = torch.stack([step.arena.master.double().sum(), step.arena.master.double().abs().sum()])
    allc = [torch.zeros_like(chk) for _ in range(world)]
    dist.all_gather(allc, chk)
    out["identical"] = all(torch.equal(allc[0], t) for t in allc)
    torch.cuda.synchronize()
    dist.barrier()
    q.put((rank, out))
    dist.destroy_process_group()


def test_shards_plus_exchange_equal_the_whole_batch_on_two_gpus():
    if not torch.cuda.is_available():
        pytest.fail("gpu tests need a CUDA device")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank in range(world):
        for mode in ("blocking", "overlap"):
            err, dloss = res[rank][mode]
            assert err < 1e-4, (rank, mode, err)       # same arithmetic per token; only fp32 summation order differs
            assert dloss < 1e-5, (rank, mode, dloss)
        assert res[rank]["identical"]
