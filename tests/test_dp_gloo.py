"""CPU, world_size 2 over gloo: the data-parallel exchange (flat-bucket mean all-reduce of weight gradients) and the batch
sharding helper.  The GPU path uses the same code over NCCL."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from jetfire_int8training_b200.dp import allreduce_mean_, shard_range
    g = torch.Generator().manual_seed(100 + rank)
    grads = [torch.randn(96, 64, generator=g).half(), torch.randn(33, generator=g), torch.randn(64, 32, generator=g).half(),
             torch.randn(7, 5, generator=g).t()]            # includes a non-contiguous tensor
    ref = [t.clone() for t in grads]
    allreduce_mean_(grads, bucket_bytes=8192)
    gathered = [[torch.zeros_like(r.contiguous()) for _ in range(world)] for r in ref]
    for r, out in zip(ref, gathered):
        dist.all_gather(out, r.contiguous())
    ok = True
    for got, parts in zip(grads, gathered):
        want = sum(p.float() for p in parts) / world
        ok &= torch.allclose(got.float(), want, rtol=2e-3, atol=1e-3)
    # the reducer object gives the same means (submit / wait contract)
    from jetfire_int8training_b200.dp import MeanReducer
    red = MeanReducer()
    g2 = [r.contiguous().clone() for r in ref]
    red.submit(g2[:2]); red.submit(g2[2:])
    done = red.wait()
    ok &= len(done) == len(g2) and not red.pending
    for got, parts in zip(g2, gathered):
        want = sum(p.float() for p in parts) / world
        ok &= torch.allclose(got.float(), want, rtol=2e-3, atol=1e-3)
    b, e = shard_range(10, rank, world)
    ok &= (e - b == 5) and (b == 5 * rank)
    q.put((rank, bool(ok)))
    dist.destroy_process_group()


def test_allreduce_mean_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]


def test_reducer_is_a_no_op_without_a_process_group():
    from jetfire_int8training_b200.dp import MeanReducer
    red = MeanReducer()
    x = torch.ones(4)
    red.submit([x])
    assert red.wait() == [] and torch.equal(x, torch.ones(4))


def test_shard_range_covers_everything():
    from jetfire_int8training_b200.dp import shard_range
    for total in (0, 1, 7, 8, 1000):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
