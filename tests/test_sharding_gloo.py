"""Token sharding across ranks, exercised with world_size-2 gloo processes on CPU: shards tile the
batch, the sharded forward equals the unsharded one row for row, and summed weight gradients equal
the full-batch gradients. The per-rank compute is the CPU oracle (the sharding logic is what is
under test here; the CUDA path is covered by the -m gpu tests)."""
import os
import socket
import sys
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _block(seed=0):
    from oracle import moe_oracle as O
    torch.manual_seed(seed)
    m = O.OracleBlock(64, 8, 192, 2, n_shared=1, std=0.2)
    m.train(False)
    return m


def _worker(rank, world, port, tokens, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nanospeaker_b200 import parallel
        torch.manual_seed(123)
        x = torch.randn(tokens, 64)
        m = _block()
        lo, hi = parallel.shard_bounds(tokens, world, rank)
        xs = parallel.shard_tokens(x, world, rank).clone().requires_grad_(True)
        out = m(xs)
        # loss normalised by the GLOBAL element count so shard gradients sum to the full gradient
        (out.square().sum() / (tokens * 64)).backward()
        parallel.all_reduce_gradients(m.parameters())
        counts = parallel.all_reduce_counts(m.expert_counts)
        # gloo's all_gather wants equal shapes: pad every shard to the largest one
        sizes = [parallel.shard_bounds(tokens, world, r) for r in range(world)]
        longest = max(b - a for a, b in sizes)
        padded = torch.zeros(longest, 64)
        padded[: hi - lo] = out.detach()
        gathered = [torch.empty(longest, 64) for _ in range(world)]
        dist.all_gather(gathered, padded)
        if rank == 0:
            full = torch.cat([g[: b - a] for g, (a, b) in zip(gathered, sizes)])
            # numpy arrays travel by value; torch tensors would be shared through file
            # descriptors that die with this process
            q.put((full.numpy(), m.W_in.grad.numpy(), m.router_W.grad.numpy(), counts.numpy(),
                   (lo, hi)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [64, 37])
def test_token_sharded_block_matches_unsharded(tokens):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tokens, q)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.time() + 120
    while q.empty():                      # never block forever on a worker that died
        assert time.time() < deadline, "gloo workers timed out"
        assert all(p.is_alive() or p.exitcode == 0 for p in procs), "a gloo worker failed"
        time.sleep(0.05)
    out, dw_in, d_router, counts = [torch.from_numpy(a) for a in q.get()[:4]]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0

    torch.manual_seed(123)
    x = torch.randn(tokens, 64).requires_grad_(True)
    m = _block()
    ref = m(x)
    (ref.square().sum() / (tokens * 64)).backward()
    assert torch.allclose(out, ref.detach(), atol=1e-6)
    assert torch.allclose(dw_in, m.W_in.grad, atol=1e-6)
    assert torch.allclose(d_router, m.router_W.grad, atol=1e-6)
    assert torch.equal(counts, m.expert_counts)


def test_shard_bounds_tile_the_batch():
    from nanospeaker_b200.parallel import shard_bounds
    for n in [0, 1, 7, 64, 131072, 131073]:
        for world in [1, 2, 3, 4, 8]:
            edges = [shard_bounds(n, world, r) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
            sizes = [hi - lo for lo, hi in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)
