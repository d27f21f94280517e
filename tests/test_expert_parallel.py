"""Host logic of the expert-parallel block on CPU: the partition, the exchange drivers (in-process
loopback and torch.distributed over gloo with two ranks) and the backward through the exchanges,
against a single-rank computation of the same block. The per-rank expert compute is injected (plain
torch here; the CUDA kernels are exercised by the GPU test of the same path)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from nanospeaker_b200 import expert_parallel as EP

D, H, E, K, S = 32, 16, 10, 3, 2


def torch_experts(rows, local_idx, w_in, w_out, activation):
    """Dropless FFN of `rows` through experts `local_idx` (plain torch, differentiable)."""
    out = rows.new_zeros((rows.shape[0], w_out.shape[2])) + (w_in.sum() + w_out.sum()) * 0
    for e in range(w_in.shape[0]):
        sel = (local_idx == e).nonzero().squeeze(1)
        if sel.numel():
            g, u = (rows[sel] @ w_in[e]).chunk(2, -1)
            out = out.index_add(0, sel, (torch.nn.functional.silu(g) * u) @ w_out[e])
    return out


def torch_shared(x, w_sh_in, w_sh_out, activation):
    out = 0
    for s in range(w_sh_in.shape[0]):
        g, u = (x @ w_sh_in[s]).chunk(2, -1)
        out = out + (torch.nn.functional.silu(g) * u) @ w_sh_out[s]
    return out


def make_problem(tokens, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x = r(tokens, D)
    logits = r(tokens, E)
    w, idx = torch.softmax(logits, -1).topk(K, -1)
    w = w / w.sum(-1, keepdim=True)
    return dict(x=x, w=w, idx=idx, W_in=r(E, D, 2 * H) * D ** -0.5, W_out=r(E, H, D) * H ** -0.5,
                W_sh_in=r(S, D, 2 * H) * D ** -0.5, W_sh_out=r(S, H, D) * H ** -0.5)


def single_rank(p, x, w, idx):
    """The same block on one rank: every pair through its expert, weighted sum, shared experts."""
    t = x.shape[0]
    rows = x[torch.arange(t * K) // K]
    y = torch_experts(rows, idx.reshape(-1), p["W_in"], p["W_out"], "silu").view(t, K, D)
    return (y * w.unsqueeze(-1)).sum(1) + torch_shared(x, p["W_sh_in"], p["W_sh_out"], "silu")


def test_partition_and_owner():
    assert [hi - lo for lo, hi in EP.expert_partition(76, 8)] == [10, 10, 10, 10, 9, 9, 9, 9]
    b = EP.expert_partition(10, 4)
    assert b == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert EP.owner_of(torch.arange(10), b).tolist() == [0, 0, 0, 1, 1, 1, 2, 2, 3, 3]
    with pytest.raises(ValueError):
        EP.expert_partition(3, 4)


@pytest.mark.parametrize("world,tokens", [(1, 40), (4, 64), (5, 3)])
def test_loopback_matches_single_rank_forward_and_backward(world, tokens):
    p = make_problem(tokens * world, seed=world)
    leaves = {k: p[k].clone().requires_grad_(True) for k in ("x", "w", "W_in", "W_out", "W_sh_in",
                                                            "W_sh_out")}
    ref_leaves = {k: p[k].clone().requires_grad_(True) for k in leaves}
    bounds = EP.expert_partition(E, world)
    gens = []
    for r in range(world):
        sl = slice(r * tokens, (r + 1) * tokens)
        lo, hi = bounds[r]
        gens.append(EP.ep_forward_steps(
            leaves["x"][sl], leaves["w"][sl], p["idx"][sl], leaves["W_in"][lo:hi],
            leaves["W_out"][lo:hi], leaves["W_sh_in"], leaves["W_sh_out"], r, bounds, "silu",
            expert_fn=torch_experts, shared_fn=torch_shared))
    out = torch.cat(EP.run_loopback(gens))
    ref = single_rank({**p, **{k: ref_leaves[k] for k in ("W_in", "W_out", "W_sh_in", "W_sh_out")}},
                      ref_leaves["x"], ref_leaves["w"], p["idx"])
    assert torch.allclose(out, ref, atol=1e-10)
    gout = torch.randn_like(out)
    out.backward(gout)
    ref.backward(gout)
    for k in leaves:
        assert torch.allclose(leaves[k].grad, ref_leaves[k].grad, atol=1e-9), k


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank, world, port, tokens, q):
    try:
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        p = make_problem(tokens * world, seed=7)
        bounds = EP.expert_partition(E, world)
        lo, hi = bounds[rank]
        sl = slice(rank * tokens, (rank + 1) * tokens)
        x = p["x"][sl].clone().requires_grad_(True)
        w_in = p["W_in"][lo:hi].clone().requires_grad_(True)
        w_sh = p["W_sh_in"].clone().requires_grad_(True)
        gen = EP.ep_forward_steps(x, p["w"][sl], p["idx"][sl], w_in, p["W_out"][lo:hi], w_sh,
                                  p["W_sh_out"], rank, bounds, "silu", expert_fn=torch_experts,
                                  shared_fn=torch_shared)
        out = EP.DistDriver().run(gen)
        gout = torch.randn(tokens * world, D, generator=torch.Generator().manual_seed(3),
                           dtype=torch.float64)[sl]
        out.backward(gout)
        EP.all_reduce_replicated_grads([w_sh])
        q.put((rank, out.detach().numpy(), x.grad.numpy(), w_in.grad.numpy(), w_sh.grad.numpy()))
        dist.destroy_process_group()
    except Exception as exc:  # surface the failure instead of hanging the parent
        q.put((rank, repr(exc)))


def test_gloo_two_ranks_match_single_rank():
    world, tokens = 2, 24
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, tokens, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    got = {}
    for _ in range(world):
        item = q.get(timeout=120)
        assert len(item) == 5, item
        got[item[0]] = item[1:]
    for pr in procs:
        pr.join(timeout=30)
    p = make_problem(tokens * world, seed=7)
    x = p["x"].clone().requires_grad_(True)
    W_in = p["W_in"].clone().requires_grad_(True)
    W_sh = p["W_sh_in"].clone().requires_grad_(True)
    ref = single_rank({**p, "W_in": W_in, "W_sh_in": W_sh}, x, p["w"], p["idx"])
    gout = torch.randn(tokens * world, D, generator=torch.Generator().manual_seed(3),
                       dtype=torch.float64)
    ref.backward(gout)
    bounds = EP.expert_partition(E, world)
    for r in range(world):
        out, dx, dw_in, dw_sh = (torch.from_numpy(a) for a in got[r])
        sl = slice(r * tokens, (r + 1) * tokens)
        lo, hi = bounds[r]
        assert torch.allclose(out, ref.detach()[sl], atol=1e-10)
        assert torch.allclose(dx, x.grad[sl], atol=1e-9)
        assert torch.allclose(dw_in, W_in.grad[lo:hi], atol=1e-9)     # owner-local, no all-reduce
        assert torch.allclose(dw_sh, W_sh.grad, atol=1e-9)            # replicated, all-reduced


def test_peer_memory_arena_layout_and_capacity():
    """Host-side arithmetic of the peer-memory path: the exchange buffers of a rank tile its arena
    without overlap, 256-byte aligned, and an owner's capacity covers every pair of every rank
    landing on its experts plus the 128-row padding of each local run."""
    from nanospeaker_b200 import ep_push, kernels
    from nanospeaker_b200.expert_parallel import expert_partition
    world, tokens, k, E, D = 8, 65536, 6, 76, 576
    cap = ep_push.EPRank.capacity(world, tokens, k, E)
    n_local = max(hi - lo for lo, hi in expert_partition(E, world))
    assert cap == kernels.l_cap(world * tokens * k, n_local) and cap % 128 == 0
    assert cap >= world * tokens * k + n_local * 127
    layout, size = ep_push.arena_layout(cap, D)
    sizes = {"xs": cap * D * 2, "douts": cap * D * 2, "y": cap * D * 2, "ydx": cap * D * 2,
             "sid": cap * 4, "pw": cap * 2, "dtw": cap * 2}
    spans = sorted((layout[n], layout[n] + sizes[n]) for n in sizes)
    assert all(lo % 256 == 0 for lo, _ in spans)
    assert all(a_hi <= b_lo for (_, a_hi), (b_lo, _) in zip(spans, spans[1:]))
    assert spans[-1][1] <= size and size % 256 == 0


@pytest.mark.parametrize("world,E,seed", [(8, 76, 0), (3, 7, 1), (2, 5, 2)])
def test_numpy_plan_of_the_peer_memory_layout_tiles_every_run(world, E, seed):
    """The layout rule itself (oracle.ep_plan; the reference has no multi-GPU form to pin it to):
    for every expert the home ranks' row ranges [send_row0, send_row0 + count) follow one another
    in rank order and fill exactly the first `total` rows of the owner's 128-aligned run; runs of an
    owner follow one another without gaps; the tile map names the run every live tile lies in."""
    import numpy as np
    from nanospeaker_b200.expert_parallel import expert_partition
    from oracle import moe_oracle as O
    rng = np.random.default_rng(seed)
    cnt = rng.integers(0, 400, size=(world, E))
    cnt[:, rng.integers(0, E)] = 0
    bounds = [lo for lo, _ in expert_partition(E, world)] + [E]
    plans = [O.ep_plan(cnt, bounds, r, 4096) for r in range(world)]
    tot = cnt.sum(0)
    for e in range(E):
        owner = int(plans[0][0][e])
        assert bounds[owner] <= e < bounds[owner + 1]
        assert all(int(p[0][e]) == owner for p in plans)
        run_start = int(plans[owner][2][e - bounds[owner]])
        nxt = run_start
        for r in range(world):                       # rank order inside the run, no gaps
            assert int(plans[r][1][e]) == nxt
            nxt += int(cnt[r, e])
        assert nxt == run_start + tot[e]
        assert int(plans[owner][3][e - bounds[owner]]) == tot[e]
    for r in range(world):
        _, _, offs, counts, live, eids = plans[r]
        assert offs[0] == 0 and offs[-1] == live and live % 128 == 0
        for i in range(len(counts)):
            assert offs[i + 1] - offs[i] == (counts[i] + 127) // 128 * 128
            assert (eids[offs[i] // 128: offs[i + 1] // 128] == i).all()
