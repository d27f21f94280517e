"""Expert-parallel block on the GPU: G virtual ranks run in lock step on one device (the exchanges
are tensor shuffles, the per-rank expert compute is the CUDA kernels) and must reproduce the
single-GPU block on the concatenated tokens, forward and backward. With two or more GPUs the same
step also runs over NCCL (see the distributed test at the end)."""
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _block(seed=0, E=76, k=6, S=2, D=576):
    from nanospeaker_b200 import MoEBlock
    torch.manual_seed(seed)
    m = MoEBlock(D, E, d_ff=192, top_k=k, n_shared=S, capacity_factor=None)
    with torch.no_grad():
        m.router.W.copy_(torch.randn(D, E) * 0.02)
        m.W_in.copy_(torch.randn(E, D, 256) * D ** -0.5)
        m.W_out.copy_(torch.randn(E, 128, D) * 128 ** -0.5)
        m.W_sh_in.copy_(torch.randn(S, D, 256) * D ** -0.5)
        m.W_sh_out.copy_(torch.randn(S, 128, D) * 128 ** -0.5)
    return m.to(torch.bfloat16).cuda().eval()


@pytest.mark.parametrize("world,tokens", [(2, 1024), (8, 300), (4, 1)])
def test_loopback_ranks_match_the_single_gpu_block(world, tokens):
    from nanospeaker_b200 import expert_parallel as EP
    m = _block(seed=world)
    E = m.router.n_experts
    x_all = torch.randn(world * tokens, 576, device="cuda").bfloat16()
    gout = torch.randn_like(x_all)

    # one routing decision for both sides (bf16 logits tie easily; the same rows routed in
    # differently shaped batches could round differently)
    from nanospeaker_b200 import fused_moe_forward
    xr = x_all.clone().requires_grad_(True)
    w_r, idx_r, _ = m.router(xr)
    ref, _ = fused_moe_forward(xr, m.W_in, m.W_out, w_r, idx_r, None, None, "silu",
                               w_sh_in=m.W_sh_in, w_sh_out=m.W_sh_out)
    ref.backward(gout)
    ref_grads = {n: p.grad.clone() for n, p in m.named_parameters()}
    for p in m.parameters():
        p.grad = None

    xe = x_all.clone().requires_grad_(True)
    w_e, idx_e, _ = m.router(xe)
    assert torch.equal(idx_e, idx_r)
    bounds = EP.expert_partition(E, world)
    gens = []
    for r in range(world):
        sl = slice(r * tokens, (r + 1) * tokens)
        lo, hi = bounds[r]
        gens.append(EP.ep_forward_steps(xe[sl], w_e[sl], idx_e[sl], m.W_in[lo:hi], m.W_out[lo:hi],
                                        m.W_sh_in, m.W_sh_out, r, bounds, "silu"))
    out = torch.cat(EP.run_loopback(gens))
    assert rel_l2(out.detach(), ref.detach().float()) < TOL
    out.backward(gout)
    assert rel_l2(xe.grad, xr.grad.float()) < TOL
    for n, p in m.named_parameters():
        assert p.grad is not None, n
        assert rel_l2(p.grad, ref_grads[n].float()) < (2e-2 if n == "router.W" else TOL), n
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


def _report_and_leave(q, rank, text):
    """A failed rank hands its error to the parent and leaves at once, without tearing the process
    group down: its peer may be inside a collective that this rank will never join, and the hard
    exit is what lets that collective end with an error instead of waiting."""
    import os
    q.put((rank, text))
    q.close()
    q.join_thread()
    os._exit(1)


def _collect(procs, q, world):
    """Results of all ranks, or an assertion; whatever happens, no worker is left behind holding a
    GPU (a rank stuck in a collective is terminated, then killed)."""
    import queue
    got = {}
    try:
        for _ in range(world):
            try:
                item = q.get(timeout=300)
            except queue.Empty:
                raise AssertionError("a rank did not report within 300 s")
            assert len(item) == 5, item
            got[item[0]] = item[1:]
        for p in procs:
            p.join(timeout=60)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    return got


def _nccl_worker(rank, world, port, tokens, q):
    try:
        import os
        import torch.distributed as dist
        from nanospeaker_b200 import expert_parallel as EP
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        import datetime
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=120))
        m = _block(seed=5)
        E = m.router.n_experts
        g = torch.Generator().manual_seed(11)
        x_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
        gout_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
        sl = slice(rank * tokens, (rank + 1) * tokens)
        lo, hi = EP.expert_partition(E, world)[rank]
        x = x_all[sl].cuda().requires_grad_(True)
        w_in = m.W_in.detach()[lo:hi].clone().requires_grad_(True)
        w_out = m.W_out.detach()[lo:hi].clone().requires_grad_(True)
        out, _ = EP.ep_block_forward(x, m.router, w_in, w_out, m.W_sh_in, m.W_sh_out, "silu")
        out.backward(gout_all[sl].cuda())
        EP.all_reduce_replicated_grads([m.router.W, m.W_sh_in, m.W_sh_out])
        torch.cuda.synchronize()
        q.put((rank, out.detach().float().cpu().numpy(), x.grad.float().cpu().numpy(),
               w_in.grad.float().cpu().numpy(), m.W_sh_in.grad.float().cpu().numpy()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # surface the failure instead of hanging the parent
        _report_and_leave(q, rank, repr(exc))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_over_nccl_match_the_single_gpu_block():
    import socket
    import torch.multiprocessing as mp
    from nanospeaker_b200 import expert_parallel as EP
    world, tokens = 2, 2048
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, tokens, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = _collect(procs, q, world)
    m = _block(seed=5)
    g = torch.Generator().manual_seed(11)
    x_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
    gout_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
    from nanospeaker_b200 import fused_moe_forward
    xr = x_all.cuda().requires_grad_(True)
    routed = [m.router(xr[r * tokens:(r + 1) * tokens]) for r in range(world)]   # as the ranks do
    ref, _ = fused_moe_forward(xr, m.W_in, m.W_out, torch.cat([w for w, _, _ in routed]),
                               torch.cat([i for _, i, _ in routed]), None, None, "silu",
                               w_sh_in=m.W_sh_in, w_sh_out=m.W_sh_out)
    ref.backward(gout_all.cuda())
    bounds = EP.expert_partition(m.router.n_experts, world)
    for r in range(world):
        out, dx, dw_in, dw_sh = (torch.from_numpy(a) for a in got[r])
        sl = slice(r * tokens, (r + 1) * tokens)
        lo, hi = bounds[r]
        assert rel_l2(out, ref.detach().float().cpu()[sl]) < TOL
        assert rel_l2(dx, xr.grad.float().cpu()[sl]) < TOL
        assert rel_l2(dw_in, m.W_in.grad.float().cpu()[lo:hi]) < TOL
        assert rel_l2(dw_sh, m.W_sh_in.grad.float().cpu()) < TOL


@pytest.mark.parametrize("world,tokens", [(2, 1024), (8, 300), (4, 1), (3, 777)])
def test_push_pull_ranks_match_the_single_gpu_block(world, tokens):
    """The peer-memory path (rows pushed straight into the owners' slot-ordered buffers, combine
    pulling from them) with G virtual ranks on one device, against the single-GPU block on the
    concatenated tokens: outputs, dX, and every weight gradient."""
    from nanospeaker_b200 import ep_push, kernels
    from nanospeaker_b200 import expert_parallel as EP
    m = _block(seed=10 + world)
    E, k, S, D = m.router.n_experts, m.router.top_k, 2, 576
    x_all = torch.randn(world * tokens, D, device="cuda").bfloat16()
    gout = torch.randn_like(x_all)

    xr = x_all.clone().requires_grad_(True)
    ref = m(xr)                                   # whole-block op, eval mode
    ref.backward(gout)
    ref_grads = {n: p.grad.clone() for n, p in m.named_parameters()}

    grp = ep_push.LoopbackGroup(world, E, k, S, D, tokens, x_all.device)
    xs = list(x_all.split(tokens))
    for step in range(2):                         # twice: the buffers keep the last step's rows
        outs = grp.forward(xs, m.router, m.W_in.detach(), m.W_out.detach(), m.W_sh_in.detach(),
                           m.W_sh_out.detach(), "silu")
        out = torch.cat([o for o, _ in outs])
        assert rel_l2(out, ref.detach().float()) < TOL
        grads = grp.backward(list(gout.split(tokens)))
        dx = torch.cat([g[0] for g in grads])
        assert rel_l2(dx, xr.grad.float()) < TOL
        bounds = EP.expert_partition(E, world)
        for r, (lo, hi) in enumerate(bounds):
            assert rel_l2(grads[r][2], ref_grads["W_in"][lo:hi].float()) < TOL
            assert rel_l2(grads[r][3], ref_grads["W_out"][lo:hi].float()) < TOL
        total = lambda i: sum(g[i].float() for g in grads)
        assert rel_l2(total(1), ref_grads["router.W"].float()) < 2e-2
        assert rel_l2(total(4), ref_grads["W_sh_in"].float()) < TOL
        assert rel_l2(total(5), ref_grads["W_sh_out"].float()) < TOL
    kernels.check_status("cuda")


def _push_worker(rank, world, port, tokens, q):
    try:
        import os
        import torch.distributed as dist
        from nanospeaker_b200 import ep_push
        from nanospeaker_b200 import expert_parallel as EP
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        import datetime
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=120))
        m = _block(seed=5)
        E = m.router.n_experts
        g = torch.Generator().manual_seed(11)
        x_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
        gout_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
        sl = slice(rank * tokens, (rank + 1) * tokens)
        lo, hi = EP.expert_partition(E, world)[rank]
        grp = ep_push.SymmetricGroup(E, m.router.top_k, 2, 576, tokens, dev)
        w_in = m.W_in.detach()[lo:hi].clone().requires_grad_(True)
        w_out = m.W_out.detach()[lo:hi].clone().requires_grad_(True)
        for step in range(2):                    # the second step reuses the exchange buffers
            x = x_all[sl].cuda().requires_grad_(True)
            for p in (w_in, w_out, m.router.W, m.W_sh_in, m.W_sh_out):
                p.grad = None
            out, _, _ = ep_push.ep_push_block_forward(x, m.router, w_in, w_out, m.W_sh_in,
                                                      m.W_sh_out, "silu", grp)
            out.backward(gout_all[sl].cuda())
        EP.all_reduce_replicated_grads([m.router.W, m.W_sh_in, m.W_sh_out])
        torch.cuda.synchronize()
        from nanospeaker_b200 import kernels
        kernels.check_status(dev)
        q.put((rank, out.detach().float().cpu().numpy(), x.grad.float().cpu().numpy(),
               w_in.grad.float().cpu().numpy(), m.W_sh_in.grad.float().cpu().numpy()))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # surface the failure instead of hanging the parent
        import traceback
        _report_and_leave(q, rank, repr(exc) + traceback.format_exc())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_over_peer_memory_match_the_single_gpu_block():
    """One process per GPU, exchange buffers in symmetric memory, rows pushed and pulled through
    peer pointers: outputs and gradients of two steps against the single-GPU block."""
    import socket
    import torch.multiprocessing as mp
    from nanospeaker_b200 import expert_parallel as EP
    world, tokens = 2, 2048
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_push_worker, args=(r, world, port, tokens, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = _collect(procs, q, world)
    m = _block(seed=5)
    g = torch.Generator().manual_seed(11)
    x_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
    gout_all = torch.randn(world * tokens, 576, generator=g).bfloat16()
    xr = x_all.cuda().requires_grad_(True)
    ref = m(xr)
    ref.backward(gout_all.cuda())
    bounds = EP.expert_partition(m.router.n_experts, world)
    for r in range(world):
        out, dx, dw_in, dw_sh = (torch.from_numpy(a) for a in got[r])
        sl = slice(r * tokens, (r + 1) * tokens)
        lo, hi = bounds[r]
        assert rel_l2(out, ref.detach().float().cpu()[sl]) < TOL
        assert rel_l2(dx, xr.grad.float().cpu()[sl]) < TOL
        assert rel_l2(dw_in, m.W_in.grad.float().cpu()[lo:hi]) < TOL
        assert rel_l2(dw_sh, m.W_sh_in.grad.float().cpu()) < TOL


@pytest.mark.parametrize("world,E,seed", [(8, 76, 0), (2, 76, 1), (3, 7, 2), (4, 200, 3)])
def test_plan_kernel_matches_the_numpy_plan(world, E, seed):
    """ep_plan's integers (owner of every expert, first destination row of this rank's pairs,
    the owner's own 128-aligned offsets / counts / live length / tile map) bit for bit, with empty
    experts and empty ranks in the count matrix."""
    import numpy as np
    from nanospeaker_b200 import kernels as K
    from nanospeaker_b200.expert_parallel import expert_partition
    from oracle import moe_oracle as O
    rng = np.random.default_rng(seed)
    cnt = rng.integers(0, 700, size=(world, E)).astype(np.int32)
    cnt[:, rng.integers(0, E, size=max(E // 5, 1))] = 0          # experts nobody picked
    cnt[rng.integers(0, world)] = 0                              # a rank without tokens
    bounds = [lo for lo, _ in expert_partition(E, world)] + [E]
    cap = K.l_cap(int(cnt.sum()), max(b - a for a, b in zip(bounds, bounds[1:])))
    cnt_d = torch.from_numpy(cnt).cuda()
    bounds_d = torch.tensor(bounds, dtype=torch.int32, device="cuda")
    for rank in range(world):
        n_local = bounds[rank + 1] - bounds[rank]
        got = K.ep_plan(cnt_d, bounds_d, rank, n_local, cap // 128)
        want = O.ep_plan(cnt, bounds, rank, cap // 128)
        live = want[4]
        assert np.array_equal(got[0].cpu().numpy(), want[0])
        assert np.array_equal(got[1].cpu().numpy(), want[1])
        assert np.array_equal(got[2].cpu().numpy(), want[2])
        assert np.array_equal(got[3].cpu().numpy()[:n_local], want[3])
        assert int(got[4]) == live
        assert np.array_equal(got[5].cpu().numpy()[: live // 128], want[5][: live // 128])
        assert not got[5].cpu().numpy()[live // 128:].any()


def test_push_pull_ranks_without_shared_experts():
    """The same comparison for a block without shared experts (no local extra buffer, the whole
    slot order is pushed) and with other sizes: E=16 over 4 ranks, top-2, D=192."""
    from nanospeaker_b200 import MoEBlock, ep_push, kernels
    from nanospeaker_b200 import expert_parallel as EP
    torch.manual_seed(3)
    world, tokens, E, k, D = 4, 500, 16, 2, 192
    m = MoEBlock(D, E, d_ff=192, top_k=k, n_shared=0, capacity_factor=None)
    with torch.no_grad():
        m.router.W.copy_(torch.randn(D, E) * 0.05)
        m.W_in.copy_(torch.randn(E, D, 256) * D ** -0.5)
        m.W_out.copy_(torch.randn(E, 128, D) * 128 ** -0.5)
    m = m.to(torch.bfloat16).cuda().eval()
    x_all = torch.randn(world * tokens, D, device="cuda").bfloat16()
    gout = torch.randn_like(x_all)
    xr = x_all.clone().requires_grad_(True)
    ref = m(xr)
    ref.backward(gout)
    grp = ep_push.LoopbackGroup(world, E, k, 0, D, tokens, x_all.device)
    outs = grp.forward(list(x_all.split(tokens)), m.router, m.W_in.detach(), m.W_out.detach(),
                       None, None, "silu")
    assert rel_l2(torch.cat([o for o, _ in outs]), ref.detach().float()) < TOL
    grads = grp.backward(list(gout.split(tokens)))
    assert rel_l2(torch.cat([g[0] for g in grads]), xr.grad.float()) < TOL
    for r, (lo, hi) in enumerate(EP.expert_partition(E, world)):
        assert rel_l2(grads[r][2], m.W_in.grad[lo:hi].float()) < TOL
        assert rel_l2(grads[r][3], m.W_out.grad[lo:hi].float()) < TOL
    assert rel_l2(sum(g[1].float() for g in grads), m.router.W.grad.float()) < 2e-2
    kernels.check_status("cuda")


def _peer_allreduce_worker(rank, world, port, q):
    try:
        import os
        import datetime
        import torch.distributed as dist
        from nanospeaker_b200.parallel import PeerGradAllReduce
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=120))
        numel = 1_000_003                      # not a multiple of anything: padded chunks
        ar = PeerGradAllReduce(numel, dev)
        worst = 0.0
        for it in range(4):                    # both buffer parities, twice
            g = torch.Generator(device="cpu").manual_seed(100 * it + rank)
            grads = [torch.randn(1000, 777, generator=g).bfloat16().to(dev),
                     torch.randn(numel - 777000, generator=g).bfloat16().to(dev)]
            ar.fill(grads)
            want = ar.bucket[:numel].clone()
            dist.all_reduce(want)
            got = ar()
            torch.cuda.synchronize()
            worst = max(worst, float((got.float() - want.float()).abs().max()))
        q.put((rank, worst, int(got.numel()), 0, 0))
        q.close()
        q.join_thread()   # os._exit below skips the queue's own flush: without this the result
        dist.barrier()    # can be lost and the parent waits for a rank that has long finished
        torch.cuda.synchronize()
        os._exit(0)       # (symmetric-memory buffers: leave without tearing the group down)
    except Exception as exc:
        _report_and_leave(q, rank, repr(exc))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_peer_memory_gradient_allreduce_equals_nccl():
    """parallel.PeerGradAllReduce (reduce-scatter + all-gather by device-to-device copies through
    peer memory, local fp32 sum in rank order) against ncclAllReduce on the same bf16 bucket: at
    two ranks both round one fp32 sum per element, so the results are bit-equal."""
    import socket
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_peer_allreduce_worker, args=(r, world, port, q))
             for r in range(world)]
    for p in procs:
        p.start()
    got = _collect(procs, q, world)
    for r in range(world):
        worst, numel = got[r][0], got[r][1]
        assert numel == 1_000_003
        assert worst == 0.0, f"rank {r}: max abs diff {worst}"
