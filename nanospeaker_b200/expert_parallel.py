"""Expert parallelism for the dropless MoE block: routed experts partitioned over the GPUs of one
node, router and shared experts replicated, one all-to-all each way per direction.

The reference is single-GPU (no `torch.distributed` anywhere in it); this is the multi-GPU form of
its block for the "experts split 10/10/10/10/9/9/9/9 over 8 GPUs" workload. The math is the block's
(src/model/moe.py:345-418), partition-invariant up to the fp32 summation order of the combine:

  home rank:   route its tokens -> sort the (token, expert) pairs by owner rank
               -> DISPATCH all-to-all of the pairs' token rows and local expert ids
  owner rank:  dropless grouped FFN over the rows it received (the block's own kernels, weight 1)
               -> COMBINE all-to-all of the per-pair outputs back to the home rank
  home rank:   out[t] = sum_j w[t, j] * y[pair(t, j)] + shared(x[t])

The backward is autograd's mirror image: dOut rows travel out with the combine's transpose, dX rows
come back with the dispatch's. Gradients of the routed experts stay on their owner (no all-reduce);
the router and the shared experts are replicated, their gradients are summed over ranks by
`all_reduce_replicated_grads`.

This first version moves the rows with the backend's all-to-all (NCCL send/recv over NVLink on
GPUs, gloo in the CPU tests) and needs one host read per step for the split sizes. The rows are
copied into the owner's own memory before any kernel touches them; no kernel reads a peer's memory.

The step is written once, as a generator that yields at every exchange; `DistDriver` fulfils the
exchanges with torch.distributed, `run_loopback` runs G virtual ranks in one process on one device
(the exchanges become tensor shuffles) -- which is how the path is tested where fewer GPUs than
ranks are available.
"""
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import moe_kernel as MK


# ------------------------------------------------------------------------------- partition
def expert_partition(n_experts: int, world_size: int) -> List[Tuple[int, int]]:
    """[lo, hi) of the routed experts each rank owns: contiguous, sizes differ by at most one, the
    earlier ranks take the extra ones (76 over 8 -> 10,10,10,10,9,9,9,9)."""
    if world_size < 1 or n_experts < world_size:
        raise ValueError(f"cannot split {n_experts} experts over {world_size} ranks")
    base, extra = divmod(n_experts, world_size)
    out, lo = [], 0
    for r in range(world_size):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def owner_of(expert_idx: torch.Tensor, bounds: Sequence[Tuple[int, int]]) -> torch.Tensor:
    """Rank that owns each expert id (same shape as expert_idx, int64)."""
    starts = torch.tensor([lo for lo, _ in bounds[1:]], device=expert_idx.device,
                          dtype=expert_idx.dtype)
    return torch.bucketize(expert_idx, starts, right=True)


# ------------------------------------------------------------------- the local expert compute
def local_experts_cuda(rows: torch.Tensor, local_idx: torch.Tensor, w_in: torch.Tensor,
                       w_out: torch.Tensor, activation: str) -> torch.Tensor:
    """Dropless grouped FFN of the received rows through this rank's experts (the block's own
    dispatch + GEMM kernels with one expert per row and weight 1)."""
    if rows.shape[0] == 0:
        # keep the graph connected so that every rank takes part in the backward's exchanges
        return rows * 0 + (w_in.sum() + w_out.sum()).to(rows.dtype) * 0
    ones = rows.new_ones((rows.shape[0], 1))
    out, _ = MK.fused_moe_forward(rows, w_in, w_out, ones, local_idx.view(-1, 1), None, None,
                                  activation)
    return out


def shared_experts_cuda(x: torch.Tensor, w_sh_in: torch.Tensor, w_sh_out: torch.Tensor,
                        activation: str) -> torch.Tensor:
    """Sum of the shared experts' outputs for every token (each shared expert is an expert that
    every token visits with weight 1)."""
    s_n = w_sh_in.shape[0]
    idx = torch.arange(s_n, device=x.device).expand(x.shape[0], s_n).contiguous()
    out, _ = MK.fused_moe_forward(x, w_sh_in, w_sh_out, x.new_ones((x.shape[0], s_n)), idx, None,
                                  None, activation)
    return out


# ------------------------------------------------ home-side row movement on the block's kernels
def _kernel_rows(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


def _plan_tensors(order: torch.Tensor, n_pairs: int):
    """order (pair ids grouped by owner) as the permute kernel's slot list: int32, padded with the
    sentinel to a multiple of 8 rows, plus the device scalar holding the padded length."""
    cap = (n_pairs + 7) // 8 * 8
    sids = torch.full((cap,), n_pairs, dtype=torch.int32, device=order.device)
    sids[:n_pairs] = order
    npp = torch.full((1,), cap, dtype=torch.int32, device=order.device)
    return sids, npp


class _GatherPairRows(torch.autograd.Function):
    """rows[i] = x[order[i] // k] (permute kernel); backward: dx[t] = sum of its k pair rows
    (combine kernel through the inverse permutation)."""

    @staticmethod
    def forward(ctx, x, sids, npp, inv32, k, n_pairs):
        from . import kernels as K
        ctx.save_for_backward(inv32)
        ctx.k, ctx.t = k, x.shape[0]
        return K.permute(x, k, sids, npp)[:n_pairs]

    @staticmethod
    def backward(ctx, grad_rows):
        from . import kernels as K
        (inv32,) = ctx.saved_tensors
        return K.combine(grad_rows.contiguous(), inv32, ctx.t, ctx.k), None, None, None, None, None


class _WeightedCombine(torch.autograd.Function):
    """out[t] = sum_j w[t, j] * y_sorted[inv[t k + j]]: rows scaled by their weight, then the
    combine kernel's fp32 sum. Backward: dOut rows gathered back into pair order (permute kernel)."""

    @staticmethod
    def forward(ctx, y_sorted, topk_w, order, sids, npp, inv32):
        from . import kernels as K
        t, k = topk_w.shape
        w_sorted = topk_w.reshape(-1)[order]
        ctx.save_for_backward(y_sorted, w_sorted, order, sids, npp)
        ctx.shape = (t, k)
        return K.combine(y_sorted * w_sorted.unsqueeze(1), inv32, t, k)

    @staticmethod
    def backward(ctx, grad_out):
        from . import kernels as K
        y_sorted, w_sorted, order, sids, npp = ctx.saved_tensors
        t, k = ctx.shape
        g_rows = K.permute(grad_out.contiguous(), k, sids, npp)[: t * k]
        d_y = g_rows * w_sorted.unsqueeze(1)
        d_w_sorted = (y_sorted * g_rows).sum(-1, dtype=torch.float32)   # no fp32 [M, D] temporaries
        d_w = torch.empty(t * k, dtype=torch.float32, device=grad_out.device)
        d_w[order] = d_w_sorted
        return d_y, d_w.view(t, k).to(w_sorted.dtype), None, None, None, None


# ------------------------------------------------------------------------ the step, as a generator
def ep_forward_steps(x: torch.Tensor, topk_w: torch.Tensor, topk_idx: torch.Tensor,
                     w_in_local: torch.Tensor, w_out_local: torch.Tensor,
                     w_sh_in: Optional[torch.Tensor], w_sh_out: Optional[torch.Tensor],
                     rank: int, bounds: Sequence[Tuple[int, int]], activation: str,
                     expert_fn: Callable = local_experts_cuda,
                     shared_fn: Callable = shared_experts_cuda):
    """One rank's forward. Yields ("counts", send_counts) and ("rows", tensor, send_counts,
    recv_counts) requests; the driver sends back the received counts / rows. Returns (through
    StopIteration.value) the block output [T, D] for this rank's tokens.

    x [T, D]; topk_w [T, k] (x.dtype); topk_idx [T, k] int64 over ALL experts."""
    world = len(bounds)
    t, k = topk_idx.shape
    flat_idx = topk_idx.reshape(-1)
    dest = owner_of(flat_idx, bounds)                                # [T*k]
    order = torch.sort(dest, stable=True).indices                    # pairs grouped by owner
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = yield ("counts", send_counts)

    lo_of_dest = torch.tensor([lo for lo, _ in bounds], device=x.device)[dest]
    n_pairs = t * k
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    use_kernels = _kernel_rows(x) and n_pairs > 0
    if use_kernels:
        sids, npp = _plan_tensors(order, n_pairs)
        inv32 = inv.to(torch.int32)
        rows_send = _GatherPairRows.apply(x.contiguous(), sids, npp, inv32, k, n_pairs)
    else:
        rows_send = x[order // k]                                    # [T*k, D], differentiable
    idx_send = (flat_idx - lo_of_dest)[order]                        # expert id local to its owner
    send_list = send_counts.tolist()
    rows_recv = yield ("rows", rows_send, send_list, recv_counts)
    idx_recv = yield ("rows", idx_send, send_list, recv_counts)

    y_recv = expert_fn(rows_recv, idx_recv, w_in_local, w_out_local, activation)
    y_sorted = yield ("rows", y_recv, recv_counts, send_list)        # back home, in send order

    if use_kernels:
        out = _WeightedCombine.apply(y_sorted.contiguous(), topk_w, order, sids, npp, inv32)
    else:
        y_pairs = y_sorted[inv].view(t, k, -1)                       # pair (t, j) at [t, j]
        acc = torch.promote_types(x.dtype, torch.float32)           # sum in fp32 at least
        out = (y_pairs.to(acc) * topk_w.to(acc).unsqueeze(-1)).sum(1).to(x.dtype)
    if w_sh_in is not None:
        out = out + shared_fn(x, w_sh_in, w_sh_out, activation).to(out.dtype)
    return out.to(x.dtype)


# ------------------------------------------------------------------------------------ drivers
class _AllToAllRows(torch.autograd.Function):
    """Rows to / from every rank with explicit split sizes; the backward is the transposed
    exchange."""

    @staticmethod
    def forward(ctx, rows, send_counts, recv_counts, group):
        ctx.send_counts, ctx.recv_counts, ctx.group = send_counts, recv_counts, group
        out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_counts,
                               input_split_sizes=send_counts, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        back = grad.new_empty((sum(ctx.send_counts),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(back, grad.contiguous(), output_split_sizes=ctx.send_counts,
                               input_split_sizes=ctx.recv_counts, group=ctx.group)
        return back, None, None, None


class DistDriver:
    """Runs one rank's generator against a torch.distributed group."""

    def __init__(self, group=None):
        self.group = group

    def run(self, gen):
        try:
            req = next(gen)
            while True:
                if req[0] == "counts":
                    send = req[1]
                    recv = torch.empty_like(send)
                    dist.all_to_all_single(recv, send, group=self.group)
                    reply = recv.tolist()                      # the one host read of the step
                else:
                    _, rows, send_counts, recv_counts = req
                    if rows.is_floating_point():
                        reply = _AllToAllRows.apply(rows, list(send_counts), list(recv_counts),
                                                    self.group)
                    else:
                        reply = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
                        dist.all_to_all_single(reply, rows.contiguous(),
                                               output_split_sizes=list(recv_counts),
                                               input_split_sizes=list(send_counts),
                                               group=self.group)
                req = gen.send(reply)
        except StopIteration as stop:
            return stop.value


def run_loopback(gens: Sequence) -> List[torch.Tensor]:
    """Runs the generators of G virtual ranks in lock step in one process; an exchange is a
    differentiable shuffle of row blocks between them. Returns every rank's result."""
    world = len(gens)
    reqs = [next(g) for g in gens]
    results: List[Optional[torch.Tensor]] = [None] * world
    live = list(range(world))
    while live:
        kind = reqs[live[0]][0]
        assert all(reqs[r][0] == kind for r in live), "virtual ranks fell out of step"
        if kind == "counts":
            matrix = torch.stack([reqs[r][1] for r in range(world)])        # [src, dst]
            replies = [matrix[:, r].tolist() for r in range(world)]
        else:
            pieces = [torch.split(reqs[r][1], list(reqs[r][2])) for r in range(world)]
            replies = [torch.cat([pieces[src][dst] for src in range(world)])
                       for dst in range(world)]
        nxt = []
        for r in live:
            try:
                reqs[r] = gens[r].send(replies[r])
                nxt.append(r)
            except StopIteration as stop:
                results[r] = stop.value
        live = nxt
    return results


# ------------------------------------------------------------------------------ convenience
def ep_block_forward(x, router, w_in_local, w_out_local, w_sh_in, w_sh_out, activation: str,
                     group=None):
    """The expert-parallel block on this rank: router (replicated) -> exchanges -> output.
    Returns (out [T, D], counts of this rank's tokens per expert [E] int64)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    bounds = expert_partition(router.n_experts, world)
    topk_w, topk_idx, _ = router(x)
    gen = ep_forward_steps(x, topk_w, topk_idx, w_in_local, w_out_local, w_sh_in, w_sh_out, rank,
                           bounds, activation)
    out = DistDriver(group).run(gen)
    counts = torch.bincount(topk_idx.reshape(-1), minlength=router.n_experts)
    return out, counts


def all_reduce_replicated_grads(params, group=None) -> None:
    """Sum the gradients of the replicated parameters (router, shared experts) over the ranks."""
    from .parallel import all_reduce_gradients
    all_reduce_gradients(params, group=group)
