"""Token sharding of the MoE block across the GPUs of one node.

Tokens are independent through the whole block (routing is per token, experts act per pair, the
combine is per token), so data parallelism needs no collective in the forward pass: every rank
holds the full weights (~34.5 MB per block in bf16) and a contiguous slice of the tokens. Training
adds one all-reduce (sum) of the weight gradients; `expert_counts` and the balance loss are
per-shard quantities unless reduced explicitly with `all_reduce_counts`.

The reference has no distributed code at all; these helpers are the multi-GPU surface of this
implementation. They work on any torch.distributed backend (NCCL on GPUs, gloo in CPU tests).
"""
from typing import Iterable, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_tokens: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[lo, hi) of this rank's contiguous token slice; slices differ by at most one token and
    earlier ranks take the extra ones."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    base, extra = divmod(n_tokens, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_tokens(x: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """This rank's rows of a [tokens, ...] tensor (a view)."""
    lo, hi = shard_bounds(x.shape[0], world_size, rank)
    return x[lo:hi]


def all_reduce_gradients(params: Iterable[torch.nn.Parameter], group=None,
                         average: bool = False) -> None:
    """Sum (or average) .grad of every parameter across ranks, in one flattened bucket per dtype:
    on NVSwitch the cost of an all-reduce is launch latency plus bytes over full-bandwidth links,
    so one large bucket beats many small ones."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    by_dtype = {}
    for p in params:
        if p.grad is not None:
            by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
    for grads in by_dtype.values():
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= dist.get_world_size(group)
        offset = 0
        for g in grads:
            g.copy_(flat[offset:offset + g.numel()].view_as(g))
            offset += g.numel()


def all_reduce_counts(counts: torch.Tensor, group=None) -> torch.Tensor:
    """Global per-expert routing counts from per-shard ones (for a global balance loss or logging)."""
    total = counts.clone()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
    return total


def enable_global_balance_loss(group=None) -> None:
    """From now on the kernel path's balance loss is that of the WHOLE batch over `group`'s ranks
    (the routing counts are all-reduced inside the block's op, 4 bytes per expert): every rank's
    `aux_loss` is its share, the shares sum to the global loss, and so do the gradients once the
    ranks' gradients are summed. Without this call (the default) each rank's loss is that of its
    own shard, which is what the reference computes in every process."""
    from . import moe_kernel as MK

    def reduce(counts: torch.Tensor) -> None:
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=group)

    MK.set_aux_reduce(reduce)


def disable_global_balance_loss() -> None:
    from . import moe_kernel as MK
    MK.set_aux_reduce(None)
