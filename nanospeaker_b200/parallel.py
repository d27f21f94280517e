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


class PeerGradAllReduce:
    """Sum of a flat gradient bucket over the GPUs of one node through peer memory and the copy
    engines, for a step that also streams its inputs from the host.

    An NCCL all-reduce is a kernel that holds SMs and moves its bytes with loads and stores; run
    under the next step's compute next to that step's host-to-device input copy it stretched the
    end-to-end step on 4 B200s to 0.77 ms. Here the bytes move by device-to-device copies into the
    peers' buffers (symmetric memory, plain stores over NVLink, no multicast) and the only kernels
    are a local sum and two one-element barriers: 0.59 ms for the same step, the device-resident
    step unchanged (0.506 ms either way; on 2 GPUs 0.504 against 0.492 and 0.544 against 0.577 end
    to end).

      1. reduce-scatter: rank r copies chunk j of its bucket into slot r of rank j's receive
         buffer (N - 1 copies of numel / N elements);           -- barrier --
      2. rank j sums its N slots in rank order in fp32 (deterministic) into chunk j of its result;
      3. all-gather: rank j copies that chunk into chunk j of every peer's result (N - 1 copies);
                                                                 -- barrier --
    The same bytes cross the links as in a ring all-reduce (2 (N - 1) / N of the bucket per rank).
    Buffers are double-buffered by call parity, so a rank that is one call ahead never writes into
    slots a peer still reads. Everything is issued on the current stream; the result is a view that
    stays valid until the call after next.

    fill(tensors) flattens into the bucket; __call__() reduces it and returns the summed flat view.
    """

    def __init__(self, numel: int, device, group=None, dtype=torch.bfloat16):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.numel = numel
        n = self.world
        self.chunk = ((numel + n - 1) // n + 255) // 256 * 256
        per_parity = 2 * n * self.chunk            # receive slots [n, chunk] + result [n * chunk]
        arena = symm_mem.empty(2 * per_parity, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(arena, group if group is not None else dist.group.WORLD)
        self.arena = arena
        self.bucket = torch.zeros(n * self.chunk, dtype=dtype, device=device)
        self.flag = torch.zeros(1, device=device)
        self.parity = 0
        c = self.chunk

        def views(rank):
            out = []
            for p in range(2):
                base = p * per_parity
                recv = self.handle.get_buffer(rank, (n, c), dtype, base)
                res = self.handle.get_buffer(rank, (n * c,), dtype, base + n * c)
                out.append((recv, res))
            return out
        self.peer = [views(j) for j in range(n)]     # [rank][parity] -> (recv [n, c], result [n c])

    def fill(self, tensors) -> None:
        torch.cat([t.reshape(-1) for t in tensors], out=self.bucket[: self.numel])

    def _barrier(self) -> None:
        dist.all_reduce(self.flag, group=self.group)

    def __call__(self) -> torch.Tensor:
        n, r, c, p = self.world, self.rank, self.chunk, self.parity
        self.parity ^= 1
        chunks = self.bucket.view(n, c)
        for step in range(n):                      # start at the next rank: ranks write to
            j = (r + 1 + step) % n                 # different peers at any one time
            self.peer[j][p][0][r].copy_(chunks[j], non_blocking=True)
        self._barrier()
        recv, res = self.peer[r][p]
        mine = res[r * c:(r + 1) * c]
        torch.sum(recv, dim=0, dtype=torch.float32, out=self._acc())
        mine.copy_(self._acc())
        for step in range(n - 1):
            j = (r + 1 + step) % n
            self.peer[j][p][1][r * c:(r + 1) * c].copy_(mine, non_blocking=True)
        self._barrier()
        return res[: self.numel]

    def _acc(self) -> torch.Tensor:
        if not hasattr(self, "_acc_buf"):
            self._acc_buf = torch.empty(self.chunk, dtype=torch.float32, device=self.bucket.device)
        return self._acc_buf


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
