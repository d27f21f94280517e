"""Decode-shaped use of the MoE block: a stack of blocks on a small, fixed batch of tokens (one
token per sequence), forward only, replayed from one CUDA graph.

At T = 64 every expert sees a handful of rows and each block's launches take a few
microseconds: the cost is launch latency, not arithmetic, so the whole stack is captured once and
replayed. The caller loop this stands for is `generate` -> `Block.forward` -> `MoEBlock.forward`
with T = batch size in eval mode (src/model/nanospeaker.py:254-269, 165-169); attention, norms and
the KV cache of that loop are outside this package, so the stack here chains the blocks through
the residual only: x <- x + block_l(x).
"""
from typing import List, Sequence

import torch

from .moe import MoEBlock


class StackedMoEDecoder:
    """`x + block(x)` over a list of MoE blocks (eval mode, CUDA, bf16), graph-replayed per batch
    size.

    step(x) runs the stack on x [T, d_model] and returns the result (a tensor owned by the runner:
    it is overwritten by the next step with the same T). The first call for a given T captures the
    graph; later calls copy x into the graph's input and replay."""

    def __init__(self, blocks: Sequence[MoEBlock], combine: str = "store"):
        # "store": per-pair rows summed in fp32 in pair order, so a replay reproduces the eager
        # stack bit for bit and a token's routing further down the stack cannot flip from run to
        # run; at decode sizes the separate combine launch costs next to nothing. "atomic" is the
        # training default of the library (see moe_kernel.COMBINE_MODES).
        self.combine = combine
        self.blocks: List[MoEBlock] = list(blocks)
        if not self.blocks:
            raise ValueError("need at least one block")
        for b in self.blocks:
            b.eval()
        self._graphs = {}
        self._consts = {}

    def _fast_args(self, b: MoEBlock, x: torch.Tensor):
        """Per-block constants of the kernel path (weights are fixed while decoding): the padded
        router weight and the weights in x.dtype, built on first use. None when the block's
        kernels decline this input (then the block's own forward runs)."""
        if not b._whole_block_ok(x):      # biases, a capacity, ...: the block's own forward
            return None
        key = (id(b), x.dtype, x.device)
        if key not in self._consts:
            from . import moe_kernel as MK
            cast = lambda t: None if t is None else t.detach().to(x.dtype).contiguous()
            bias = b.router.logit_bias
            self._consts[key] = (
                MK.pad_router_weight(b.router.W.detach(), x.dtype),
                None if bias is None else bias.detach().to(torch.float32).contiguous(),
                cast(b.W_in), cast(b.W_out), cast(b.W_sh_in), cast(b.W_sh_out),
                b.n_experts, b.router.top_k, bool(b.router.normalize_weights), b._kernel_act)
        return self._consts[key]

    @torch.no_grad()
    def eager(self, x: torch.Tensor) -> torch.Tensor:
        """x <- x + block(x) through the stack. On the kernel path a block is six launches: the
        residual is added inside the combine, the padded router weight is kept between steps,
        and the per-call bookkeeping of MoEBlock.forward (expert_counts, aux_loss) is skipped."""
        from . import moe_kernel as MK
        x = x.contiguous()
        for b in self.blocks:
            args = self._fast_args(b, x)
            x = x + b(x) if args is None else MK.moe_block_inference(x, *args, residual=x,
                                                                      combine=b.combine_mode or self.combine)
        return x

    @torch.no_grad()
    def _capture(self, x: torch.Tensor):
        static_x = x.clone()
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):           # warm-up outside the capture (lazy initialisations)
            for _ in range(2):
                self.eager(static_x)
        torch.cuda.current_stream(x.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.eager(static_x)
        return graph, static_x, out

    @torch.no_grad()
    def step(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("StackedMoEDecoder runs on CUDA tensors only")
        key = (tuple(x.shape), x.dtype, x.device)
        if key not in self._graphs:
            self._graphs[key] = self._capture(x)
        graph, static_x, out = self._graphs[key]
        static_x.copy_(x)
        graph.replay()
        return out
