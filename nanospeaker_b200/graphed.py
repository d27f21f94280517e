"""CUDA-graph replay of a MoE block behind the module interface.

A block's training step is ~40 launches of a few to a few tens of microseconds each; issued one by
one from Python they cost more host time than the GPU needs to run them (about 1.0 ms against
0.45 ms at T = 16384). Nothing in the kernel path reads a value on the host or has a data-dependent
shape, so forward and backward can each be captured once per input shape and replayed.
`GraphedMoEBlock` does that and stays a drop-in for the block: same call, same post-forward
attributes (`aux_loss`, `expert_counts`, `dropped`), autograd works as usual (the two graphs are
tied together by torch.cuda.make_graphed_callables), parameters stay those of the wrapped block.

The caller loop this serves is the reference's micro-step, `loss, aux = model(x, y); (loss + aux)
.backward()` (src/train/train.py:317-324), where the block is called once per layer and step with a
fixed [batch, seq, d_model] shape.
"""
from typing import Dict, Tuple

import torch
from torch import nn

from .moe import MoEBlock


class _BlockWithAux(nn.Module):
    """(out, aux_loss as fp32, expert_counts as fp32): the tensors a graph has to hand back."""

    def __init__(self, block: MoEBlock):
        super().__init__()
        self.block = block

    def forward(self, x):
        out = self.block(x)
        aux = self.block.aux_loss.to(torch.float32).reshape(())
        return out, aux, self.block.expert_counts.to(torch.float32)


class GraphedMoEBlock(nn.Module):
    """`block(x)` replayed from CUDA graphs, one forward/backward pair per (input shape, dtype,
    training mode), captured on first use. Inputs the kernels decline (CPU tensors, other dtypes,
    exploration noise: anything `block._whole_block_ok` turns down) go through the block itself.

    The captured graphs hold the parameters by address: change them in place (an optimizer step
    does), do not replace them. A capture costs a few warm-up steps; do the first call of every
    shape outside any timed region."""

    def __init__(self, block: MoEBlock, warmup_iters: int = 3):
        super().__init__()
        self.block = block
        self.warmup_iters = warmup_iters
        self._pair = _BlockWithAux(block)
        self._graphed: Dict[Tuple, object] = {}

    # the attributes callers read after a forward (src/train/metrics.py:84-97)
    @property
    def aux_loss(self):
        return self.block.aux_loss

    @property
    def expert_counts(self):
        return self.block.expert_counts

    @property
    def dropped(self):
        return self.block.dropped

    @property
    def router(self):
        return self.block.router

    def _callable_for(self, x: torch.Tensor):
        key = (tuple(x.shape), x.dtype, x.device, self.block.training, x.requires_grad)
        fn = self._graphed.get(key)
        if fn is None:
            sample = torch.zeros_like(x).normal_().requires_grad_(x.requires_grad)
            fn = torch.cuda.make_graphed_callables(
                self._pair, (sample,), num_warmup_iters=self.warmup_iters,
                allow_unused_input=True)
            self._graphed[key] = fn
        return fn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b = self.block
        x2 = x.reshape(-1, x.shape[-1]) if x.dim() > 1 else x
        # (without autograd there is no backward to pair the forward with: the block's own
        # inference path is the lighter one then, and nanospeaker_b200.decode graphs it)
        if (not x.is_cuda or x2.shape[0] == 0 or x.shape[-1] != b.d_model
                or not torch.is_grad_enabled() or not b._whole_block_ok(x2)
                or (b.training and b.router.noise_std)):   # noise: fresh random numbers every call
            return b(x)
        out, aux, counts = self._callable_for(x)(x)
        full = b.router.wants_probs()
        b.aux_loss = aux if full else torch.zeros((), device=x.device, dtype=x.dtype)
        b.expert_counts = counts.detach().to(torch.int32)
        return out
