"""MoEBlock: drop-in for nanoSpeaker's sparse Mixture-of-Experts feed-forward block
(src/model/moe.py:42-474) with the dropless path running on hand-written sm_100a kernels.

Constructor keywords, parameter names and shapes, the `router` sub-module, `forward`,
`dense_forward` and the post-forward attributes `aux_loss`, `expert_counts`, `dropped` are those of
the reference, so its callers (Block in src/model/nanospeaker.py:153-169, moe_health in
src/train/metrics.py:84-97) and its checkpoints work unchanged.

Paths, in the order `forward` tries them:
  1. kernel    CUDA + bf16 + a named activation + shapes the tiles cover: router top-k, dispatch,
               permute, grouped GEMMs, combine and the shared experts all run as the `moe_b200`
               ops (one whole-block op when there are no biases and no capacity; router +
               dispatch + experts ops otherwise). No host sync. A missing or
               failing library raises; nothing is silently rerouted. An explicit capacity_factor
               (the reference's padded path, src/model/moe.py:225-283) runs on the same kernels:
               the dispatch drops the pairs over capacity instead of padding a batch.
  2. torch     the per-expert loop in plain torch (src/model/moe.py:377-418) for everything the
               kernels decline (CPU, fp32/fp64, custom activations), with or without a capacity.
"""
import math

import torch
from torch import nn

from . import moe_kernel as MK
from .glu import glu_hidden_dim, make_glu
from .moe_kernel import (KERNEL_ACTIVATIONS, fused_moe_block, fused_moe_forward,
                         kernel_supported)
from .router import TopKRouter
from .utils import ACTIVATIONS, resolve_activation

# Capacity the "auto" setting resolves to where the kernels do not run.
AUTO_CAPACITY = 1.25


class MoEBlock(nn.Module):
    """Sparse MoE feed-forward block with GLU experts (SwiGLU by default).

    Args (identical to src/model/moe.py:96-112):
        d_model, n_experts, d_ff (FFN width each expert replaces; GLU hidden = 2*d_ff//3,
        default 4*d_model), top_k, n_shared (always-on experts), capacity_factor (float, None
        for dropless, or "auto" = None where the kernels run and 1.25 elsewhere), activation,
        bias, normalize_weights, aux_loss_coef, noise_std, fused (accepted, unused: the GLU is
        fused into the GEMM epilogue on the kernel path), kernel, std.
    """

    def __init__(self, d_model, n_experts, d_ff=None, top_k=2, n_shared=0,
                 capacity_factor="auto", activation="silu", bias=False, normalize_weights=True,
                 aux_loss_coef=1e-2, noise_std=0.0, fused=True, kernel=True, std=0.02):
        super().__init__()
        d_ff = 4 * d_model if d_ff is None else d_ff
        self.d_model, self.n_experts, self.d_ff = d_model, n_experts, d_ff
        self.d_hidden = glu_hidden_dim(d_ff)
        self.top_k = top_k
        if n_shared < 0:
            raise ValueError(f"n_shared ({n_shared}) cannot be negative.")
        self.n_shared = n_shared
        if capacity_factor != "auto" and capacity_factor is not None and capacity_factor <= 0:
            raise ValueError(
                f"capacity_factor ({capacity_factor}) must be > 0, None, or \"auto\"."
            )
        self._capacity_setting = capacity_factor

        self.router = TopKRouter(d_model, n_experts, top_k, normalize_weights, aux_loss_coef,
                                 noise_std, std)
        self.activation, act_fn = resolve_activation(activation)
        self.glu = make_glu(act_fn, fused)
        self.kernel = kernel
        # how the kernel path sums a token's per-pair rows: None = the library default
        # (moe_kernel.get_combine_mode()), or "atomic" / "store" for this block
        self.combine_mode = None
        # a registered name bound to its registered function, and known to the epilogues
        named = ACTIVATIONS.get(self.activation) is act_fn and self.activation in KERNEL_ACTIVATIONS
        self._kernel_act = self.activation if named else None

        h = self.d_hidden
        self.W_in = nn.Parameter(torch.randn(n_experts, d_model, 2 * h) * std)    # [gate | up]
        self.W_out = nn.Parameter(torch.randn(n_experts, h, d_model) * std)
        self.b_in = nn.Parameter(torch.zeros(n_experts, 2 * h)) if bias else None
        self.b_out = nn.Parameter(torch.zeros(n_experts, d_model)) if bias else None
        self.W_sh_in = self.W_sh_out = self.b_sh_in = self.b_sh_out = None
        if n_shared:
            self.W_sh_in = nn.Parameter(torch.randn(n_shared, d_model, 2 * h) * std)
            self.W_sh_out = nn.Parameter(torch.randn(n_shared, h, d_model) * std)
            if bias:
                self.b_sh_in = nn.Parameter(torch.zeros(n_shared, 2 * h))
                self.b_sh_out = nn.Parameter(torch.zeros(n_shared, d_model))

        # refreshed by every forward
        self.aux_loss = torch.zeros(())
        self.expert_counts = torch.zeros(n_experts)
        self.dropped = torch.zeros((), dtype=torch.long)
        self.register_buffer("edges", torch.arange(n_experts + 1, dtype=torch.long),
                             persistent=False)

    # ------------------------------------------------------------------------------ gating
    def _kernel_config_ok(self) -> bool:
        """Everything about this block, other than the tensor it is handed, that the kernels need."""
        return (self.kernel and self._kernel_act is not None
                and MK.shapes_supported(self.d_model, self.d_hidden, self.n_experts, self.top_k,
                                        self.n_shared))

    def _kernel_ready(self) -> bool:
        return self._kernel_config_ok() and kernel_supported(self.W_in)

    @property
    def capacity_factor(self):
        """Effective capacity: the explicit setting, or for "auto" None where the kernels take
        this block's weights as they sit now and AUTO_CAPACITY elsewhere
        (src/model/moe.py:189-206)."""
        if self._capacity_setting != "auto":
            return self._capacity_setting
        return None if self._kernel_ready() else AUTO_CAPACITY

    def _use_kernel(self, x: torch.Tensor) -> bool:
        """The dropless kernel path (the gate of src/model/moe.py:331-343)."""
        return (self._kernel_config_ok() and self.capacity_factor is None
                and kernel_supported(x))

    def _kernels_take(self, x: torch.Tensor) -> bool:
        """Any kernel path: dropless, or an explicit capacity as a variant of the dispatch."""
        return self._kernel_config_ok() and kernel_supported(x)

    def _whole_block_ok(self, x: torch.Tensor) -> bool:
        """Can `forward` hand x to the single whole-block op? It has no bias operands and knows no
        capacity, so those cases take router + fused_moe_forward."""
        return self._use_kernel(x) and self.b_in is None and self.b_sh_in is None

    # ---------------------------------------------------------------------------- bookkeeping
    def _record(self, probs, counts, x):
        self.expert_counts = counts.detach()
        if probs is not None:
            self.aux_loss = self.router.balance_loss(probs, counts)
        else:
            self.aux_loss = torch.zeros((), device=x.device, dtype=x.dtype)

    def _plan(self, topk_idx: torch.Tensor):
        """(experts, order, token_idx, counts), all int64: the flat pair ids `order` sorted by
        expert with ties in ascending pair id, the expert and the token of each sorted pair, and
        the per-expert histogram -- the canonical permutation of src/model/moe.py:208-223, which
        the CUDA dispatch reproduces."""
        flat = topk_idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.zeros(self.n_experts, dtype=torch.long, device=flat.device)
        counts.scatter_add_(0, flat, torch.ones_like(flat))
        return flat[order], order, order // self.top_k, counts

    def _capacity(self, n_tokens: int) -> int:
        """Pairs an expert may keep: capacity_factor x the fair share of the n_tokens * top_k
        pairs, at least 1 and at most all of them (src/model/moe.py:225-231)."""
        pairs = n_tokens * self.top_k
        return min(max(math.ceil(self.capacity_factor * pairs / self.n_experts), 1), pairs)

    # ------------------------------------------------------------------------ torch paths
    def _mlp(self, x, w_in, b_in, w_out, b_out):
        """One GLU expert on the rows of x."""
        h = x @ w_in
        if b_in is not None:
            h = h + b_in
        gate, up = h.chunk(2, dim=-1)
        y = self.glu(gate, up) @ w_out
        return y if b_out is None else y + b_out

    def _shared(self, x):
        """Sum of the always-on experts on every token (src/model/moe.py:310-329)."""
        total = None
        for s in range(self.n_shared):
            y = self._mlp(x, self.W_sh_in[s], None if self.b_sh_in is None else self.b_sh_in[s],
                          self.W_sh_out[s], None if self.b_sh_out is None else self.b_sh_out[s])
            total = y if total is None else total + y
        return total

    def _torch_experts(self, x, topk_w, topk_idx, cap: int):
        """The routed experts in plain torch, for what the kernels decline (CPU tensors, fp32 /
        fp64, unnamed activations): expert by expert over the sorted pairs, each expert's rows
        gathered, run through its GLU MLP, scaled by the router weight and added to their tokens
        (the arithmetic of src/model/moe.py:285-308, 396-413). With a capacity only the first
        `cap` pairs of a run are visited; the rest are dropped (src/model/moe.py:233-283)."""
        _, order, token_idx, counts = self._plan(topk_idx)
        pair_w = topk_w.reshape(-1)[order]
        kept = counts.clamp(max=cap) if cap else counts
        if cap:
            self.dropped = (counts - kept).sum().detach()
        starts = (counts.cumsum(0) - counts).tolist()      # the one host sync of this path
        out = torch.zeros_like(x)
        for e, (lo, n) in enumerate(zip(starts, kept.tolist())):
            if n == 0:
                continue
            rows = token_idx[lo:lo + n]
            y = self._mlp(x[rows], self.W_in[e], None if self.b_in is None else self.b_in[e],
                          self.W_out[e], None if self.b_out is None else self.b_out[e])
            out.index_add_(0, rows, y * pair_w[lo:lo + n, None])
        return out, counts

    # ------------------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.d_model:
            raise ValueError(f"expected last dim {self.d_model}, got {tuple(x.shape)}.")
        shape = x.shape
        x = x.reshape(-1, self.d_model)
        if x.shape[0] == 0:
            return x.clone().view(shape)
        if self._whole_block_ok(x):
            # whole block as one op: router GEMM, top-k, dispatch, experts, combine, balance loss
            full = self.router.wants_probs()
            noise = None
            if self.training and self.router.noise_std:
                # exploration noise on the logits (src/model/router.py:76-77), drawn here so that
                # the op stays a pure function of its inputs
                noise = torch.randn(x.shape[0], self.n_experts, device=x.device,
                                    dtype=torch.float32) * self.router.noise_std
            out, aux, counts = fused_moe_block(
                x, self.router, self.W_in, self.W_out, self.W_sh_in, self.W_sh_out,
                self._kernel_act, full, combine=self.combine_mode, noise=noise)
            self.expert_counts = counts.detach()
            self.aux_loss = aux if full else torch.zeros((), device=x.device, dtype=x.dtype)
            return out.view(shape)

        topk_w, topk_idx, probs = self.router(x)
        cap = self._capacity(x.shape[0]) if self.capacity_factor is not None else 0

        if self._kernels_take(x):
            # biases or a capacity: the same kernels behind the router, the capacity as a variant of
            # the dispatch schedule
            out, counts = fused_moe_forward(
                x, self.W_in, self.W_out, topk_w, topk_idx, self.b_in, self.b_out,
                self._kernel_act, w_sh_in=self.W_sh_in, w_sh_out=self.W_sh_out,
                combine=self.combine_mode, b_sh_in=self.b_sh_in, b_sh_out=self.b_sh_out,
                capacity=cap)
            self._record(probs, counts, x)
            if cap:
                self.dropped = (counts - cap).clamp(min=0).sum().detach().long()
            return out.view(shape)

        out, counts = self._torch_experts(x, topk_w, topk_idx, cap)
        self._record(probs, counts, x)
        if self.n_shared:
            out = out + self._shared(x)
        return out.view(shape)

    def dense_forward(self, x: torch.Tensor) -> torch.Tensor:
        """Every expert on every token, mixed by a dense [N, E] gate matrix that is zero off the
        selected (and, under a capacity, kept) pairs: the shape-static cross-check of `forward`
        (src/model/moe.py:420-474). Same side effects as `forward`."""
        if x.shape[-1] != self.d_model:
            raise ValueError(f"expected last dim {self.d_model}, got {tuple(x.shape)}.")
        shape = x.shape
        x = x.reshape(-1, self.d_model)
        topk_w, topk_idx, probs = self.router(x)
        experts, order, _, counts = self._plan(topk_idx)
        self._record(probs, counts, x)
        if self.capacity_factor is not None and x.shape[0]:
            cap = self._capacity(x.shape[0])
            pos = torch.arange(order.numel(), device=x.device) - (counts.cumsum(0) - counts)[experts]
            kept = torch.zeros_like(order, dtype=torch.bool).scatter_(0, order, pos < cap)
            self.dropped = (~kept).sum().detach()
            topk_w = topk_w * kept.view_as(topk_w)
        gates = torch.zeros(x.shape[0], self.n_experts, dtype=x.dtype, device=x.device)
        gates.scatter_(1, topk_idx, topk_w)
        out = torch.zeros_like(x)
        for e in range(self.n_experts):
            y = self._mlp(x, self.W_in[e], None if self.b_in is None else self.b_in[e],
                          self.W_out[e], None if self.b_out is None else self.b_out[e])
            out = out + gates[:, e:e + 1] * y
        if self.n_shared:
            out = out + self._shared(x)
        return out.view(shape)
