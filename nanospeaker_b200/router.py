"""Token-choice softmax top-k router with the selection running as a CUDA kernel.

Same constructor, attributes and return contract as TopKRouter in src/model/router.py:8-111.
On CUDA the softmax / top-k / renormalise step is the `moe_b200::router_topk` op (one warp per
token); elsewhere the same arithmetic runs through torch ops so the module stays usable on CPU.
"""
import torch
import torch.nn.functional as F
from torch import nn

from . import moe_kernel as MK


class TopKRouter(nn.Module):
    """x [N, d_model] -> (topk_w [N, k] in x.dtype, topk_idx [N, k] int64, probs [N, E] fp32 | None).

    `probs` is returned only while training with a non-zero balance-loss weight, as in
    src/model/router.py:52-54, 79-98. `noise_std` may be reassigned between steps.

    CUDA selection rule: descending logit, ties to the lowest expert index. torch.topk leaves tie
    order unspecified, so on rows with exactly tied logits the two may pick different (equally
    valid) experts; on rows without ties they agree bit for bit.
    """

    def __init__(self, d_model: int, n_experts: int, top_k: int = 2,
                 normalize_weights: bool = True, aux_loss_coef: float = 1e-2,
                 noise_std: float = 0.0, std: float = 0.02):
        super().__init__()
        if min(d_model, n_experts, top_k) < 1:
            raise ValueError(
                f"d_model ({d_model}), n_experts ({n_experts}) and top_k ({top_k}) "
                f"must all be >= 1."
            )
        if top_k > n_experts:
            raise ValueError(f"top_k ({top_k}) cannot exceed n_experts ({n_experts}).")
        self.n_experts = n_experts
        self.top_k = top_k
        self.normalize_weights = normalize_weights
        self.aux_loss_coef = aux_loss_coef
        self.noise_std = noise_std
        self.W = nn.Parameter(torch.randn(d_model, n_experts) * std)
        # Optional additive per-expert logit bias [n_experts] (fp32, not a parameter, not saved):
        # None in the reference's configuration; benchmarks set it to skew the expert load.
        self.logit_bias = None

    def wants_probs(self) -> bool:
        return self.training and self.aux_loss_coef != 0.0

    def _kernel_ok(self, logits: torch.Tensor) -> bool:
        return (logits.is_cuda and self.n_experts <= MK.MAX_EXPERTS
                and self.top_k <= MK.MAX_TOPK)

    def forward(self, x: torch.Tensor):
        # matmul in x's dtype, selection in fp32 (src/model/router.py:65-69)
        logits = (x @ self.W.to(x.dtype)).float()
        if self.logit_bias is not None:
            logits = logits + self.logit_bias
        if self.training and self.noise_std:
            logits = logits + torch.randn_like(logits) * self.noise_std
        full = self.wants_probs()

        if self._kernel_ok(logits):
            w, idx, probs = MK.router_topk(logits, self.top_k, self.normalize_weights, full)
            return w.to(x.dtype), idx, (probs if full else None)

        # same arithmetic in torch (CPU, or more experts than the kernel keeps on chip)
        if full:
            probs = F.softmax(logits, dim=-1)
            w, idx = probs.topk(self.top_k, dim=-1)
            if self.normalize_weights and self.top_k > 1:
                w = w / w.sum(dim=-1, keepdim=True)
        else:
            probs = None
            top_logits, idx = logits.topk(self.top_k, dim=-1)
            if self.normalize_weights:
                w = F.softmax(top_logits, dim=-1)
            else:
                w = F.softmax(logits, dim=-1).gather(1, idx)
        return w.to(x.dtype), idx, probs

    def balance_loss(self, probs: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """coef * E * sum_e f_e * mean_t probs[t, e], f = share of assignments
        (src/model/router.py:100-111); the gradient flows through probs only."""
        share = counts.float() / counts.sum().clamp(min=1)
        return self.aux_loss_coef * self.n_experts * (share * probs.mean(0)).sum()
