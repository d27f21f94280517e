"""Muon's batched Newton-Schulz orthogonalisation on the stacked expert weights, and the optimizer
step around it (src/train/optim.py:27-105).

The MoE block's weight gradients arrive stacked -- dW_in [E, d_model, 2H], dW_out [E, H, d_model] --
exactly as the weight-gradient kernels leave them, and Muon's update of such a parameter is five
iterations of

    A = X X^T;   X <- a X + (b A + c A A) X            (src/train/optim.py:37-39)

on X = G / (|G|_F + eps), per expert, with the smaller dimension leading. Here every product of the
iteration is one launch of the block's own grouped tcgen05 GEMM kernels on their fixed schedule (one
group per expert), and the three element-wise steps (normalisation, b A + c A A, a X + ...) are the
`axpby` kernel, so an [E, 576, 256] stack is orthogonalised in 26 launches with no per-expert loop and
no transposed copy:

  * tall matrices (rows > cols: W_in, [576, 256]) are never transposed. With X = G^T the Gram matrix
    is A = G^T G, a contraction over G's rows, which is what the weight-gradient kernel computes
    (C[e] = a_e^T b_e); and X <- a X + B X reads G <- a G + G B (B is symmetric), a row GEMM.
  * wide matrices (W_out, [128, 576]) use A = X X^T with X itself as the K-major weight operand, and
    B X as a row GEMM against X as the MN-major one.

On anything the kernels decline (CPU tensors, shapes off the tile grid) the same arithmetic runs as
torch batched matmuls in bf16.
"""
from typing import Iterable

import torch

from . import kernels as K

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def _kernel_ok(g: torch.Tensor) -> bool:
    if not (g.is_cuda and g.dim() == 3 and g.dtype == torch.bfloat16):
        return False
    m, n = min(g.shape[-2:]), max(g.shape[-2:])
    # tile grid of the grouped GEMMs: the small side is a whole number of 128-row blocks, the
    # large side a multiple of 32 columns with at least one 64-column K block
    return m % 128 == 0 and m <= 256 and n % 32 == 0 and n >= 64 and g.shape[0] <= 256


def _ns_torch(g: torch.Tensor, steps: int, eps: float) -> torch.Tensor:
    a, b, c = NS_COEFFS
    x = g.bfloat16()
    tall = x.size(-2) > x.size(-1)
    if tall:
        x = x.mT
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + eps)
    for _ in range(steps):
        gram = x @ x.mT
        x = a * x + (b * gram + c * (gram @ gram)) @ x
    return x.mT if tall else x


@torch.no_grad()
def newton_schulz5(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate orthogonal factor of every matrix of the stack g [E, rows, cols] (or of one
    matrix [rows, cols]), bf16 in and out: zeropower_via_newtonschulz5 of src/train/optim.py:27-40."""
    single = g.dim() == 2
    if single:
        g = g.unsqueeze(0)
    x = g.bfloat16().contiguous()
    if not _kernel_ok(x):
        out = _ns_torch(x, steps, eps)
        return out[0] if single else out
    a, b, c = NS_COEFFS
    e_n, rows, cols = x.shape
    tall = rows > cols
    x = K.axpby(x, 1.0, sumsq=K.group_sumsq(x), eps=eps)          # X / (|X|_F + eps)
    for _ in range(steps):
        if tall:
            gram = K.wgrad(x, x, None, e_n, a_grouped=True, b_grouped=True)      # G^T G  [E, c, c]
        else:
            gram = K.dx_gemm(x, x, None, None, e_n)                              # X X^T  [E, r, r]
        gram2 = K.dx_gemm(gram, gram, None, None, e_n)                           # A A (A = A^T)
        poly = K.axpby(gram, b, gram2, c)                                        # b A + c A A
        if tall:
            upd = K.down_gemm(x, poly, None, None, e_n, None, None, 0)           # G B
        else:
            upd = K.down_gemm(poly, x, None, None, e_n, None, None, 0)           # B X
        x = K.axpby(x, a, upd, 1.0)                                              # a X + ...
    return x[0] if single else x


class Muon(torch.optim.Optimizer):
    """Nesterov momentum whose direction is replaced by its orthogonal factor
    (src/train/optim.py:43-105): momentum buffer in bf16, update scaled by sqrt(max(1, rows / cols)),
    decoupled weight decay, |dW| and |W| accumulated on the device for `update_norm_ratio`.
    Stacked [E, rows, cols] parameters are orthogonalised per expert in one batched call."""

    def __init__(self, params: Iterable, lr: float = 0.02, momentum: float = 0.95,
                 weight_decay: float = 0.1, ns_steps: int = 5):
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay,
                                      ns_steps=ns_steps))
        self._update_sq = 0.0
        self._param_sq = 0.0

    def load_state_dict(self, state_dict):
        # the base class casts state to the parameter's dtype: put the momentum back in bf16
        super().load_state_dict(state_dict)
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p, {})
                if "momentum" in st:
                    st["momentum"] = st["momentum"].bfloat16()

    def update_norm_ratio(self) -> float:
        """|dW| / |W| of the most recent step."""
        if not torch.is_tensor(self._update_sq):
            return 0.0
        return float((self._update_sq / self._param_sq.clamp(min=1e-12)).sqrt())

    @torch.no_grad()
    def step(self):
        self._update_sq = self._param_sq = 0.0
        for group in self.param_groups:
            lr, mom, wd = group["lr"], group["momentum"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if "momentum" not in state:
                    state["momentum"] = torch.zeros_like(p, dtype=torch.bfloat16)
                buf = state["momentum"]
                grad = p.grad.to(buf.dtype)
                buf.lerp_(grad, 1 - mom)
                update = newton_schulz5(grad.lerp(buf, mom), group["ns_steps"])
                scale = max(1.0, p.size(-2) / p.size(-1)) ** 0.5
                delta = update.to(p.dtype) * (-lr * scale)
                p.mul_(1 - lr * wd)
                p.add_(delta)
                self._update_sq = self._update_sq + delta.float().pow(2).sum()
                self._param_sq = self._param_sq + p.detach().float().pow(2).sum()
