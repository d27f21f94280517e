"""The FFN sublayer around the MoE block: `x + ffn(rmsnorm(x))` with the balance loss riding out
next to the activations, as the tail of Block.forward does (src/model/nanospeaker.py:165-169 with
RMSNorm from src/model/ln.py:24-38).

On the kernel path the sublayer is one autograd node over three pieces of this library: the RMSNorm
kernel, the whole-block op with the residual added inside its combine, and in the backward the
block's backward followed by the RMSNorm backward with the residual branch's gradient folded in.
Against norm -> block -> add as three separate steps this drops one full [T, D] round trip in each
direction (the residual add and its gradient). Anything the kernels decline (CPU tensors, fp32,
training noise on the logits, ...) runs the same arithmetic in plain torch through the block's own
fallbacks.
"""
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import kernels as K
from . import moe_kernel as MK
from .moe import MoEBlock


class _FFNSublayerFn(torch.autograd.Function):
    """out = x + block(rmsnorm(x) * gamma); aux = the block's balance loss."""

    @staticmethod
    def forward(ctx, x, gamma, eps, router_w, logit_bias, w_in, w_out, w_sh_in, w_sh_out, top_k,
                normalize, full_softmax, aux_coef, activation, atomic_combine):
        cast = lambda t: None if t is None else t.to(x.dtype)
        h, rstd = K.rmsnorm(x, cast(gamma).contiguous(), eps)
        res = MK.moe_block(h, cast(router_w), logit_bias, cast(w_in), cast(w_out), cast(w_sh_in),
                           cast(w_sh_out), top_k, normalize, full_softmax, aux_coef, activation,
                           True, x, atomic_combine)
        out, aux, counts = res[0], res[1], res[2]
        ctx.has_shared = w_sh_in is not None
        ctx.has_bias = logit_bias is not None
        saved = [x, gamma, rstd, h, router_w, w_in, w_out] + list(res[3:])
        if ctx.has_shared:
            saved += [w_sh_in, w_sh_out]
        if ctx.has_bias:
            saved.append(logit_bias)
        ctx.save_for_backward(*saved)
        ctx.args = (top_k, normalize, full_softmax, aux_coef, activation, atomic_combine)
        ctx.mark_non_differentiable(counts)
        ctx.set_materialize_grads(False)
        return out, aux, counts

    @staticmethod
    def backward(ctx, grad_out, grad_aux, _grad_counts):
        saved = list(ctx.saved_tensors)
        x, gamma, rstd, h, router_w, w_in, w_out = saved[:7]
        kept = saved[7:19]
        rest = saved[19:]
        w_sh_in, w_sh_out = (rest[0], rest[1]) if ctx.has_shared else (None, None)
        bias = rest[-1] if ctx.has_bias else None
        if grad_out is None:
            grad_out = torch.zeros_like(x)
        grad_out = grad_out.to(x.dtype).contiguous()
        cast = lambda t: None if t is None else t.to(x.dtype)
        dh, d_router, dw_in, dw_out, dsi, dso = MK.moe_block_bwd(
            grad_out, grad_aux, h, bias, cast(w_in), cast(w_out), cast(w_sh_in), cast(w_sh_out),
            *kept, *ctx.args)
        dx, dgamma = K.rmsnorm_bwd(dh, x, rstd, cast(gamma).contiguous(), add=grad_out)
        return (dx, dgamma.to(gamma.dtype), None, d_router.to(router_w.dtype), None,
                dw_in.to(w_in.dtype), dw_out.to(w_out.dtype),
                dsi.to(w_sh_in.dtype) if ctx.has_shared else None,
                dso.to(w_sh_out.dtype) if ctx.has_shared else None, None, None, None, None, None,
                None)


class MoEFFNSublayer(nn.Module):
    """`x + ffn(norm_ffn(x))`, returning (out, aux_loss) like the tail of the reference's
    Block.forward. `norm_gamma` is RMSNorm's scale (src/model/ln.py:29), `ffn` a MoEBlock."""

    def __init__(self, ffn: MoEBlock, epsilon: float = 1e-6):
        super().__init__()
        self.ffn = ffn
        self.epsilon = epsilon
        self.norm_gamma = nn.Parameter(torch.ones(ffn.d_model))

    def _fused_ok(self, x: torch.Tensor) -> bool:
        f = self.ffn
        # (the whole-block op has no bias operands; exploration noise goes through the block itself)
        return (f._whole_block_ok(x) and not (f.training and f.router.noise_std)
                and f.d_model % 8 == 0 and f.d_model <= 2048)

    def forward(self, x: torch.Tensor):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        f = self.ffn
        if x2.shape[0] > 0 and self._fused_ok(x2):
            full = f.router.wants_probs()
            bias = f.router.logit_bias
            if bias is not None:
                bias = bias.to(torch.float32).contiguous()
            out, aux, counts = _FFNSublayerFn.apply(
                x2.contiguous(), self.norm_gamma, self.epsilon, f.router.W, bias, f.W_in, f.W_out,
                f.W_sh_in, f.W_sh_out, f.router.top_k, bool(f.router.normalize_weights),
                bool(full), float(f.router.aux_loss_coef), f._kernel_act,
                MK._atomic(f.combine_mode))
            f.expert_counts = counts.detach()
            f.aux_loss = aux if full else torch.zeros((), device=x.device, dtype=x.dtype)
            return out.view(shape), f.aux_loss
        h = F.rms_norm(x, (shape[-1],), self.norm_gamma.to(x.dtype), self.epsilon)
        return x + f(h), f.aux_loss
