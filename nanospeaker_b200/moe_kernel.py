"""Differentiable torch.library ops over the sm_100a MoE kernels, and the three names the MoE module
imports from its kernel module: KERNEL_ACTIVATIONS, fused_moe_forward, kernel_supported
(the interface of src/model/moe_kernel.py:71-108, 785-803).

Ops (namespace `moe_b200`, all functional, all with fake kernels so torch.compile traces them):

  router_topk      fp32 logits -> (topk_w, topk_idx, probs)          src/model/router.py:79-97
  moe_dispatch     topk_idx -> six int32 plan tensors                src/model/moe_kernel.py:180-218
  moe_experts      routed (+ shared) experts on dispatched pairs     src/model/moe_kernel.py:558-623
  moe_experts_bwd  its backward as one opaque op                     src/model/moe_kernel.py:626-749

No op synchronises the host: buffers are sized by the worst case `l_cap` and the live padded length
stays in a 1-element device tensor that the kernels read.
"""
from typing import List, Optional, Tuple

import torch

from . import kernels as K
from .kernels import ALIGN_M, KERNEL_ACTIVATIONS, l_cap as _l_cap  # noqa: F401  (re-exported)

# dtypes the tcgen05 path computes in (fp32 accumulation inside).
KERNEL_DTYPES = (torch.bfloat16,)

# How a token's k (+ S) per-pair rows are summed, in the forward (out) and in the backward (dx):
#   "atomic"  the down / dX GEMM adds every row straight into the token-major result (bf16 atomics
#             in L2): no per-pair [l_cap, D] buffer is written or read back and there is no combine
#             launch. The sum is taken in bf16 in arrival order, so results can differ in the last
#             bf16 bit from run to run (the reference's eager path also sums in bf16,
#             src/model/moe.py:407-413).
#   "store"   the GEMM stores per-pair rows and a combine kernel sums them in fp32 in pair order:
#             bitwise reproducible, what the reference's kernel path does
#             (src/model/moe_kernel.py:26-30, 579-582).
COMBINE_MODES = ("atomic", "store")
_combine_mode = "atomic"


def set_combine_mode(mode: str) -> None:
    """Library-wide default for how per-pair rows are summed ("atomic" or "store")."""
    global _combine_mode
    if mode not in COMBINE_MODES:
        raise ValueError(f"combine mode must be one of {COMBINE_MODES}, got {mode!r}")
    _combine_mode = mode


def get_combine_mode() -> str:
    return _combine_mode


def _atomic(mode: Optional[str]) -> bool:
    mode = _combine_mode if mode is None else mode
    if mode not in COMBINE_MODES:
        raise ValueError(f"combine mode must be one of {COMBINE_MODES}, got {mode!r}")
    return mode == "atomic"


# Balance loss over more than one rank's tokens. With tokens sharded over ranks every rank's own
# loss uses its shard's routing counts (what the reference computes per process); for the loss of the
# WHOLE batch the counts have to be summed over the ranks first. _aux_reduce, when set, is called
# inside the whole-block op on a copy of the routed experts' counts (int32 [E], in place, e.g.
# torch.distributed.all_reduce): the op then weighs its probability sums by the global counts, and
# fused_moe_block scales the result by T_local / T_global, so that every rank holds ITS SHARE of the
# global loss -- the shares sum to the global loss, and so do their gradients when the ranks'
# gradients are summed. nanospeaker_b200.parallel.enable_global_balance_loss sets it.
_aux_reduce = None


def set_aux_reduce(fn) -> None:
    """fn(counts int32 [E]) -> None reduces the counts over the ranks in place; None switches the
    global balance loss off."""
    global _aux_reduce
    _aux_reduce = fn


MAX_EXPERTS = 256  # per-expert state of the routing kernels lives on chip
MAX_TOPK = 16
MAX_SHARED = 8     # shared experts are dispatched as extra experts: E + S <= MAX_EXPERTS


def kernel_supported(t: torch.Tensor) -> bool:
    """Device + dtype half of the gate (src/model/moe_kernel.py:81-90): CUDA and bf16."""
    return t.is_cuda and t.dtype in KERNEL_DTYPES


def shapes_supported(d_model: int, d_hidden: int, n_experts: int, top_k: int,
                     n_shared: int = 0) -> bool:
    """Shape half of the gate: what the tile shapes of the sm_100a kernels cover."""
    return (d_hidden == 128 and d_model >= 64 and d_model % 32 == 0
            and 1 <= n_experts and 1 <= top_k <= min(MAX_TOPK - n_shared, n_experts)
            and 0 <= n_shared <= MAX_SHARED and n_experts + n_shared <= MAX_EXPERTS)


# ------------------------------------------------------------------------------ router top-k
@torch.library.custom_op("moe_b200::router_topk", mutates_args=())
def router_topk(logits: torch.Tensor, top_k: int, normalize: bool,
                full_softmax: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(topk_w fp32 [T,k], topk_idx int64 [T,k], probs fp32 [T,E] or empty when not full_softmax).

    Winners by descending logit, ties to the lowest expert index.
    """
    w, idx, probs = K.router_topk(logits.float(), top_k, normalize, full_softmax, full_softmax)
    return w, idx, probs if probs is not None else logits.new_empty(0, dtype=torch.float32)


@router_topk.register_fake
def _(logits, top_k, normalize, full_softmax):
    t, e = logits.shape
    return (logits.new_empty((t, top_k), dtype=torch.float32),
            logits.new_empty((t, top_k), dtype=torch.int64),
            logits.new_empty((t, e) if full_softmax else (0,), dtype=torch.float32))


@torch.library.custom_op("moe_b200::router_topk_bwd", mutates_args=())
def router_topk_bwd(logits: torch.Tensor, topk_idx: torch.Tensor, d_topk_w: torch.Tensor,
                    d_probs: Optional[torch.Tensor], normalize: bool,
                    full_softmax: bool) -> torch.Tensor:
    return K.router_topk_bwd(logits.float(), topk_idx, d_topk_w, d_probs, normalize,
                             full_softmax).to(logits.dtype)


@router_topk_bwd.register_fake
def _(logits, topk_idx, d_topk_w, d_probs, normalize, full_softmax):
    return torch.empty_like(logits)


def _router_setup(ctx, inputs, output):
    logits, top_k, normalize, full_softmax = inputs
    ctx.save_for_backward(logits, output[1])
    ctx.normalize, ctx.full_softmax = normalize, full_softmax
    ctx.mark_non_differentiable(output[1])


def _router_backward(ctx, d_w, d_idx, d_probs):
    logits, idx = ctx.saved_tensors
    if d_w is None:
        d_w = torch.zeros(idx.shape, dtype=torch.float32, device=idx.device)
    if not ctx.full_softmax or d_probs is None or d_probs.numel() == 0:
        d_probs = None
    return router_topk_bwd(logits, idx, d_w, d_probs, ctx.normalize, ctx.full_softmax), None, None, None


router_topk.register_autograd(_router_backward, setup_context=_router_setup)


# ---------------------------------------------------------------------------------- dispatch
@torch.library.custom_op("moe_b200::moe_dispatch", mutates_args=())
def moe_dispatch(topk_idx: torch.Tensor, n_experts: int, capacity: int = 0,
                 n_capped: int = -1) -> Tuple[
    torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor
]:
    """(sorted_ids [l_cap], expert_ids [l_cap/128], pad_offsets [E+1], counts [E], n_post_pad [1],
    inv_ids [M]) as int32 -- the tuple of src/model/moe_kernel.py:180-209, with one stronger
    guarantee: inside a run, pairs are in ascending pair id (a stable sort by expert).

    capacity > 0 turns the plan into the fixed-capacity schedule (src/model/moe.py:225-283): the
    experts below n_capped (default: all) keep the first `capacity` pairs of their runs, the other
    pairs get no slot (inv_ids = -1); counts still holds the routing decisions."""
    return K.dispatch(topk_idx, n_experts, capacity, n_capped)


@moe_dispatch.register_fake
def _(topk_idx, n_experts, capacity=0, n_capped=-1):
    m = topk_idx.numel()
    cap = _l_cap(m, n_experts)
    mk = lambda n: topk_idx.new_empty((n,), dtype=torch.int32)
    return mk(cap), mk(cap // ALIGN_M), mk(n_experts + 1), mk(n_experts), mk(1), mk(m)


# ----------------------------------------------------------------------------------- experts
def _act_id(activation: str) -> int:
    if activation not in KERNEL_ACTIVATIONS:
        raise ValueError(
            f"activation {activation!r} has no kernel; use one of "
            f"{sorted(set(KERNEL_ACTIVATIONS))} or fall back to the eager path."
        )
    return KERNEL_ACTIVATIONS[activation]


def _check_inputs(x, w_in, w_out, w_sh_in):
    if not kernel_supported(x):
        raise RuntimeError(
            f"moe_b200 kernels need CUDA bf16 tensors, got {x.device} {x.dtype}; there is no "
            "CPU or other-dtype implementation behind these ops")
    n_shared = 0 if w_sh_in is None else w_sh_in.shape[0]
    if not shapes_supported(x.shape[1], w_in.shape[2] // 2, w_in.shape[0], 1, n_shared):
        raise RuntimeError(
            f"moe_b200 kernels do not cover d_model={x.shape[1]}, d_hidden={w_in.shape[2] // 2}, "
            f"n_experts={w_in.shape[0]}, n_shared={n_shared}")


def _down_combine_atomic(hid, w_out, w_sh_out, expert_ids, n_post_pad, pad_offsets, sorted_ids, tw,
                         m, topk, x, b_out, out):
    """The down GEMM with the atomic combine. `out` given (a residual, or zeros when there are
    biases): every row, shared experts included, is added to it. Otherwise the shared experts'
    rows -- token-ordered, weight 1 -- are summed by one plain-store GEMM that gives the accumulator
    its initial value (no fill pass, a quarter fewer atomic adds at S = 2, k = 6), and only the
    routed experts' rows are added."""
    if out is None and w_sh_out is not None and b_out is None:
        e_n = w_out.shape[0]
        out = K.down_gemm_sum(hid, w_sh_out, pad_offsets[e_n:], x.shape[0])
        return K.down_gemm_acc(hid, w_out, expert_ids, pad_offsets[e_n:e_n + 1], 0, sorted_ids, tw,
                               m, topk, out)
    if out is None:
        out = torch.zeros_like(x)
    return K.down_gemm_acc(hid, w_out, expert_ids, n_post_pad, 0, sorted_ids, tw, m, topk, out,
                           w_extra=w_sh_out, bias=b_out)


def _dx_first_value(da1, w_sh_in, pad_offsets, e_n, x):
    """dX's accumulator with its first value: the shared experts' share by one plain-store GEMM
    (see _down_combine_atomic), zeros without shared experts."""
    if w_sh_in is not None:
        return K.dx_gemm_sum(da1, w_sh_in, pad_offsets[e_n:], x.shape[0])
    return torch.zeros_like(x)


def _dx_add_routed(da1, w_in, shared_done, expert_ids, n_post_pad, pad_offsets, sorted_ids, m, topk,
                   dx):
    """The routed experts' rows of dX added to dx (atomic combine in the GEMM's epilogue)."""
    e_n = w_in.shape[0]
    if shared_done:   # the tile list ends where the first shared run starts
        return K.dx_gemm_acc(da1, w_in, expert_ids, pad_offsets[e_n:e_n + 1], 0, sorted_ids, m,
                             topk, dx, pad_offsets=pad_offsets[:e_n + 1])
    return K.dx_gemm_acc(da1, w_in, expert_ids, n_post_pad, 0, sorted_ids, m, topk, dx,
                         pad_offsets=pad_offsets)


def _dx_combine_atomic(da1, w_in, w_sh_in, expert_ids, n_post_pad, pad_offsets, sorted_ids, m,
                       topk, x):
    """dX with the atomic combine: first value, then the routed rows."""
    dx = _dx_first_value(da1, w_sh_in, pad_offsets, w_in.shape[0], x)
    return _dx_add_routed(da1, w_in, w_sh_in is not None, expert_ids, n_post_pad, pad_offsets,
                          sorted_ids, m, topk, dx)


@torch.library.custom_op("moe_b200::moe_experts", mutates_args=())
def moe_experts(
    x: torch.Tensor,
    w_in: torch.Tensor,
    w_out: torch.Tensor,
    topk_w: torch.Tensor,
    w_sh_in: Optional[torch.Tensor],
    w_sh_out: Optional[torch.Tensor],
    sorted_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    pad_offsets: torch.Tensor,
    counts: torch.Tensor,
    n_post_pad: torch.Tensor,
    inv_ids: torch.Tensor,
    activation: str,
    save_for_backward: bool,
    b_in: Optional[torch.Tensor] = None,
    b_out: Optional[torch.Tensor] = None,
    atomic_combine: bool = False,
    b_sh_in: Optional[torch.Tensor] = None,
    b_sh_out: Optional[torch.Tensor] = None,
    has_dropped: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """out[t] = sum_j topk_w[t,j] * expert_{idx[t,j]}(x[t]) on pre-dispatched pairs.

    Optional per-expert biases, b_in [E, 2H] / b_out [E, D] of the routed experts and b_sh_in
    [S, 2H] / b_sh_out [S, D] of the shared ones, are added in the GEMM epilogues (before the GLU /
    before the weight scale, src/model/moe.py:295-305, 317-326). has_dropped: the plan was built
    with a capacity, so some pairs may have no slot (their d topk_w is then zero).

    up/gate GEMM with the GLU fused -> down GEMM with fused router weight -> token-major fp32
    combine. All tensors share x's dtype (the wrapper casts). Two ways to feed the up GEMM:
      * inference (save_for_backward False): its producer warps gather the token rows themselves,
        no permuted copy of x exists;
      * training: x is permuted once into slot order (xs) and kept, because the weight-gradient
        GEMM reads the same rows again and TMA tiles of a materialised buffer stream several times
        faster than per-row cp.async gathers.

    Shared experts: when w_sh_in / w_sh_out [S, ...] are given, the plan must have been built over
    E + S experts with every token also routed (weight 1) to experts E .. E+S-1; those ids read the
    shared weight stacks, so the always-on experts run inside the same launches as the routed ones
    (`fused_moe_forward` builds that plan).

    Returns (out, xs, a1). With save_for_backward the forward keeps xs [l_cap, D] and the up GEMM's
    pre-activations a1 [l_cap, 2H] so the backward neither re-permutes nor recomputes -- 180 GB of
    HBM make keeping ~250 MB per block the cheaper side of the trade the reference settles the
    other way on a 4 GB card (src/model/moe_kernel.py:663-664). Without it both are empty.
    """
    x, w_in, w_out = x.contiguous(), w_in.contiguous(), w_out.contiguous()
    _check_inputs(x, w_in, w_out, w_sh_in)
    act = _act_id(activation)
    n, d = x.shape
    topk = topk_w.shape[-1]
    m = n * topk
    if n == 0:
        return x.new_zeros((0, d)), x.new_empty(0), x.new_empty(0)
    tw = topk_w.reshape(-1).contiguous()
    if w_sh_in is not None:
        w_sh_in, w_sh_out = w_sh_in.contiguous(), w_sh_out.contiguous()
    b_in, b_out = _all_bias(b_in, b_sh_in, w_in, w_sh_in, 2), _all_bias(b_out, b_sh_out, w_out, w_sh_out, 2)
    if save_for_backward:
        live, tok = _routed_rows(x, w_in, w_sh_in, pad_offsets, n_post_pad)
        xs = K.permute(x, topk, sorted_ids, live)
        hid, a1 = K.up_gemm(xs, w_in, expert_ids, n_post_pad, 0, act, True, w_extra=w_sh_in,
                            token_rows=tok, bias=b_in, pad_offsets=pad_offsets)
    else:
        xs, a1 = x.new_empty(0), x.new_empty(0)
        hid, _ = K.up_gemm(x, w_in, expert_ids, n_post_pad, 0, act, False,
                           gather=(sorted_ids, topk), w_extra=w_sh_in, bias=b_in)
    if atomic_combine:
        out = _down_combine_atomic(hid, w_out, w_sh_out, expert_ids, n_post_pad, pad_offsets,
                                   sorted_ids, tw, m, topk, x, b_out, None)
    else:
        y = K.down_gemm(hid, w_out, expert_ids, n_post_pad, 0, sorted_ids, tw, m, w_extra=w_sh_out,
                        bias=b_out)
        out = K.combine(y, inv_ids, n, topk)
    return out, xs, a1


@moe_experts.register_fake
def _(x, w_in, w_out, topk_w, w_sh_in, w_sh_out, sorted_ids, expert_ids, pad_offsets, counts,
      n_post_pad, inv_ids, activation, save_for_backward, b_in=None, b_out=None,
      atomic_combine=False, b_sh_in=None, b_sh_out=None, has_dropped=False):
    n, d = x.shape
    if n == 0 or not save_for_backward:
        return x.new_empty((n, d)), x.new_empty(0), x.new_empty(0)
    cap = sorted_ids.shape[0]
    return x.new_empty(x.shape), x.new_empty((cap, d)), x.new_empty((cap, w_in.shape[2]))


def _all_bias(b, b_sh, w, w_sh, dim):
    """One bias row per group of both weight stacks ([E + S, width] in w's dtype), as the GEMM
    epilogues index them; None when neither stack has a bias."""
    if b is None and b_sh is None:
        return None
    e_n, s_n, width = w.shape[0], 0 if w_sh is None else w_sh.shape[0], w.shape[dim]
    rows = [b if b is not None else w.new_zeros((e_n, width))]
    if s_n:
        rows.append(b_sh if b_sh is not None else w.new_zeros((s_n, width)))
    return torch.cat([r.to(w.dtype) for r in rows], 0).contiguous()


def _routed_rows(src, w_in, w_sh_in, pad_offsets, n_post_pad):
    """How far the permute has to copy, and where the shared experts read their rows from.
    The shared experts visit every token once, in token order, and own the last runs of the slot
    order: their slot rows would be a plain copy of the token-major matrix `src`. So the permute
    stops at the start of the first shared run (a device scalar inside pad_offsets) and the GEMMs
    read those runs from `src` itself. Returns (live-row count tensor for the permute,
    token_rows argument for the GEMM wrappers)."""
    if w_sh_in is None:
        return n_post_pad, None
    e_n = w_in.shape[0]
    return pad_offsets[e_n:e_n + 1], (src, pad_offsets)


@torch.library.custom_op("moe_b200::moe_experts_bwd", mutates_args=())
def moe_experts_bwd(
    grad_out: torch.Tensor,
    x: torch.Tensor,
    xs: torch.Tensor,
    a1: torch.Tensor,
    w_in: torch.Tensor,
    w_out: torch.Tensor,
    topk_w: torch.Tensor,
    w_sh_in: Optional[torch.Tensor],
    w_sh_out: Optional[torch.Tensor],
    sorted_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    pad_offsets: torch.Tensor,
    counts: torch.Tensor,
    n_post_pad: torch.Tensor,
    inv_ids: torch.Tensor,
    activation: str,
    b_out: Optional[torch.Tensor] = None,
    need_db_in: bool = False,
    atomic_combine: bool = False,
    need_db_out: bool = False,
    has_dropped: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor]:
    """(dx, dW_in, dW_out, dtopk_w, dW_sh_in, dW_sh_out, db_in_all, db_out_all); the shared-expert
    and bias gradients are empty when the forward had none. The bias gradients cover the groups of
    both weight stacks ([E + S, width]: routed experts first). The kept pre-activations a1 already
    include b_in, so only b_out's value ([E, D], routed experts) enters the backward, through
    dtopk_w. xs (x in slot order) and a1 are what the forward kept; grad_out is permuted once and
    feeds both the dHidden GEMM and the dW_out GEMM. The bias gradients are segment sums over each
    expert's run (src/model/moe_kernel.py:723-737), here one column-sum kernel each."""
    grad_out = grad_out.to(x.dtype).contiguous()
    x, w_in, w_out = x.contiguous(), w_in.contiguous(), w_out.contiguous()
    _check_inputs(x, w_in, w_out, w_sh_in)
    act = _act_id(activation)
    n, d = x.shape
    e_n = w_in.shape[0]
    s_n = 0
    if w_sh_in is not None:
        w_sh_in, w_sh_out = w_sh_in.contiguous(), w_sh_out.contiguous()
        s_n = w_sh_in.shape[0]
    topk = topk_w.shape[-1]
    m = n * topk
    tw = topk_w.reshape(-1).contiguous()
    # pairs without a slot (dropped by a capacity) are never visited by the dHidden epilogue
    dtw_buf = torch.zeros(m, dtype=x.dtype, device=x.device) if has_dropped else None

    live, tok = _routed_rows(grad_out, w_in, w_sh_in, pad_offsets, n_post_pad)
    douts = K.permute(grad_out, topk, sorted_ids, live)
    da1, hidw, dtw = K.dhidden_glu_bwd(douts, w_out, expert_ids, n_post_pad, 0, sorted_ids, tw, m,
                                       a1, act, True, w_extra=w_sh_out, token_rows=tok,
                                       dtw_out=dtw_buf)
    if atomic_combine:
        dx = _dx_combine_atomic(da1, w_in, w_sh_in, expert_ids, n_post_pad, pad_offsets,
                                sorted_ids, m, topk, x)
    else:
        ydx = K.dx_gemm(da1, w_in, expert_ids, n_post_pad, 0, w_extra=w_sh_in)
        dx = K.combine(ydx, inv_ids, n, topk)
    g_in = K.wgrad(xs, da1, pad_offsets, e_n + s_n, n_extra=s_n,
                   token_rows=("a", x) if s_n else None)
    g_out = K.wgrad(hidw, douts, pad_offsets, e_n + s_n, n_extra=s_n,
                    token_rows=("b", grad_out) if s_n else None)
    if s_n:
        (dw_in, dw_sh_in), (dw_out, dw_sh_out) = g_in, g_out
    else:
        dw_in, dw_out, dw_sh_in, dw_sh_out = g_in, g_out, x.new_empty(0), x.new_empty(0)
    dtw = dtw.view_as(topk_w)
    db_in, db_out = x.new_empty(0), x.new_empty(0)
    if need_db_in:      # db_in[e] = column sums of dA1 over e's run
        db_in = K.segment_colsum(da1, expert_ids, n_post_pad, e_n + s_n).to(x.dtype)
    if need_db_out:     # db_out[e] = sum over e's pairs of w * dOut[t]
        db_out = K.segment_colsum(
            douts, expert_ids, n_post_pad, e_n + s_n, sorted_ids, tw, m,
            token_rows=(grad_out, pad_offsets, e_n) if s_n else None).to(x.dtype)
    if b_out is not None:
        # y_pair = (hid W_out + b_out[e]) * w: dtopk_w gains <dOut[t], b_out[e]>. One row GEMM
        # dOut @ b_out^T -> [T, E (padded)], then each pair picks its expert's column.
        ld = _router_ld(e_n)
        bt = K.copy_cols(b_out.to(x.dtype).t().contiguous(), ld).unsqueeze(0)      # [1, D, ld]
        gb = K.down_gemm(grad_out, bt, None, None, 1, None, None, 0)[0]             # [T, ld]
        slot = inv_ids.long().view(n, topk)
        e_of_pair = expert_ids.long()[slot.clamp(min=0) // ALIGN_M]
        routed = (e_of_pair < e_n) & (slot >= 0)       # shared experts' d topk_w is not used
        pick = gb.gather(1, e_of_pair.clamp(max=e_n - 1)).float()
        dtw = (dtw.float() + torch.where(routed, pick, torch.zeros((), device=x.device))) \
            .to(topk_w.dtype)
    return dx, dw_in, dw_out, dtw, dw_sh_in, dw_sh_out, db_in, db_out


@moe_experts_bwd.register_fake
def _(grad_out, x, xs, a1, w_in, w_out, topk_w, w_sh_in, w_sh_out, sorted_ids, expert_ids,
      pad_offsets, counts, n_post_pad, inv_ids, activation, b_out=None, need_db_in=False,
      atomic_combine=False, need_db_out=False, has_dropped=False):
    g_n = w_in.shape[0] + (0 if w_sh_in is None else w_sh_in.shape[0])
    return (torch.empty_like(x), torch.empty_like(w_in), torch.empty_like(w_out),
            torch.empty_like(topk_w),
            torch.empty_like(w_sh_in) if w_sh_in is not None else x.new_empty(0),
            torch.empty_like(w_sh_out) if w_sh_out is not None else x.new_empty(0),
            x.new_empty((g_n, w_in.shape[2])) if need_db_in else x.new_empty(0),
            x.new_empty((g_n, x.shape[1])) if need_db_out else x.new_empty(0))


def _experts_setup(ctx, inputs, output):
    (x, w_in, w_out, topk_w, w_sh_in, w_sh_out, sorted_ids, expert_ids, pad_offsets, counts,
     n_post_pad, inv_ids, activation, save_for_backward, b_in, b_out, atomic_combine, b_sh_in,
     b_sh_out, has_dropped) = inputs
    out, xs, a1 = output
    ctx.atomic_combine, ctx.has_dropped = atomic_combine, has_dropped
    ctx.mark_non_differentiable(xs, a1)
    # without this autograd would hand the backward zero-filled gradients for the kept buffers
    ctx.set_materialize_grads(False)
    if not save_for_backward:
        raise RuntimeError("moe_experts was run with save_for_backward=False but a gradient is "
                           "being recorded; call it through fused_moe_forward")
    saved = [x, xs, a1, w_in, w_out, topk_w, sorted_ids, expert_ids, pad_offsets, counts,
             n_post_pad, inv_ids]
    ctx.has_shared = w_sh_in is not None
    if ctx.has_shared:
        saved += [w_sh_in, w_sh_out]
    # the values of b_in / b_sh_* are not needed again (a1 was kept with b_in inside, the shared
    # experts' router weight is a constant), b_out's is (for dtopk_w)
    ctx.has_b = (b_in is not None, b_out is not None, b_sh_in is not None, b_sh_out is not None)
    if b_out is not None:
        saved.append(b_out)
    ctx.save_for_backward(*saved)
    ctx.activation = activation


def _experts_backward(ctx, grad_out, g_xs, g_a1):
    (x, xs, a1, w_in, w_out, topk_w, sorted_ids, expert_ids, pad_offsets, counts, n_post_pad,
     inv_ids, *rest) = ctx.saved_tensors
    w_sh_in, w_sh_out = (rest[0], rest[1]) if ctx.has_shared else (None, None)
    has_b_in, has_b_out, has_b_sh_in, has_b_sh_out = ctx.has_b
    b_out = rest[-1] if has_b_out else None
    if grad_out is None:
        grad_out = torch.zeros_like(x)
    dx, dw_in, dw_out, dtw, dsi, dso, db_in, db_out = moe_experts_bwd(
        grad_out, x, xs, a1, w_in, w_out, topk_w, w_sh_in, w_sh_out, sorted_ids, expert_ids,
        pad_offsets, counts, n_post_pad, inv_ids, ctx.activation, b_out,
        has_b_in or has_b_sh_in, ctx.atomic_combine, has_b_out or has_b_sh_out, ctx.has_dropped)
    e_n = w_in.shape[0]
    return (dx, dw_in, dw_out, dtw, dsi if ctx.has_shared else None,
            dso if ctx.has_shared else None, None, None, None, None, None, None, None, None,
            db_in[:e_n] if has_b_in else None, db_out[:e_n] if has_b_out else None, None,
            db_in[e_n:] if has_b_sh_in else None, db_out[e_n:] if has_b_sh_out else None, None)


moe_experts.register_autograd(_experts_backward, setup_context=_experts_setup)


# ------------------------------------------------------------------------------- whole block
_T15 = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]
_T6 = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]


_SIDE_STREAMS = {}
# Debugging aid, off in normal use: True keeps every launch of the backward on the caller's stream.
_DEBUG_ONE_STREAM = False
# The whole-block op's common training form (atomic combine, no residual) is issued by ONE call into
# the library per direction (moe_b200_block_fwd / _bwd) instead of ~22 calls from Python; False
# keeps the stage-by-stage sequence below, which is the same launches.
_ONE_CALL = True


def _side_streams(device: torch.device):
    """Two extra streams per device for the independent branches of the block's backward. Work put
    on them is fenced on both sides by wait_stream, so callers (and CUDA-graph capture) only ever
    see the current stream."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = (torch.cuda.Stream(device=key), torch.cuda.Stream(device=key))
    return _SIDE_STREAMS[key]


def _router_ld(n_experts: int) -> int:
    """Column count the router logits are padded to: TMA tiles of the padded router weight are
    64 columns wide."""
    return (n_experts + 63) // 64 * 64


@torch.library.custom_op("moe_b200::moe_block", mutates_args=())
def moe_block(
    x: torch.Tensor,
    router_w: torch.Tensor,
    logit_bias: Optional[torch.Tensor],
    w_in: torch.Tensor,
    w_out: torch.Tensor,
    w_sh_in: Optional[torch.Tensor],
    w_sh_out: Optional[torch.Tensor],
    top_k: int,
    normalize: bool,
    full_softmax: bool,
    aux_coef: float,
    activation: str,
    save_for_backward: bool,
    residual: Optional[torch.Tensor] = None,
    atomic_combine: bool = False,
    noise: Optional[torch.Tensor] = None,
    global_aux: bool = False,
) -> _T15:
    """The whole MoE block as one op: router GEMM, top-k, dispatch, experts (routed + shared),
    combine and the balance loss, with no PyTorch glue kernels in between
    (MoEBlock.forward, src/model/moe.py:345-375, with TopKRouter.forward and balance_loss inlined).

    Returns [out, aux (fp32, 0-dim), counts (int32 [E]), then what the backward needs: xs, a1,
    logits, w_all, idx_all, sorted_ids, expert_ids, pad_offsets, counts_all, n_post_pad, inv_ids,
    router_w_padded]. The router GEMM runs on the same tcgen05 kernels as the experts against a
    copy of router_w zero-padded to a multiple of 64 columns, so the logits are [T, ld] bf16.
    noise: optional fp32 [T, E] added to the logits before the selection -- the exploration noise of
    a training step (src/model/router.py:76-77), drawn by the caller: the random stream stays
    outside the op, so a reentrant checkpoint replays it like any other input.
    """
    x, w_in, w_out = x.contiguous(), w_in.contiguous(), w_out.contiguous()
    _check_inputs(x, w_in, w_out, w_sh_in)
    act = _act_id(activation)
    n, d = x.shape
    e_n = w_in.shape[0]
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    if w_sh_in is not None:
        w_sh_in, w_sh_out = w_sh_in.contiguous(), w_sh_out.contiguous()
    ld = _router_ld(e_n)
    ks = top_k + s_n
    if (_ONE_CALL and atomic_combine and save_for_backward and residual is None
            and not (global_aux and _aux_reduce is not None)):
        # the common training form: the whole sequence below issued by one call into the library
        if noise is not None:
            noise = noise.to(torch.float32).contiguous()
        return K.block_fwd(x, router_w.contiguous(), logit_bias, noise, w_in, w_out, w_sh_in,
                           w_sh_out, top_k, normalize, full_softmax, aux_coef, act, ld)
    out = None
    if atomic_combine and residual is not None:   # the residual is the accumulator's initial value
        out = residual.contiguous().clone()

    wp = K.copy_cols(router_w, ld).unsqueeze(0)   # [1, D, ld], zero pad columns
    logits = K.down_gemm(x, wp, None, None, 1, None, None, 0)[0]
    if noise is not None:
        noise = noise.to(torch.float32).contiguous()
    w_all, idx_all, colsum, sids, eids, offs, counts_all, npp, inv = K.router_dispatch(
        logits, logit_bias, e_n, top_k, s_n, normalize, full_softmax, noise)
    tw = w_all.reshape(-1)
    m = n * ks
    if save_for_backward:
        live, tok = _routed_rows(x, w_in, w_sh_in, offs, npp)
        xs = K.permute(x, ks, sids, live)
        hid, a1 = K.up_gemm(xs, w_in, eids, npp, 0, act, True, w_extra=w_sh_in, token_rows=tok,
                            pad_offsets=offs)
    else:
        xs, a1 = x.new_empty(0), x.new_empty(0)
        hid, _ = K.up_gemm(x, w_in, eids, npp, 0, act, False, gather=(sids, ks), w_extra=w_sh_in)
    if atomic_combine:
        out = _down_combine_atomic(hid, w_out, w_sh_out, eids, npp, offs, sids, tw, m, ks, x, None,
                                   out)
    else:
        y = K.down_gemm(hid, w_out, eids, npp, 0, sids, tw, m, w_extra=w_sh_out)
        out = K.combine(y, inv, n, ks, residual)   # + residual [T, D] in the same fp32 sum when given
    counts = counts_all[:e_n].clone()
    if full_softmax:
        if global_aux and _aux_reduce is not None:
            # the loss (and, in the backward, its gradient) weighs the experts by the counts of all
            # ranks; the plan tensors keep the local ones
            counts_all = counts_all.clone()
            _aux_reduce(counts_all[:e_n])
        aux = K.balance_loss(colsum, counts_all, e_n, n, aux_coef)
    else:
        aux = torch.zeros((), dtype=torch.float32, device=x.device)
    return (out, aux, counts, xs, a1, logits, w_all, idx_all, sids, eids, offs,
            counts_all, npp, inv, wp)


@moe_block.register_fake
def _(x, router_w, logit_bias, w_in, w_out, w_sh_in, w_sh_out, top_k, normalize, full_softmax,
      aux_coef, activation, save_for_backward, residual=None, atomic_combine=False, noise=None,
      global_aux=False):
    n, d = x.shape
    e_n = w_in.shape[0]
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    ld, ks = _router_ld(e_n), top_k + s_n
    cap = _l_cap(n * ks, e_n + s_n)
    i32 = lambda *shape: x.new_empty(shape, dtype=torch.int32)
    kept = (x.new_empty((cap, d)), x.new_empty((cap, w_in.shape[2]))) if save_for_backward \
        else (x.new_empty(0), x.new_empty(0))
    return (x.new_empty(x.shape), x.new_empty((), dtype=torch.float32), i32(e_n), kept[0], kept[1],
            x.new_empty((n, ld)), x.new_empty((n, ks)), x.new_empty((n, ks), dtype=torch.int64),
            i32(cap), i32(cap // ALIGN_M), i32(e_n + s_n + 1), i32(e_n + s_n), i32(1), i32(n * ks),
            x.new_empty((1, d, ld)))


@torch.library.custom_op("moe_b200::moe_block_bwd", mutates_args=())
def moe_block_bwd(
    grad_out: torch.Tensor,
    grad_aux: Optional[torch.Tensor],
    x: torch.Tensor,
    logit_bias: Optional[torch.Tensor],
    w_in: torch.Tensor,
    w_out: torch.Tensor,
    w_sh_in: Optional[torch.Tensor],
    w_sh_out: Optional[torch.Tensor],
    xs: torch.Tensor,
    a1: torch.Tensor,
    logits: torch.Tensor,
    w_all: torch.Tensor,
    idx_all: torch.Tensor,
    sorted_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    pad_offsets: torch.Tensor,
    counts_all: torch.Tensor,
    n_post_pad: torch.Tensor,
    inv_ids: torch.Tensor,
    router_w_padded: torch.Tensor,
    top_k: int,
    normalize: bool,
    full_softmax: bool,
    aux_coef: float,
    activation: str,
    atomic_combine: bool = False,
    noise: Optional[torch.Tensor] = None,
) -> _T6:
    """[dx, d_router_w [D, E], dW_in, dW_out, dW_sh_in, dW_sh_out] of moe_block."""
    grad_out = grad_out.to(x.dtype).contiguous()
    dx = None
    act = _act_id(activation)
    n, d = x.shape
    e_n = w_in.shape[0]
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    ks = top_k + s_n
    m = n * ks
    tw = w_all.reshape(-1)
    if _ONE_CALL and atomic_combine:
        d_aux = None if grad_aux is None else grad_aux.to(torch.float32).reshape(1)
        side = None if _DEBUG_ONE_STREAM else _side_streams(x.device)
        dx, d_router, dw_in, dw_out, dw_sh_in, dw_sh_out = K.block_bwd(
            grad_out, d_aux, x, logit_bias, noise, w_in, w_out, w_sh_in, w_sh_out, xs, a1, logits,
            w_all, idx_all, sorted_ids, expert_ids, pad_offsets, counts_all, n_post_pad,
            router_w_padded, top_k, normalize, full_softmax, aux_coef, act, side)
        if not s_n:
            dw_sh_in, dw_sh_out = x.new_empty(0), x.new_empty(0)
        return dx, d_router, dw_in, dw_out, dw_sh_in, dw_sh_out

    live, tok = _routed_rows(grad_out, w_in, w_sh_in, pad_offsets, n_post_pad)
    douts = K.permute(grad_out, ks, sorted_ids, live)
    da1, hidw, dtw = K.dhidden_glu_bwd(douts, w_out, expert_ids, n_post_pad, 0, sorted_ids, tw, m,
                                       a1, act, True, w_extra=w_sh_out, token_rows=tok)
    # Everything below only depends on the two launches above and meets again in the combine. Three
    # branches on three streams: the small router kernels hide behind the expert GEMMs, and the
    # tail of one persistent GEMM (SMs that ran out of tiles) is filled by the next one's CTAs.
    main = torch.cuda.current_stream(x.device)
    side_out, side_router = _side_streams(x.device)
    if _DEBUG_ONE_STREAM:
        side_out = side_router = main
    side_out.wait_stream(main)
    side_router.wait_stream(main)
    if atomic_combine:
        # dx gets its first value by plain stores (the shared experts' share, or zeros); the
        # router's share on the third stream is added once that has happened
        dx = _dx_first_value(da1, w_sh_in, pad_offsets, e_n, x)
        dx_ready = torch.cuda.Event()
        dx_ready.record(main)
    g_in = K.wgrad(xs, da1, pad_offsets, e_n + s_n, n_extra=s_n,
                   token_rows=("a", x) if s_n else None)
    if atomic_combine:
        _dx_add_routed(da1, w_in, w_sh_in is not None, expert_ids, n_post_pad, pad_offsets,
                       sorted_ids, m, ks, dx)
    else:
        ydx = K.dx_gemm(da1, w_in, expert_ids, n_post_pad, 0, w_extra=w_sh_in)
    with torch.cuda.stream(side_out):
        g_out = K.wgrad(hidw, douts, pad_offsets, e_n + s_n, n_extra=s_n,
                        token_rows=("b", grad_out) if s_n else None)
    with torch.cuda.stream(side_router):
        # router: d(logits) from d(topk_w) and the balance loss, then the two router GEMMs
        d_aux = None if grad_aux is None else grad_aux.to(torch.float32).reshape(1)
        dl = K.router_fused_bwd(logits, logit_bias, idx_all, dtw.view(n, ks), e_n, top_k, s_n,
                                normalize, full_softmax, d_aux, counts_all, aux_coef,
                                logits.shape[1], noise)
        d_router = K.copy_cols(K.wgrad(x, dl, None, 1)[0], e_n)   # pad columns dropped
        if atomic_combine:   # the router's share of dx joins the same accumulator
            side_router.wait_event(dx_ready)
            K.dx_gemm_acc(dl.unsqueeze(0), router_w_padded, None, None, 1, None, 0, 1, dx)
        else:
            dx_router = K.dx_gemm(dl, router_w_padded, None, None, 1)[0]
    main.wait_stream(side_out)
    main.wait_stream(side_router)
    if s_n:
        (dw_in, dw_sh_in), (dw_out, dw_sh_out) = g_in, g_out
    else:
        dw_in, dw_out, dw_sh_in, dw_sh_out = g_in, g_out, x.new_empty(0), x.new_empty(0)
    if not atomic_combine:
        dx = K.combine(ydx, inv_ids, n, ks, dx_router)
    return dx, d_router, dw_in, dw_out, dw_sh_in, dw_sh_out


@moe_block_bwd.register_fake
def _(grad_out, grad_aux, x, logit_bias, w_in, w_out, w_sh_in, w_sh_out, xs, a1, logits, w_all,
      idx_all, sorted_ids, expert_ids, pad_offsets, counts_all, n_post_pad, inv_ids,
      router_w_padded, top_k, normalize, full_softmax, aux_coef, activation,
      atomic_combine=False, noise=None):
    return (torch.empty_like(x), x.new_empty((x.shape[1], w_in.shape[0])), torch.empty_like(w_in),
            torch.empty_like(w_out),
            torch.empty_like(w_sh_in) if w_sh_in is not None else x.new_empty(0),
            torch.empty_like(w_sh_out) if w_sh_out is not None else x.new_empty(0))


def _block_setup(ctx, inputs, output):
    (x, router_w, logit_bias, w_in, w_out, w_sh_in, w_sh_out, top_k, normalize, full_softmax,
     aux_coef, activation, save_for_backward, residual, atomic_combine, noise, global_aux) = inputs
    ctx.has_residual = residual is not None
    ctx.has_noise = noise is not None
    ctx.atomic_combine = atomic_combine
    ctx.mark_non_differentiable(*output[2:])
    ctx.set_materialize_grads(False)
    if not save_for_backward:
        raise RuntimeError("moe_block was run with save_for_backward=False but a gradient is "
                           "being recorded")
    ctx.has_shared = w_sh_in is not None
    ctx.has_bias = logit_bias is not None
    saved = [x, w_in, w_out] + list(output[3:])
    if ctx.has_shared:
        saved += [w_sh_in, w_sh_out]
    if ctx.has_bias:
        saved.append(logit_bias)
    if ctx.has_noise:
        saved.append(noise)
    ctx.save_for_backward(*saved)
    ctx.n_experts = w_in.shape[0]
    ctx.router_dtype = router_w.dtype
    ctx.args = (top_k, normalize, full_softmax, aux_coef, activation)


def _block_backward(ctx, grad_out, grad_aux, *unused):
    saved = list(ctx.saved_tensors)
    x, w_in, w_out = saved[:3]
    kept = saved[3:15]
    rest = saved[15:]
    w_sh_in, w_sh_out = (rest[0], rest[1]) if ctx.has_shared else (None, None)
    noise = rest.pop() if ctx.has_noise else None
    bias = rest[-1] if ctx.has_bias else None
    if grad_out is None:
        grad_out = torch.zeros_like(x)
    dx, d_router, dw_in, dw_out, dsi, dso = moe_block_bwd(
        grad_out, grad_aux, x, bias, w_in, w_out, w_sh_in, w_sh_out, *kept, *ctx.args,
        ctx.atomic_combine, noise)
    d_router = d_router.to(ctx.router_dtype)
    return (dx, d_router, None, dw_in, dw_out, dsi if ctx.has_shared else None,
            dso if ctx.has_shared else None, None, None, None, None, None, None,
            grad_out if ctx.has_residual else None, None, None, None)


moe_block.register_autograd(_block_backward, setup_context=_block_setup)


class _BlockFn(torch.autograd.Function):
    """The same forward / backward as the registered op `moe_b200::moe_block`, as a plain autograd
    node. Eager training calls go through this: a Python-registered torch.library op costs the
    host ~100 us per call in dispatcher and schema work (twice per step), which at T = 16384 is a
    quarter of what the GPU needs for the whole step. The registered ops remain what
    torch.compile, fake tensors and opcheck see."""

    @staticmethod
    def forward(ctx, *inputs):
        output = moe_block._init_fn(*inputs)
        _block_setup(ctx, inputs, output)
        return output

    @staticmethod
    def backward(ctx, grad_out, grad_aux, *unused):
        saved = list(ctx.saved_tensors)
        x, w_in, w_out = saved[:3]
        kept = saved[3:15]
        rest = saved[15:]
        w_sh_in, w_sh_out = (rest[0], rest[1]) if ctx.has_shared else (None, None)
        noise = rest.pop() if ctx.has_noise else None
        bias = rest[-1] if ctx.has_bias else None
        if grad_out is None:
            grad_out = torch.zeros_like(x)
        dx, d_router, dw_in, dw_out, dsi, dso = moe_block_bwd._init_fn(
            grad_out, grad_aux, x, bias, w_in, w_out, w_sh_in, w_sh_out, *kept, *ctx.args,
            ctx.atomic_combine, noise)
        d_router = d_router.to(ctx.router_dtype)
        return (dx, d_router, None, dw_in, dw_out, dsi if ctx.has_shared else None,
                dso if ctx.has_shared else None, None, None, None, None, None, None,
                grad_out if ctx.has_residual else None, None, None, None)


def _call_block(*args):
    """moe_block through the light autograd node when a gradient is being recorded in plain eager
    mode, through the registered op otherwise (no grad, tracing, compiling)."""
    if args[12] and not torch.compiler.is_compiling():     # args[12] = save_for_backward
        return _BlockFn.apply(*args)
    return moe_block(*args)


def fused_moe_block(x, router, w_in, w_out, w_sh_in, w_sh_out, activation, full_softmax,
                    combine: Optional[str] = None, noise: Optional[torch.Tensor] = None):
    """(out, aux_loss fp32, counts int32 [E]) for a TopKRouter-like `router` (attributes W,
    logit_bias, top_k, normalize_weights, aux_loss_coef) -- the path MoEBlock.forward takes
    whenever no exploration noise has to be added to the logits."""
    _act_id(activation)
    cast = lambda t: None if t is None else t.to(x.dtype)
    tensors = (x, router.W, w_in, w_out, w_sh_in, w_sh_out)
    save = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)
    bias = router.logit_bias
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
    res = _call_block(x, cast(router.W), bias, cast(w_in), cast(w_out), cast(w_sh_in),
                      cast(w_sh_out), router.top_k, bool(router.normalize_weights),
                      bool(full_softmax), float(router.aux_loss_coef), activation, save, None,
                      _atomic(combine), noise, _aux_reduce is not None)
    aux = res[1]
    if full_softmax and _aux_reduce is not None:
        # this rank's share of the global loss: T_local / T_global, with T_global read off the
        # reduced counts (sum = T_global * top_k) on the device
        total = res[11][: w_in.shape[0]].sum().clamp(min=1).to(torch.float32)
        aux = aux * (float(x.shape[0] * router.top_k) / total)
    return res[0], aux, res[2]


def pad_router_weight(router_w: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """router.W [D, E] as the [1, D, ld] zero-padded operand of the logits GEMM (what moe_block
    builds on every call; an inference loop with fixed weights builds it once)."""
    return K.copy_cols(router_w.to(dtype).contiguous(), _router_ld(router_w.shape[1])).unsqueeze(0)


@torch.no_grad()
def moe_block_inference(x, router_w_padded, logit_bias, w_in, w_out, w_sh_in, w_sh_out,
                        n_experts: int, top_k: int, normalize: bool, activation: str,
                        residual: Optional[torch.Tensor] = None,
                        combine: Optional[str] = None) -> torch.Tensor:
    """Forward of the whole block for a caller that wants nothing but `out` (+ residual): the
    launches of moe_block's inference branch without its per-call extras (the padded copy of the
    router weight, the counts tensor, the zero balance loss). Logits GEMM, router top-k + dispatch
    (one launch up to 128 tokens, else two), up/gate GEMM on gathered rows, down GEMM, combine (the
    residual rides in its fp32 sum); issued by one call into the library (moe_b200_block_infer). x [T, D] bf16 contiguous; weights already in x.dtype."""
    act = _act_id(activation)
    n, _ = x.shape
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    ks = top_k + s_n
    if _ONE_CALL and n > 0:
        return K.block_infer(x, router_w_padded, logit_bias, w_in, w_out, w_sh_in, w_sh_out, top_k,
                             normalize, act, None if residual is None else residual.contiguous(),
                             _atomic(combine))
    logits = K.down_gemm(x, router_w_padded, None, None, 1, None, None, 0)[0]
    w_all, _, _, sids, eids, _, _, npp, inv = K.router_dispatch(
        logits, logit_bias, n_experts, top_k, s_n, normalize, False)
    hid, _ = K.up_gemm(x, w_in, eids, npp, 0, act, False, gather=(sids, ks), w_extra=w_sh_in)
    if _atomic(combine):
        out = torch.zeros_like(x) if residual is None else residual.clone()
        return K.down_gemm_acc(hid, w_out, eids, npp, 0, sids, w_all.reshape(-1), n * ks, ks, out,
                               w_extra=w_sh_out)
    y = K.down_gemm(hid, w_out, eids, npp, 0, sids, w_all.reshape(-1), n * ks, w_extra=w_sh_out)
    return K.combine(y, inv, n, ks, residual)


# ------------------------------------------------------------------------------- entry point
def fused_moe_forward(x, w_in, w_out, topk_w, topk_idx, b_in, b_out, activation,
                      w_sh_in=None, w_sh_out=None, combine: Optional[str] = None,
                      b_sh_in=None, b_sh_out=None, capacity: int = 0):
    """Dispatch + experts on the GPU; returns (out [N, d_model], counts [n_experts] int32).

    Same contract as src/model/moe_kernel.py:785-803, plus optional stacked shared-expert weights
    (`w_sh_in [S, D, 2H]`, `w_sh_out [S, H, D]`, biases `b_sh_in [S, 2H]`, `b_sh_out [S, D]`) whose
    outputs are then included in `out`, and an optional per-expert `capacity` (> 0: every routed
    expert keeps the first `capacity` pairs of its run, the padded path's rule,
    src/model/moe.py:225-283; counts still reports the routing decisions).
    Parameters are cast to x.dtype here (what autocast would do); gradients flow back through
    the cast. Per-expert biases b_in [E, 2H] / b_out [E, D] (either may be None) are applied in
    the GEMM epilogues and get gradients.
    """
    _act_id(activation)
    n_experts = w_in.shape[0]
    topk_w = topk_w.to(x.dtype)
    if w_sh_in is not None:
        # the shared experts become experts E .. E+S-1 that every token is routed to with weight 1
        s_n, t = w_sh_in.shape[0], topk_idx.shape[0]
        ids = torch.arange(n_experts, n_experts + s_n, device=topk_idx.device, dtype=topk_idx.dtype)
        topk_idx = torch.cat([topk_idx, ids.expand(t, s_n)], dim=1)
        topk_w = torch.cat([topk_w, topk_w.new_ones((t, s_n))], dim=1)
        n_experts += s_n
    sids, eids, offs, counts, npp, inv = moe_dispatch(topk_idx, n_experts, int(capacity),
                                                      w_in.shape[0])
    cast = lambda t: None if t is None else t.to(x.dtype)
    tensors = (x, w_in, w_out, topk_w, w_sh_in, w_sh_out, b_in, b_out, b_sh_in, b_sh_out)
    save = torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)
    out, _, _ = moe_experts(x, cast(w_in), cast(w_out), topk_w, cast(w_sh_in), cast(w_sh_out), sids,
                            eids, offs, counts, npp, inv, activation, save, cast(b_in), cast(b_out),
                            _atomic(combine), cast(b_sh_in), cast(b_sh_out), capacity > 0)
    return out, counts[: w_in.shape[0]]
