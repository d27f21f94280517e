"""CPU oracle for the dropless MoE block -- TEST INFRASTRUCTURE, not product code.

A plain restatement, in torch CPU ops and numpy, of what nanoSpeaker's pure-PyTorch MoE path
computes (src/model/router.py, src/model/moe.py) plus closed-form backward formulas. It exists so
the CUDA kernels can be checked against the reference's arithmetic on a machine that has no copy of
the reference. Only tests/, __graft_entry__.smoke() and the CPU-baseline leg of bench.py import it.

Parity pinning: tests/test_oracle.py checks every function here (a) against golden vectors that
tests/golden/make_golden.py produced by running the unmodified reference modules, and (b), when a
checkout of the reference is present, against the reference imported live. One exception:
`ep_plan` at the end restates this repository's own multi-GPU layout rule (the reference is
single-GPU and has nothing to pin it to); its properties are checked in tests/test_expert_parallel.py.

Everything takes and returns CPU tensors. fp32 in -> the reference's fp32 path; bf16 in -> its
bf16 path (each op rounds to bf16 as eager PyTorch does).
"""
import math
from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

ALIGN_M = 128

ACTS = {
    "silu": F.silu, "swish": F.silu, "gelu": F.gelu, "relu": F.relu,
    "sigmoid": torch.sigmoid, "tanh": torch.tanh,
}


# ------------------------------------------------------------------------------------ router
def router_logits(x: torch.Tensor, w_router: torch.Tensor) -> torch.Tensor:
    """logits = (x @ W).float(): matmul in x's dtype, widened afterwards (src/model/router.py:69)."""
    return (x @ w_router).float()


def canonical_topk(logits: torch.Tensor, k: int) -> torch.Tensor:
    """The tie rule the CUDA router uses: descending value, ties to the lowest expert index.
    Equal to torch.topk wherever a row's top-(k+1) values are pairwise distinct."""
    return torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :k]


def tied_rows(logits: torch.Tensor, k: int) -> torch.Tensor:
    """Rows whose top-(k+1) values contain a duplicate (where torch.topk's pick is unspecified)."""
    kk = min(k + 1, logits.shape[-1])
    top = torch.sort(logits, dim=-1, descending=True).values[:, :kk]
    return (top[:, 1:] == top[:, :-1]).any(-1)


def router_select(logits: torch.Tensor, k: int, normalize: bool, full_softmax: bool,
                  idx: Optional[torch.Tensor] = None):
    """(topk_w fp32, topk_idx, probs | None) from fp32 logits.

    full_softmax=True is the training spelling (src/model/router.py:79-81, 96-97): softmax over
    all experts, top-k of the probabilities, renormalise when normalize and k > 1.
    full_softmax=False is the eval spelling (src/model/router.py:86-92): top-k of the logits, then
    a softmax over the winners (normalize) or a gather of the full softmax.
    `idx` forces the selection (e.g. the canonical one); by default torch.topk picks, as the
    reference does.
    """
    if full_softmax:
        probs = F.softmax(logits, dim=-1)
        if idx is None:
            w, idx = probs.topk(k, dim=-1)
        else:
            w = probs.gather(1, idx)
        if normalize and k > 1:
            w = w / w.sum(dim=-1, keepdim=True)
        return w, idx, probs
    if idx is None:
        top, idx = logits.topk(k, dim=-1)
    else:
        top = logits.gather(1, idx)
    w = F.softmax(top, dim=-1) if normalize else F.softmax(logits, dim=-1).gather(1, idx)
    return w, idx, None


def balance_loss(probs: torch.Tensor, counts: torch.Tensor, coef: float, n_experts: int):
    """coef * E * sum_e f_e * mean_t probs[t,e] (src/model/router.py:100-111)."""
    f = counts.float() / counts.sum().clamp(min=1)
    return coef * n_experts * (f * probs.mean(0)).sum()


def router_backward(logits, idx, d_w, d_probs, normalize: bool, full_softmax: bool):
    """d(logits) in closed form for router_select (fp32). d_probs may be None."""
    k = idx.shape[1]
    p = F.softmax(logits, dim=-1)
    if not full_softmax and normalize:
        w = F.softmax(logits.gather(1, idx), dim=-1)
        dl_sel = w * (d_w - (w * d_w).sum(-1, keepdim=True))
        return torch.zeros_like(logits).scatter_(1, idx, dl_sel)
    dp = torch.zeros_like(logits)
    if full_softmax and normalize and k > 1:
        ps = p.gather(1, idx)
        s = ps.sum(-1, keepdim=True)
        w = ps / s
        dp.scatter_(1, idx, (d_w - (d_w * w).sum(-1, keepdim=True)) / s)
    else:
        dp.scatter_(1, idx, d_w)
    if d_probs is not None:
        dp = dp + d_probs
    return p * (dp - (p * dp).sum(-1, keepdim=True))


# ------------------------------------------------------------------------------------- plan
def plan(topk_idx: torch.Tensor, n_experts: int):
    """(experts, order, token_idx, counts): stable sort of the flat expert ids
    (src/model/moe.py:208-223), in numpy."""
    k = topk_idx.shape[1]
    flat = topk_idx.reshape(-1).numpy()
    order = np.argsort(flat, kind="stable")
    experts = flat[order]
    counts = np.bincount(flat, minlength=n_experts)
    return (torch.from_numpy(experts), torch.from_numpy(order),
            torch.from_numpy(order // k), torch.from_numpy(counts))


def l_cap(n_pairs: int, n_experts: int) -> int:
    """Worst-case padded length (src/model/moe_kernel.py:100-108)."""
    return -(-(n_pairs + min(n_experts, n_pairs) * (ALIGN_M - 1)) // ALIGN_M) * ALIGN_M


def dispatch(topk_idx: torch.Tensor, n_experts: int):
    """The six int32 tensors of moe_dispatch (src/model/moe_kernel.py:180-209) with the run order
    fixed to the stable one: sorted_ids, expert_ids, pad_offsets, counts, n_post_pad, inv_ids."""
    m = topk_idx.numel()
    _, order, _, counts = plan(topk_idx, n_experts)
    order, counts = order.numpy(), counts.numpy()
    cap = l_cap(m, n_experts)
    padded = -(-counts // ALIGN_M) * ALIGN_M
    offs = np.concatenate([[0], np.cumsum(padded)]).astype(np.int32)
    sids = np.full(cap, m, dtype=np.int32)
    inv = np.empty(m, dtype=np.int32)
    eids = np.zeros(cap // ALIGN_M, dtype=np.int32)
    start = 0
    for e in range(n_experts):
        c = int(counts[e])
        run = order[start:start + c]
        sids[offs[e]:offs[e] + c] = run
        inv[run] = np.arange(offs[e], offs[e] + c)
        eids[offs[e] // ALIGN_M: offs[e + 1] // ALIGN_M] = e
        start += c
    t = torch.from_numpy
    return (t(sids), t(eids), t(offs), t(counts.astype(np.int32)),
            torch.tensor([int(offs[-1])], dtype=torch.int32), t(inv))


# ---------------------------------------------------------------------------------- experts
def shared_forward(x, w_sh_in, w_sh_out, act="silu", b_sh_in=None, b_sh_out=None):
    """Always-on experts, weight 1, summed, with their optional biases
    (src/model/moe.py:310-329)."""
    fn = ACTS[act]
    total = None
    for s in range(w_sh_in.shape[0]):
        h = x @ w_sh_in[s]
        if b_sh_in is not None:
            h = h + b_sh_in[s]
        gate, up = h.chunk(2, dim=-1)
        y = (fn(gate) * up) @ w_sh_out[s]
        if b_sh_out is not None:
            y = y + b_sh_out[s]
        total = y if total is None else total + y
    return total


def experts_forward(x, w_in, w_out, topk_w, topk_idx, act="silu", w_sh_in=None, w_sh_out=None,
                    b_in=None, b_out=None, b_sh_in=None, b_sh_out=None):
    """Eager ragged dispatch (src/model/moe.py:377-418): gather per expert, two matmuls with the GLU
    between, scale by the router weight, index_add_ into the output, then the shared experts.
    Optional per-expert biases b_in [E, 2H] / b_out [E, D] as in src/model/moe.py:295-305 (added
    after each matmul; b_out before the weight scale). Differentiable: the bias tests take its
    gradients from autograd."""
    fn = ACTS[act]
    n_experts, k = w_in.shape[0], topk_idx.shape[1]
    _, order, token_idx, counts = plan(topk_idx, n_experts)
    sizes = counts.tolist()
    xs = x.index_select(0, token_idx).split(sizes)
    ws = topk_w.reshape(-1).index_select(0, order).split(sizes)
    rows = token_idx.split(sizes)
    out = torch.zeros_like(x)
    for e in range(n_experts):
        if sizes[e] == 0:
            continue
        h = xs[e] @ w_in[e]
        if b_in is not None:
            h = h + b_in[e]
        gate, up = h.chunk(2, dim=-1)
        y = (fn(gate) * up) @ w_out[e]
        if b_out is not None:
            y = y + b_out[e]
        out = out.index_add(0, rows[e], y * ws[e][:, None])
    if w_sh_in is not None:
        out = out + shared_forward(x, w_sh_in, w_sh_out, act, b_sh_in, b_sh_out)
    return out


def seeded_block_weights(seed, d_model, n_experts, d_hidden, n_shared, dtype=torch.bfloat16):
    """Weights of a block drawn from one CPU generator in a fixed order (router W ~ N(0, 0.02),
    expert weights ~ N(0, 1/sqrt(fan_in))), rounded once to dtype: what lets a golden file for
    nanoSpeaker's real block shape (34 MB of weights) hold only the seed."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape: torch.randn(*shape, generator=g)
    w = {"router_W": rn(d_model, n_experts) * 0.02,
         "W_in": rn(n_experts, d_model, 2 * d_hidden) * d_model ** -0.5,
         "W_out": rn(n_experts, d_hidden, d_model) * d_hidden ** -0.5}
    if n_shared:
        w["W_sh_in"] = rn(n_shared, d_model, 2 * d_hidden) * d_model ** -0.5
        w["W_sh_out"] = rn(n_shared, d_hidden, d_model) * d_hidden ** -0.5
    return {k: v.to(dtype) for k, v in w.items()}


def dense_forward(x, w_in, w_out, topk_w, topk_idx, act="silu", w_sh_in=None, w_sh_out=None):
    """Every expert on every token mixed by a dense gate matrix (src/model/moe.py:459-474)."""
    fn = ACTS[act]
    gates = torch.zeros(x.shape[0], w_in.shape[0], dtype=x.dtype)
    gates.scatter_(1, topk_idx, topk_w)
    gate, up = (x @ w_in).chunk(2, dim=-1)
    y = (fn(gate) * up) @ w_out
    out = torch.einsum("enf,ne->nf", y, gates)
    if w_sh_in is not None:
        out = out + shared_forward(x, w_sh_in, w_sh_out, act)
    return out


def _act_grad(g, act):
    if act in ("silu", "swish"):
        s = torch.sigmoid(g)
        return s * (1 + g * (1 - s))
    if act == "gelu":
        return 0.5 * (1 + torch.erf(g * 0.7071067811865476)) + \
            g * 0.3989422804014327 * torch.exp(-0.5 * g * g)
    if act == "relu":
        return (g > 0).to(g.dtype)
    if act == "sigmoid":
        s = torch.sigmoid(g)
        return s * (1 - s)
    t = torch.tanh(g)
    return 1 - t * t


def experts_backward(d_out, x, w_in, w_out, topk_w, topk_idx, act="silu", w_sh_in=None,
                     w_sh_out=None):
    """Closed-form gradients of experts_forward in the input dtype's fp32 view:
    (dx, dW_in, dW_out, dtopk_w, dW_sh_in, dW_sh_out). Formulas as in
    src/model/moe_kernel.py:510-553, 626-739: G = dOut W_out^T, dw = <G, hid>,
    dA1 = [w G u act'(g) | w G act(g)], dx = sum dA1 W_in^T, dW_in = x^T dA1,
    dW_out = hid^T (w dOut). Inputs are promoted to fp32; no intermediate rounding."""
    fn = ACTS[act]
    f = lambda t: None if t is None else t.float()
    d_out, x, w_in, w_out, topk_w = f(d_out), f(x), f(w_in), f(w_out), f(topk_w)
    n_experts, k = w_in.shape[0], topk_idx.shape[1]
    _, order, token_idx, counts = plan(topk_idx, n_experts)
    sizes = counts.tolist()
    dx = torch.zeros_like(x)
    dw_in, dw_out = torch.zeros_like(w_in), torch.zeros_like(w_out)
    dtw = torch.zeros(topk_w.numel())
    w_sorted = topk_w.reshape(-1).index_select(0, order)
    start = 0
    for e in range(n_experts):
        c = sizes[e]
        if c == 0:
            continue
        tok, pairs, w = token_idx[start:start + c], order[start:start + c], w_sorted[start:start + c]
        start += c
        xe, de = x[tok], d_out[tok]
        g, u = (xe @ w_in[e]).chunk(2, dim=-1)
        a = fn(g)
        hid = a * u
        G = de @ w_out[e].t()
        dtw[pairs] = (G * hid).sum(-1)
        dh = w[:, None] * G
        da1 = torch.cat([dh * u * _act_grad(g, act), dh * a], dim=-1)
        dx.index_add_(0, tok, da1 @ w_in[e].t())
        dw_in[e] = xe.t() @ da1
        dw_out[e] = hid.t() @ (w[:, None] * de)
    dsi = dso = None
    if w_sh_in is not None:
        w_sh_in, w_sh_out = f(w_sh_in), f(w_sh_out)
        dsi, dso = torch.zeros_like(w_sh_in), torch.zeros_like(w_sh_out)
        for s in range(w_sh_in.shape[0]):
            g, u = (x @ w_sh_in[s]).chunk(2, dim=-1)
            a = fn(g)
            hid = a * u
            G = d_out @ w_sh_out[s].t()
            da1 = torch.cat([G * u * _act_grad(g, act), G * a], dim=-1)
            dx += da1 @ w_sh_in[s].t()
            dsi[s] = x.t() @ da1
            dso[s] = hid.t() @ d_out
    return dx, dw_in, dw_out, dtw.view_as(topk_w), dsi, dso


# ------------------------------------------------------------------------------- whole block
class OracleBlock(torch.nn.Module):
    """The reference block's forward restated as an autograd-capable CPU module: parameters with
    the reference's names and shapes, forward = router -> plan -> eager ragged loop -> shared.
    Used for end-to-end output and gradient parity and as the timed CPU baseline."""

    def __init__(self, d_model, n_experts, d_ff, top_k, n_shared=0, activation="silu",
                 normalize_weights=True, aux_loss_coef=1e-2, std=0.02, canonical_ties=False):
        super().__init__()
        h = 2 * d_ff // 3
        self.d_model, self.n_experts, self.top_k, self.n_shared = d_model, n_experts, top_k, n_shared
        self.activation, self.normalize_weights = activation, normalize_weights
        self.aux_loss_coef, self.canonical_ties = aux_loss_coef, canonical_ties
        P = torch.nn.Parameter
        self.router_W = P(torch.randn(d_model, n_experts) * std)
        self.W_in = P(torch.randn(n_experts, d_model, 2 * h) * std)
        self.W_out = P(torch.randn(n_experts, h, d_model) * std)
        self.W_sh_in = P(torch.randn(n_shared, d_model, 2 * h) * std) if n_shared else None
        self.W_sh_out = P(torch.randn(n_shared, h, d_model) * std) if n_shared else None
        self.aux_loss = torch.zeros(())
        self.expert_counts = torch.zeros(n_experts)
        self.routing_bias = None  # optional additive per-expert logit bias (benchmark skew)
        # optional [N, E] fp32 tensor whose VALUES replace the logits (gradients still flow to x
        # and router_W): lets a test make both sides select from bit-identical logits
        self.logits_override = None

    def route(self, x):
        logits = router_logits(x, self.router_W)
        if self.routing_bias is not None:
            logits = logits + self.routing_bias
        if self.logits_override is not None:
            logits = logits + (self.logits_override - logits).detach()
        full = self.training and self.aux_loss_coef != 0.0
        idx = canonical_topk(logits.detach(), self.top_k) if self.canonical_ties else None
        w, idx, probs = router_select(logits, self.top_k, self.normalize_weights, full, idx)
        return logits, w.to(x.dtype), idx, probs

    def forward(self, x):
        shape = x.shape
        x = x.reshape(-1, self.d_model)
        _, w, idx, probs = self.route(x)
        counts = torch.bincount(idx.reshape(-1), minlength=self.n_experts)
        self.expert_counts = counts
        self.aux_loss = (balance_loss(probs, counts, self.aux_loss_coef, self.n_experts)
                         if probs is not None else torch.zeros((), dtype=x.dtype))
        out = experts_forward(x, self.W_in, self.W_out, w, idx, self.activation, self.W_sh_in,
                              self.W_sh_out)
        return out.view(shape)


# ------------------------------------------------------------------------- the FFN sublayer
def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm.forward of the reference (src/model/ln.py:31-38): the row is rescaled by the
    reciprocal RMS of its features and multiplied by gamma; no mean, no shift."""
    return F.rms_norm(x, (x.shape[-1],), gamma, eps)


def rmsnorm_backward(dh: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6):
    """Closed form of the gradient through rmsnorm, in fp32: (dx, dgamma).
    With r = rsqrt(mean(x^2) + eps):  dx = r * (gamma * dh) - x * r^3 / D * <gamma * dh, x>,
    dgamma = sum over rows of dh * x * r."""
    xf, df, gf = x.float(), dh.float(), gamma.float()
    r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    dot = (gf * df * xf).sum(-1, keepdim=True)
    dx = r * gf * df - xf * r.pow(3) * dot / x.shape[-1]
    return dx, (df * xf * r).sum(0)


class OracleSublayer(torch.nn.Module):
    """x + ffn(norm_ffn(x)) with the balance loss next to it: the tail of Block.forward
    (src/model/nanospeaker.py:165-169)."""

    def __init__(self, block: "OracleBlock", eps: float = 1e-6):
        super().__init__()
        self.block = block
        self.eps = eps
        self.gamma = torch.nn.Parameter(torch.ones(block.router_W.shape[0]))

    def forward(self, x: torch.Tensor):
        out = x + self.block(rmsnorm(x, self.gamma, self.eps))
        return out, self.block.aux_loss


# --------------------------------------------------------------------- expert-parallel plan
def ep_plan(cnt_all, bounds, rank: int, cap_tiles: int):
    """Where the pairs of every home rank live in the owners' slot-ordered buffers, in numpy
    integers (the reference is single-GPU; this restates the layout rule the peer-memory path
    defines, to check the CUDA plan kernel bit for bit).

    cnt_all [G, E]: pairs of home rank g routed to expert e. bounds [G+1]: rank r owns experts
    [bounds[r], bounds[r+1]). An owner's buffer holds its experts' runs in expert order, each run
    padded to a multiple of 128 rows, and inside a run the home ranks' pairs in rank order (each
    rank's pairs in the order of its own stable sort, as `plan` gives them).

    Returns for `rank`: owner_of [E], send_row0 [E] (row of its first pair of expert e in the
    owner's buffer), own_offs [E_r+1], own_counts [E_r], own_npp, own_eids [cap_tiles]."""
    cnt_all = np.asarray(cnt_all, dtype=np.int64)
    n_ranks, n_experts = cnt_all.shape
    tot = cnt_all.sum(0)
    before = cnt_all[:rank].sum(0)
    owner_of = np.zeros(n_experts, dtype=np.int32)
    start = np.zeros(n_experts, dtype=np.int64)
    for r in range(n_ranks):
        run = 0
        for e in range(bounds[r], bounds[r + 1]):
            owner_of[e] = r
            start[e] = run
            run += (tot[e] + ALIGN_M - 1) // ALIGN_M * ALIGN_M
        if r == rank:
            live = run
    lo, hi = bounds[rank], bounds[rank + 1]
    own_offs = np.concatenate([start[lo:hi], [live]]).astype(np.int32)
    own_eids = np.zeros(cap_tiles, dtype=np.int32)
    for e in range(lo, hi):
        own_eids[start[e] // ALIGN_M: (start[e] + (tot[e] + ALIGN_M - 1) // ALIGN_M * ALIGN_M)
                 // ALIGN_M] = e - lo
    return (owner_of, (start + before).astype(np.int32), own_offs, tot[lo:hi].astype(np.int32),
            int(live), own_eids)


# ------------------------------------------------------------------- Muon's Newton-Schulz
def newton_schulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """zeropower_via_newtonschulz5 (src/train/optim.py:27-40) restated: the quintic Newton-Schulz
    iteration X <- a X + (b A + c A A) X with A = X X^T on X = G / (|G|_F + eps), in bf16, the
    smaller dimension leading (tall matrices are transposed on the way in and out). Batched over
    leading dimensions."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.to(torch.bfloat16)
    tall = X.shape[-2] > X.shape[-1]
    if tall:
        X = X.transpose(-2, -1)
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + eps)
    for _ in range(steps):
        A = X @ X.transpose(-2, -1)
        X = a * X + (b * A + c * (A @ A)) @ X
    return X.transpose(-2, -1) if tall else X


def muon_step(p, grad, buf, lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5):
    """One Muon update of parameter p in place (src/train/optim.py:75-100): bf16 momentum buffer
    `buf` lerped towards the gradient, Nesterov direction orthogonalised, aspect-ratio scale,
    decoupled weight decay. Returns the applied delta."""
    g = grad.to(buf.dtype)
    buf.lerp_(g, 1 - momentum)
    update = newton_schulz5(g.lerp(buf, momentum), ns_steps)
    scale = max(1.0, p.shape[-2] / p.shape[-1]) ** 0.5
    delta = update.to(p.dtype) * (-lr * scale)
    p.mul_(1 - lr * weight_decay)
    p.add_(delta)
    return delta


MUON_SHAPES = (("in", (1, 576, 256)), ("out", (1, 128, 576)))


def seeded_muon_inputs(seed=21):
    """The inputs of the Muon golden, re-drawn from the seed: per shape a gradient for the bare
    Newton-Schulz call (g_*), a weight (w_*) and two optimizer-step gradients (grad_*_0/1)."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for tag, shape in MUON_SHAPES:
        out[f"g_{tag}"] = (torch.randn(*shape, generator=gen) * 0.02).bfloat16()
        out[f"w_{tag}"] = (torch.randn(*shape, generator=gen) * 0.05).bfloat16()
        for step in range(2):
            out[f"grad_{tag}_{step}"] = (torch.randn(*shape, generator=gen) * 0.02).bfloat16()
    return out
