"""Generate the golden vectors in this directory by running the UNMODIFIED reference.

Usage (needs a checkout of Osmansiddiquer/nanospeaker):
    python tests/golden/make_golden.py /path/to/nanospeaker [--sublayer-only | --bias-only | --real-only | --muon-only]

Each .npz holds the inputs and everything the reference's pure-PyTorch MoE path
(MoEBlock(..., fused=False, kernel=False, capacity_factor=None) on CPU) computes from them:
router logits, top-k, the stable-sort plan, the block output, the balance loss and -- for the
training cases -- all gradients of `out.float().square().mean() + aux_loss`.
bf16 tensors are stored as their uint16 bit patterns under the key suffix `__bf16`.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def put(store, name, t):
    t = t.detach()
    if t.dtype == torch.bfloat16:
        store[name + "__bf16"] = t.contiguous().view(torch.int16).numpy().view(np.uint16)
    else:
        store[name] = t.contiguous().numpy()


def block_case(MoEBlock, name, *, d_model, n_experts, d_ff, top_k, n_shared, tokens, dtype, train,
               seed, activation="silu", normalize=True, bias=False):
    torch.manual_seed(seed)
    m = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                 capacity_factor=None, activation=activation, normalize_weights=normalize,
                 fused=False, kernel=False, bias=bias)
    with torch.no_grad():
        m.router.W.copy_(torch.randn_like(m.router.W) * 0.3)
        m.W_in.copy_(torch.randn_like(m.W_in) * d_model ** -0.5)
        m.W_out.copy_(torch.randn_like(m.W_out) * m.d_hidden ** -0.5)
        if n_shared:
            m.W_sh_in.copy_(torch.randn_like(m.W_sh_in) * d_model ** -0.5)
            m.W_sh_out.copy_(torch.randn_like(m.W_sh_out) * m.d_hidden ** -0.5)
    x = torch.randn(tokens, d_model)
    if bias:   # drawn after everything else so the other cases keep their values
        with torch.no_grad():
            m.b_in.copy_(torch.randn_like(m.b_in) * 0.5)
            m.b_out.copy_(torch.randn_like(m.b_out) * 0.5)
            if n_shared:
                m.b_sh_in.copy_(torch.randn_like(m.b_sh_in) * 0.5)
                m.b_sh_out.copy_(torch.randn_like(m.b_sh_out) * 0.5)
    m = m.to(dtype)
    x = x.to(dtype).requires_grad_(train)
    m.train(train)

    s = {}
    put(s, "x", x)
    put(s, "router_W", m.router.W)
    put(s, "W_in", m.W_in)
    put(s, "W_out", m.W_out)
    if n_shared:
        put(s, "W_sh_in", m.W_sh_in)
        put(s, "W_sh_out", m.W_sh_out)
    if bias:
        put(s, "b_in", m.b_in)
        put(s, "b_out", m.b_out)
        if n_shared:
            put(s, "b_sh_in", m.b_sh_in)
            put(s, "b_sh_out", m.b_sh_out)
    s["meta"] = np.array([d_model, n_experts, d_ff, top_k, n_shared, tokens, int(train),
                          int(normalize)], dtype=np.int64)
    s["activation"] = np.array(activation)
    s["dtype"] = np.array(str(dtype).replace("torch.", ""))

    with torch.set_grad_enabled(train):
        logits = (x.detach() @ m.router.W.detach()).float()
        topk_w, topk_idx, probs = m.router(x.detach())
        experts, order, token_idx, counts = m._plan(topk_idx)
        out = m(x)
        if not train:
            dense = m.dense_forward(x)
            put(s, "dense_out", dense)
    put(s, "logits", logits)
    put(s, "topk_w", topk_w)
    put(s, "topk_idx", topk_idx)
    if probs is not None:
        put(s, "probs", probs)
    put(s, "plan_experts", experts)
    put(s, "plan_order", order)
    put(s, "plan_token_idx", token_idx)
    put(s, "plan_counts", counts)
    put(s, "out", out)
    put(s, "aux_loss", m.aux_loss.float())
    if train:
        (out.float().square().mean() + m.aux_loss).backward()
        put(s, "grad_x", x.grad)
        put(s, "grad_router_W", m.router.W.grad)
        put(s, "grad_W_in", m.W_in.grad)
        put(s, "grad_W_out", m.W_out.grad)
        if n_shared:
            put(s, "grad_W_sh_in", m.W_sh_in.grad)
            put(s, "grad_W_sh_out", m.W_sh_out.grad)
        if bias:
            put(s, "grad_b_in", m.b_in.grad)
            put(s, "grad_b_out", m.b_out.grad)
            if n_shared:
                put(s, "grad_b_sh_in", m.b_sh_in.grad)
                put(s, "grad_b_sh_out", m.b_sh_out.grad)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **s)
    print(name, {k: v.shape for k, v in s.items() if hasattr(v, "shape") and v.ndim})


def sublayer_case(MoEBlock, RMSNorm, name, *, d_model, n_experts, d_ff, top_k, n_shared, tokens,
                  dtype, seed):
    """The FFN sublayer of the reference's Block: x + ffn(norm_ffn(x)), training mode, all
    gradients of out^2.mean() + aux_loss (src/model/nanospeaker.py:165-169)."""
    torch.manual_seed(seed)
    m = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                 capacity_factor=None, normalize_weights=True, fused=False, kernel=False)
    norm = RMSNorm(d_model)
    with torch.no_grad():
        m.router.W.copy_(torch.randn_like(m.router.W) * 0.3)
        m.W_in.copy_(torch.randn_like(m.W_in) * d_model ** -0.5)
        m.W_out.copy_(torch.randn_like(m.W_out) * m.d_hidden ** -0.5)
        m.W_sh_in.copy_(torch.randn_like(m.W_sh_in) * d_model ** -0.5)
        m.W_sh_out.copy_(torch.randn_like(m.W_sh_out) * m.d_hidden ** -0.5)
        norm.gamma.copy_(1.0 + 0.2 * torch.randn(d_model))
    x = (torch.randn(tokens, d_model) * 1.7).to(dtype).requires_grad_(True)
    m, norm = m.to(dtype).train(), norm.to(dtype).train()
    s = {}
    put(s, "x", x)
    put(s, "gamma", norm.gamma)
    put(s, "router_W", m.router.W)
    put(s, "W_in", m.W_in)
    put(s, "W_out", m.W_out)
    put(s, "W_sh_in", m.W_sh_in)
    put(s, "W_sh_out", m.W_sh_out)
    s["meta"] = np.array([d_model, n_experts, d_ff, top_k, n_shared, tokens], dtype=np.int64)
    s["epsilon"] = np.array(norm.epsilon)
    s["dtype"] = np.array(str(dtype).replace("torch.", ""))
    h = norm(x)
    put(s, "h", h)
    put(s, "logits", (h.detach() @ m.router.W.detach()).float())
    out = x + m(h)
    put(s, "out", out)
    put(s, "aux_loss", m.aux_loss.float())
    (out.float().square().mean() + m.aux_loss).backward()
    put(s, "grad_x", x.grad)
    put(s, "grad_gamma", norm.gamma.grad)
    put(s, "grad_router_W", m.router.W.grad)
    put(s, "grad_W_in", m.W_in.grad)
    put(s, "grad_W_out", m.W_out.grad)
    put(s, "grad_W_sh_in", m.W_sh_in.grad)
    put(s, "grad_W_sh_out", m.W_sh_out.grad)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **s)
    print(name, tuple(out.shape))


# every REAL_STRIDE-th element of the big weight gradients goes into the real-shape golden
REAL_STRIDE = 61


def real_shape_case(MoEBlock, name, *, tokens, seed):
    """nanoSpeaker's own block shape (d_model 576, 76 routed + 2 shared experts, d_expert 128,
    top-6), bf16, training mode: forward, balance loss and all gradients of
    out^2.mean() + aux_loss. The 34 MB of weights are not stored: they come from
    oracle.moe_oracle.seeded_block_weights(seed, ...), and the two big weight gradients are stored
    as every REAL_STRIDE-th element plus per-expert norms. bf16-derived logits tie now and then,
    and torch.topk's choice among equal logits is unspecified: the seed is one for which every
    token's selected SET is the same under any tie rule (checked by tests/test_oracle.py), so the
    output and the gradients do not depend on the rule."""
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.moe_oracle import seeded_block_weights
    D, E, k, S, d_ff, H = 576, 76, 6, 2, 192, 128
    w = seeded_block_weights(seed, D, E, H, S)
    m = MoEBlock(D, E, d_ff=d_ff, top_k=k, n_shared=S, capacity_factor=None, fused=False,
                 kernel=False).to(torch.bfloat16)
    with torch.no_grad():
        m.router.W.copy_(w["router_W"])
        for key in ("W_in", "W_out", "W_sh_in", "W_sh_out"):
            getattr(m, key).copy_(w[key])
    x = torch.randn(tokens, D, generator=torch.Generator().manual_seed(seed + 1)).bfloat16()
    x.requires_grad_(True)
    m.train()
    s = {}
    put(s, "x", x)
    s["meta"] = np.array([D, E, d_ff, k, S, tokens, seed, REAL_STRIDE], dtype=np.int64)
    # exact (integer) fingerprint of the drawn weights: the sum of their bf16 bit patterns
    s["weights_fingerprint"] = np.array(
        [int(w[key].view(torch.int16).long().sum())
         for key in ("router_W", "W_in", "W_out", "W_sh_in", "W_sh_out")], dtype=np.int64)
    put(s, "logits", (x.detach() @ m.router.W.detach()).float())
    topk_w, topk_idx, _ = m.router(x.detach())
    _, order, _, counts = m._plan(topk_idx)
    put(s, "topk_idx", topk_idx)
    put(s, "topk_w", topk_w)
    put(s, "plan_order", order)
    put(s, "plan_counts", counts)
    out = m(x)
    put(s, "out", out)
    put(s, "aux_loss", m.aux_loss.float())
    (out.float().square().mean() + m.aux_loss).backward()
    put(s, "grad_x", x.grad)
    put(s, "grad_router_W", m.router.W.grad)
    put(s, "grad_W_sh_in", m.W_sh_in.grad)
    put(s, "grad_W_sh_out", m.W_sh_out.grad)
    for key in ("W_in", "W_out"):
        grad = getattr(m, key).grad
        put(s, f"grad_{key}_strided", grad.reshape(-1)[::REAL_STRIDE])
        put(s, f"grad_{key}_norms", grad.float().flatten(1).norm(dim=1))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **s)
    print(name, tuple(out.shape))


MUON_STRIDE = 7


def muon_case(name):
    """Muon's Newton-Schulz and two optimizer steps of the reference (src/train/optim.py) on
    gradients shaped like one expert of the block's stacked weights: W_in-like [1, 576, 256] (tall:
    taken transposed) and W_out-like [1, 128, 576] (wide). Inputs come from
    oracle.moe_oracle.seeded_muon_inputs(seed); stored
    are the orthogonalised gradients and every MUON_STRIDE-th element of the weights after the steps."""
    from src.train.optim import Muon, zeropower_via_newtonschulz5
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.moe_oracle import MUON_SHAPES, seeded_muon_inputs
    t = seeded_muon_inputs()
    s = {"fingerprint": np.array([int(v.view(torch.int16).long().sum()) for v in t.values()],
                                 dtype=np.int64)}
    for tag, _ in MUON_SHAPES:
        put(s, f"ns_{tag}", zeropower_via_newtonschulz5(t[f"g_{tag}"]))
        w = torch.nn.Parameter(t[f"w_{tag}"].clone())
        opt = Muon([w], lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5)
        for step in range(2):
            w.grad = t[f"grad_{tag}_{step}"].clone()
            opt.step()
        put(s, f"w_{tag}_after", w.reshape(-1)[::MUON_STRIDE])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **s)
    print(name, sorted(s))


def routing_case(MoEBlock, name, *, tokens, n_experts, top_k, seed, bf16_logits):
    """Routing only at nanoSpeaker's width: logits -> torch.topk -> stable-sort plan."""
    torch.manual_seed(seed)
    m = MoEBlock(64, n_experts, d_ff=192, top_k=top_k, capacity_factor=None, fused=False,
                 kernel=False)
    logits = torch.randn(tokens, n_experts) * 0.5
    if bf16_logits:
        logits = logits.bfloat16().float()
    topk_idx = logits.topk(top_k, dim=-1).indices
    experts, order, token_idx, counts = m._plan(topk_idx)
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"), logits=logits.numpy(), topk_idx=topk_idx.numpy(),
        plan_order=order.numpy(), plan_token_idx=token_idx.numpy(), plan_counts=counts.numpy(),
        meta=np.array([tokens, n_experts, top_k, int(bf16_logits)], dtype=np.int64))
    print(name, tuple(logits.shape))


def main():
    # path of the reference checkout: first argument, else $NANOSPEAKER_REF
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["NANOSPEAKER_REF"]
    sys.path.insert(0, ref)
    from src.model.moe import MoEBlock  # the reference, unmodified
    from src.model.ln import RMSNorm

    if "--muon-only" in sys.argv:
        muon_case("muon_newton_schulz")
        return
    if "--real-only" in sys.argv:
        real_shape_case(MoEBlock, "block_real_shape_bf16_train", tokens=256, seed=27)
        return
    sub = dict(d_model=64, n_experts=4, d_ff=192, top_k=2, n_shared=1, tokens=80)
    sublayer_case(MoEBlock, RMSNorm, "sublayer_fp32_train", dtype=torch.float32, seed=7, **sub)
    sublayer_case(MoEBlock, RMSNorm, "sublayer_bf16_train", dtype=torch.bfloat16, seed=8, **sub)
    if "--sublayer-only" in sys.argv:
        return
    common = dict(d_model=64, n_experts=4, d_ff=192, top_k=2, n_shared=1, tokens=80)
    block_case(MoEBlock, "block_fp32_train_bias", dtype=torch.float32, train=True, seed=9,
               bias=True, **common)
    block_case(MoEBlock, "block_bf16_train_bias", dtype=torch.bfloat16, train=True, seed=10,
               bias=True, **common)
    if "--bias-only" in sys.argv:
        return

    common = dict(d_model=64, n_experts=4, d_ff=192, top_k=2, n_shared=1, tokens=80)
    block_case(MoEBlock, "block_fp32_eval", dtype=torch.float32, train=False, seed=1, **common)
    block_case(MoEBlock, "block_fp32_train", dtype=torch.float32, train=True, seed=2, **common)
    block_case(MoEBlock, "block_bf16_train", dtype=torch.bfloat16, train=True, seed=3, **common)
    block_case(MoEBlock, "block_bf16_eval_gelu", dtype=torch.bfloat16, train=False, seed=4,
               activation="gelu", normalize=False, **common)
    routing_case(MoEBlock, "routing_e76_k6_fp32", tokens=512, n_experts=76, top_k=6, seed=5,
                 bf16_logits=False)
    routing_case(MoEBlock, "routing_e76_k6_bf16", tokens=512, n_experts=76, top_k=6, seed=6,
                 bf16_logits=True)
    real_shape_case(MoEBlock, "block_real_shape_bf16_train", tokens=256, seed=27)
    muon_case("muon_newton_schulz")


if __name__ == "__main__":
    main()
