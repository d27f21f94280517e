"""End-to-end GPU parity of the MoE block against the CPU oracle and the reference's golden vectors.

Bars (from the block's acceptance criteria): expert selection and permutation bit-exact given
identical fp32 logits; outputs and gradients within rel-L2 1e-2 of the reference's bf16 path
(fp32 accumulation on the GPU side). The tighter 5e-3 bar is against the fp32 oracle evaluated on
the same bf16 inputs."""
import copy

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2        # vs the reference's own bf16 path
TOL_FP32 = 5e-3   # vs fp32 math on the same bf16 inputs


def _cuda_block_from_golden(g):
    from nanospeaker_b200 import MoEBlock
    d_model, n_experts, d_ff, top_k, n_shared, tokens, train, normalize = g["meta"].tolist()
    m = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                 capacity_factor=None, activation=g["activation"],
                 normalize_weights=bool(normalize))
    m = m.to(torch.bfloat16)
    with torch.no_grad():
        m.router.W.copy_(g["router_W"])
        m.W_in.copy_(g["W_in"])
        m.W_out.copy_(g["W_out"])
        if n_shared:
            m.W_sh_in.copy_(g["W_sh_in"])
            m.W_sh_out.copy_(g["W_sh_out"])
    m.train(bool(train))
    return m.cuda()


@pytest.mark.parametrize("case", ["block_bf16_train", "block_bf16_eval_gelu"])
def test_fused_forward_matches_reference_golden(case):
    """Experts driven with the reference's own routing, so tie-breaking cannot leak in."""
    from nanospeaker_b200 import fused_moe_forward
    g = load_golden(case)
    m = _cuda_block_from_golden(g)
    out, counts = fused_moe_forward(
        g["x"].cuda(), m.W_in, m.W_out, g["topk_w"].cuda(), g["topk_idx"].cuda(), None, None,
        g["activation"], w_sh_in=m.W_sh_in, w_sh_out=m.W_sh_out)
    assert torch.equal(counts.cpu().long(), g["plan_counts"])
    assert rel_l2(out.cpu(), g["out"]) < TOL
    f = lambda t: t.float()
    ref32 = O.experts_forward(f(g["x"]), f(g["W_in"]), f(g["W_out"]), f(g["topk_w"]),
                              g["topk_idx"], g["activation"], f(g["W_sh_in"]), f(g["W_sh_out"]))
    assert rel_l2(out.cpu(), ref32) < TOL_FP32


def test_module_forward_backward_matches_reference_golden():
    """Whole module (router included) on the reference's bf16 training case: every gradient the
    reference produced, within the bf16 bar."""
    g = load_golden("block_bf16_train")
    m = _cuda_block_from_golden(g)
    x = g["x"].cuda().requires_grad_(True)
    out = m(x)
    assert m._use_kernel(x), "kernel path was not taken"
    assert torch.equal(m.expert_counts.cpu().long(), g["plan_counts"])
    assert abs(float(m.aux_loss) - float(g["aux_loss"])) < 1e-4
    (out.float().square().mean() + m.aux_loss).backward()
    assert rel_l2(out.detach().cpu(), g["out"]) < TOL
    for got, key in [(x.grad, "grad_x"), (m.W_in.grad, "grad_W_in"), (m.W_out.grad, "grad_W_out"),
                     (m.W_sh_in.grad, "grad_W_sh_in"), (m.W_sh_out.grad, "grad_W_sh_out"),
                     (m.router.W.grad, "grad_router_W")]:
        assert rel_l2(got.cpu(), g[key]) < (2e-2 if key == "grad_router_W" else TOL), key


def test_module_with_expert_biases_matches_reference_golden():
    """bias=True: b_in / b_sh_in before the GLU, b_out / b_sh_out before the weight scale, in the
    kernels' epilogues; output and every gradient of the reference's bf16 training case, the four
    bias gradients and the router's (whose dtopk_w carries <dOut, b_out>) included."""
    from nanospeaker_b200 import MoEBlock, fused_moe_forward
    g = load_golden("block_bf16_train_bias")
    d_model, n_experts, d_ff, top_k, n_shared, tokens, train, normalize = g["meta"].tolist()
    m = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared, bias=True,
                 capacity_factor=None).to(torch.bfloat16)
    with torch.no_grad():
        for name, key in [("router.W", "router_W"), ("W_in", "W_in"), ("W_out", "W_out"),
                          ("W_sh_in", "W_sh_in"), ("W_sh_out", "W_sh_out"), ("b_in", "b_in"),
                          ("b_out", "b_out"), ("b_sh_in", "b_sh_in"), ("b_sh_out", "b_sh_out")]:
            m.get_parameter(name).copy_(g[key])
    assert float(g["b_sh_in"].abs().sum()) > 0 and float(g["b_sh_out"].abs().sum()) > 0
    m = m.cuda().train()
    x = g["x"].cuda().requires_grad_(True)
    assert m._use_kernel(x), "kernel path was not taken"
    # experts alone on the reference's routing, forward
    out_e, _ = fused_moe_forward(x.detach(), m.W_in, m.W_out, g["topk_w"].cuda(),
                                 g["topk_idx"].cuda(), m.b_in, m.b_out, "silu",
                                 w_sh_in=m.W_sh_in, w_sh_out=m.W_sh_out, b_sh_in=m.b_sh_in,
                                 b_sh_out=m.b_sh_out)
    assert rel_l2(out_e.detach().cpu(), g["out"]) < TOL
    # whole module, forward + backward
    out = m(x)
    assert torch.equal(m.expert_counts.cpu().long(), g["plan_counts"])
    (out.float().square().mean() + m.aux_loss).backward()
    assert rel_l2(out.detach().cpu(), g["out"]) < TOL
    for got, key in [(x.grad, "grad_x"), (m.W_in.grad, "grad_W_in"), (m.W_out.grad, "grad_W_out"),
                     (m.W_sh_in.grad, "grad_W_sh_in"), (m.W_sh_out.grad, "grad_W_sh_out"),
                     (m.b_in.grad, "grad_b_in"), (m.b_out.grad, "grad_b_out"),
                     (m.b_sh_in.grad, "grad_b_sh_in"), (m.b_sh_out.grad, "grad_b_sh_out"),
                     (m.router.W.grad, "grad_router_W")]:
        assert rel_l2(got.cpu(), g[key]) < (2e-2 if key == "grad_router_W" else TOL), key
    # the sublayer and the decode runner have no bias operands in their fused ops: with biases they
    # must go through the block's own forward instead of dropping them
    from nanospeaker_b200.decode import StackedMoEDecoder
    from nanospeaker_b200.sublayer import MoEFFNSublayer
    xd = g["x"].cuda()
    sub = MoEFFNSublayer(m).cuda().to(torch.bfloat16)
    assert not sub._fused_ok(xd)
    m.eval()
    with torch.no_grad():
        want = xd + m(xd)
        h = torch.nn.functional.rms_norm(xd, (xd.shape[-1],), sub.norm_gamma, sub.epsilon)
        assert rel_l2(sub(xd)[0], xd + m(h)) < 4e-3
        dec = StackedMoEDecoder([m])
        assert dec._fast_args(m, xd) is None
        assert rel_l2(dec.eager(xd), want) < 4e-3
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


@pytest.mark.parametrize("combine", ["atomic", "store"])
@pytest.mark.parametrize("cf,top_k", [(0.5, 2), (1.0, 2), (0.25, 1)])
def test_capacity_factor_runs_on_the_kernels_as_a_dispatch_variant(cf, top_k, combine):
    """An explicit capacity_factor (the reference's padded path, src/model/moe.py:225-283): the
    dispatch drops every pair past an expert's first `cap`, the same GEMM kernels run over what is
    kept. Against the module's torch path on the same weights: output, dropped count, counts
    (routing decisions, before the drop) and gradients; dropped pairs get no gradient."""
    from nanospeaker_b200 import MoEBlock
    torch.manual_seed(4)
    m = MoEBlock(64, 8, d_ff=192, top_k=top_k, n_shared=1, capacity_factor=cf)
    m = m.to(torch.bfloat16).cuda()
    with torch.no_grad():
        for p in (m.W_in, m.W_out, m.W_sh_in, m.W_sh_out):
            p.mul_(6.0)
        m.router.W.mul_(4.0)                         # an uneven load: some experts overflow
    m.combine_mode = combine
    twin = copy.deepcopy(m)
    twin.kernel = False
    x = torch.randn(700, 64, device="cuda").bfloat16()
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    oa, ob = m(xa), twin(xb)
    assert m._kernels_take(xa) and not m._use_kernel(xa) and not twin._kernels_take(xb)
    assert int(m.dropped) == int(twin.dropped) > 0
    assert torch.equal(m.expert_counts.long(), twin.expert_counts.long())
    assert int(m.expert_counts.sum()) == 700 * top_k
    assert rel_l2(oa, ob) < TOL
    (oa.float().square().mean() + m.aux_loss).backward()
    (ob.float().square().mean() + twin.aux_loss).backward()
    for name in ("W_in", "W_out", "W_sh_in", "W_sh_out"):
        assert rel_l2(getattr(m, name).grad, getattr(twin, name).grad) < 2e-2, name
    assert rel_l2(xa.grad, xb.grad) < 2e-2
    assert rel_l2(m.router.W.grad, twin.router.W.grad) < 3e-2
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


def _model_shape_pair(T, train, bias_std=0.0, seed=0):
    """nanoSpeaker's block (D=576, E=76, k=6, S=2, d_ff=192) with the benchmark's init, as a CUDA
    module and a CPU oracle twin sharing bf16 weights."""
    from nanospeaker_b200 import MoEBlock
    torch.manual_seed(seed)
    D, E, k, S = 576, 76, 6, 2
    x = torch.randn(T, D).bfloat16()
    m = MoEBlock(D, E, d_ff=192, top_k=k, n_shared=S, capacity_factor=None)
    with torch.no_grad():
        m.router.W.copy_(torch.randn(D, E) * 0.02)
        m.W_in.copy_(torch.randn(E, D, 256) * D ** -0.5)
        m.W_out.copy_(torch.randn(E, 128, D) * 128 ** -0.5)
        m.W_sh_in.copy_(torch.randn(S, D, 256) * D ** -0.5)
        m.W_sh_out.copy_(torch.randn(S, 128, D) * 128 ** -0.5)
    m = m.to(torch.bfloat16)
    o = O.OracleBlock(D, E, 192, k, S, canonical_ties=True).to(torch.bfloat16)
    with torch.no_grad():
        o.router_W.copy_(m.router.W)
        o.W_in.copy_(m.W_in)
        o.W_out.copy_(m.W_out)
        o.W_sh_in.copy_(m.W_sh_in)
        o.W_sh_out.copy_(m.W_sh_out)
    m.train(train)
    o.train(train)
    return x, m.cuda(), o


def test_config1_forward_T2048():
    """BASELINE config 1 (bf16 leg): T=2048 forward, eval mode, vs the oracle's bf16 and fp32 paths
    and its dense cross-check."""
    x, m, o = _model_shape_pair(2048, train=False)
    with torch.no_grad():
        xc = x.cuda()
        out = m(xc)
        gpu_logits = (xc @ m.router.W).float().cpu()
        o.logits_override = gpu_logits                       # identical fp32 logits on both sides
        ref = o(x)
        _, w, idx, _ = o.route(x)
        # selection is bit-exact given identical logits
        got_w, got_idx, _ = m.router(xc)
        assert torch.equal(got_idx.cpu(), idx)
        assert torch.equal(got_idx.cpu(), O.canonical_topk(gpu_logits, 6))
        assert torch.equal(m.expert_counts.cpu().long(), o.expert_counts)
        assert rel_l2(out.cpu(), ref) < TOL
        f = lambda t: t.detach().float()
        ref32 = O.experts_forward(f(x), f(o.W_in), f(o.W_out), f(w), idx, "silu", f(o.W_sh_in),
                                  f(o.W_sh_out))
        assert rel_l2(out.cpu(), ref32) < TOL_FP32
        dense = O.dense_forward(x, o.W_in, o.W_out, w, idx, "silu", o.W_sh_in, o.W_sh_out)
        assert rel_l2(out.cpu(), dense) < TOL
    assert float(m.aux_loss) == 0.0 and int(m.dropped) == 0


@pytest.mark.parametrize("skew_std", [0.27, 1.5])
def test_config2_forward_backward_T16384_skewed(skew_std):
    """BASELINE config 2 through MoEBlock.forward -- the whole-block op the benchmark times:
    T=16384, training mode, per-expert logit bias N(0, std) on the router (std 0.27: load CV ~ 1;
    the literal 1.5: CV ~ 3 with most experts empty), loss = out^2.mean() + aux. Output, balance
    loss, routing counts and all six gradients against the CPU oracle's autograd."""
    T = 16384
    x, m, o = _model_shape_pair(T, train=True, seed=2)
    torch.manual_seed(1)
    bias = torch.randn(76) * skew_std
    m.router.logit_bias = bias.cuda()
    xc = x.cuda().requires_grad_(True)
    out = m(xc)
    assert m._whole_block_ok(xc), "the whole-block op was not taken"
    (out.float().square().mean() + m.aux_loss).backward()

    o.logits_override = (_block_logits(m, xc.detach()) + bias.cuda()).cpu()   # identical logits
    xo = x.clone().requires_grad_(True)
    ref = o(xo)
    (ref.float().square().mean() + o.aux_loss).backward()

    assert torch.equal(m.expert_counts.cpu().long(), o.expert_counts)
    cnt = o.expert_counts.float()
    cv = float(cnt.std() / cnt.mean())
    assert (0.5 < cv < 2.0) if skew_std < 1 else (cv > 2.0 and int((cnt == 0).sum()) > 20), cv
    assert rel_l2(out.detach().cpu(), ref.detach()) < TOL
    assert abs(float(m.aux_loss) - float(o.aux_loss)) < 1e-4
    pairs = [("dx", xc.grad, xo.grad), ("dW_in", m.W_in.grad, o.W_in.grad),
             ("dW_out", m.W_out.grad, o.W_out.grad), ("dW_sh_in", m.W_sh_in.grad, o.W_sh_in.grad),
             ("dW_sh_out", m.W_sh_out.grad, o.W_sh_out.grad),
             ("d_router", m.router.W.grad, o.router_W.grad)]
    for name, a, b in pairs:
        assert rel_l2(a.cpu(), b) < (2e-2 if name == "d_router" else TOL), name
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


@pytest.mark.parametrize("combine", ["atomic", "store"])
def test_real_shape_block_matches_reference_golden(combine):
    """nanoSpeaker's own block shape against the golden the unmodified reference produced (d_model
    576, 76 + 2 experts, top-6, 256 tokens, bf16, training mode): MoEBlock.forward + backward on the
    GPU, output, balance loss, counts and every gradient."""
    from test_oracle import real_shape_oracle
    from nanospeaker_b200 import MoEBlock
    g = load_golden("block_real_shape_bf16_train")
    _, w, stride = real_shape_oracle(g)
    D, E, d_ff, k, S, *_ = g["meta"].tolist()
    m = MoEBlock(D, E, d_ff=d_ff, top_k=k, n_shared=S, capacity_factor=None).to(torch.bfloat16)
    with torch.no_grad():
        m.router.W.copy_(w["router_W"])
        for key in ("W_in", "W_out", "W_sh_in", "W_sh_out"):
            getattr(m, key).copy_(w[key])
    m = m.cuda().train()
    m.combine_mode = combine
    x = g["x"].cuda().requires_grad_(True)
    out = m(x)
    assert m._whole_block_ok(x)
    assert torch.equal(m.expert_counts.cpu().long(), g["plan_counts"])
    assert abs(float(m.aux_loss) - float(g["aux_loss"])) < 1e-4
    (out.float().square().mean() + m.aux_loss).backward()
    assert rel_l2(out.detach().cpu(), g["out"]) < TOL
    for got, key in [(x.grad, "grad_x"), (m.W_sh_in.grad, "grad_W_sh_in"),
                     (m.W_sh_out.grad, "grad_W_sh_out"), (m.router.W.grad, "grad_router_W")]:
        assert rel_l2(got.cpu(), g[key]) < (2e-2 if key == "grad_router_W" else TOL), key
    for key in ("W_in", "W_out"):
        grad = getattr(m, key).grad.cpu()
        assert rel_l2(grad.reshape(-1)[::stride], g[f"grad_{key}_strided"]) < TOL, key
        norms = grad.float().flatten(1).norm(dim=1)
        assert rel_l2(norms, g[f"grad_{key}_norms"]) < TOL, key
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


# What "the same" means for two runs of the kernel path. "store" sums a token's per-pair rows in fp32
# in pair order: bit-identical. "atomic" sums them with bf16 atomics in arrival order: equal up to
# the rounding of k + S bf16 additions.
ATOMIC_TOL = 5e-3


def _same(a, b, combine):
    if combine == "store":
        return torch.equal(a, b)
    return rel_l2(a, b) < ATOMIC_TOL


@pytest.mark.parametrize("combine", ["store", "atomic"])
def test_size_independent_properties_at_full_size(combine):
    """Properties that need no oracle: run-to-run determinism and token-permutation equivariance
    (bitwise with the fp32 store-then-reduce combine, to bf16 summation noise with the atomic
    one), linearity of the backward in grad_out, and the two combine modes against each other."""
    from nanospeaker_b200 import fused_moe_forward
    T = 16384
    x, m, _ = _model_shape_pair(T, train=False, seed=5)
    xc = x.cuda()
    with torch.no_grad():
        w, idx, _ = m.router(xc)
        run = lambda xx, ww, ii, mode=combine: fused_moe_forward(
            xx, m.W_in, m.W_out, ww, ii, None, None, "silu", w_sh_in=m.W_sh_in,
            w_sh_out=m.W_sh_out, combine=mode)[0]
        a, b = run(xc, w, idx), run(xc, w, idx)
        assert _same(a, b, combine)
        perm = torch.randperm(T, device="cuda")
        c = run(xc[perm], w[perm], idx[perm])
        assert _same(c, a[perm], combine)
        assert rel_l2(a, run(xc, w, idx, "store")) < ATOMIC_TOL
    xg = xc.clone().requires_grad_(True)
    out = fused_moe_forward(xg, m.W_in, m.W_out, w, idx, None, None, "silu",
                            w_sh_in=m.W_sh_in, w_sh_out=m.W_sh_out, combine=combine)[0]
    g1 = torch.randn_like(out)
    (d1,) = torch.autograd.grad(out, xg, g1, retain_graph=True)
    (d2,) = torch.autograd.grad(out, xg, 2 * g1)
    assert rel_l2(d2, 2 * d1.float()) < 1e-2


@pytest.mark.parametrize("n,top_k", [(1, 1), (1, 2), (3, 8), (127, 2), (128, 2), (129, 2)])
def test_degenerate_and_block_boundary_shapes(n, top_k):
    """Single tokens, fewer pairs than a block, exact block multiples
    (the shapes of tests/test_moe_kernel.py:125-130), forward and backward vs the eager twin."""
    from nanospeaker_b200 import MoEBlock
    m = MoEBlock(64, 8, d_ff=192, top_k=top_k, n_shared=1, capacity_factor=None)
    m = m.to(torch.bfloat16).cuda()
    with torch.no_grad():
        for p in (m.W_in, m.W_out, m.W_sh_in, m.W_sh_out):
            p.mul_(6.0)
    twin = copy.deepcopy(m)
    twin.kernel = False
    x = torch.randn(n, 64, device="cuda").bfloat16()
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    oa, ob = m(xa), twin(xb)
    assert m._use_kernel(xa) and not twin._use_kernel(xb)
    assert rel_l2(oa, ob) < TOL
    (oa.float().square().mean() + m.aux_loss).backward()
    (ob.float().square().mean() + twin.aux_loss).backward()
    assert rel_l2(xa.grad, xb.grad) < 2e-2
    assert rel_l2(m.W_out.grad, twin.W_out.grad) < 2e-2
    assert torch.equal(m.expert_counts.long(), twin.expert_counts.long())


def test_collapsed_router_exercises_the_ragged_tail():
    from nanospeaker_b200 import MoEBlock
    m = MoEBlock(64, 8, d_ff=192, top_k=1, capacity_factor=None).to(torch.bfloat16).cuda()
    with torch.no_grad():
        m.router.W.zero_()
        m.W_in.mul_(6.0)
        m.W_out.mul_(6.0)
    twin = copy.deepcopy(m)
    twin.kernel = False
    x = torch.randn(200, 64, device="cuda").bfloat16()
    with torch.no_grad():
        a, b = m(x), twin(x)
    assert m.expert_counts.tolist() == [200, 0, 0, 0, 0, 0, 0, 0]   # ties -> lowest index
    assert rel_l2(a, b) < TOL


def test_module_contract_on_cuda():
    from nanospeaker_b200 import MoEBlock
    m = MoEBlock(64, 8, d_ff=192, top_k=2, n_shared=2).to(torch.bfloat16).cuda()
    assert m.capacity_factor is None                       # "auto" -> dropless where kernels run
    x = torch.randn(2, 3, 5, 64, device="cuda").bfloat16()
    out = m(x)
    assert out.shape == x.shape and out.dtype == x.dtype   # leading dims and dtype preserved
    assert m.expert_counts.shape == (8,) and int(m.expert_counts.sum()) == 30 * 2
    assert int(m.dropped) == 0 and m.aux_loss.dim() == 0 and m.aux_loss.device == x.device
    empty = m(x[:0])
    assert empty.shape == (0, 3, 5, 64)
    with pytest.raises(ValueError):
        m(torch.randn(4, 63, device="cuda").bfloat16())
    assert set(m.state_dict()) == {"router.W", "W_in", "W_out", "W_sh_in", "W_sh_out"}
    # what the kernels decline runs the eager loop, never a wrong kernel
    assert not m.float()._use_kernel(torch.zeros(1, 64, device="cuda"))
    assert MoEBlock(64, 8, d_ff=192, bias=True).to(torch.bfloat16).cuda()._use_kernel(
        torch.zeros(1, 64, device="cuda").bfloat16())      # biases ride in the GEMM epilogues
    assert not MoEBlock(64, 8, d_ff=192, capacity_factor=1.25).to(torch.bfloat16).cuda()._use_kernel(
        torch.zeros(1, 64, device="cuda").bfloat16())
    assert not MoEBlock(64, 8, d_ff=192, activation=lambda t: t * torch.sigmoid(t))._kernel_act


@pytest.mark.parametrize("combine", ["store", "atomic"])
def test_reentrant_checkpoint_gives_identical_gradients(combine):
    """The block is re-run by activation checkpointing in the reference's trunk
    (src/model/nanospeaker.py:227); results must not change (bitwise with the fp32 combine; with
    the atomic one the recomputed forward differs by bf16 summation noise, which then runs through
    the backward)."""
    from torch.utils.checkpoint import checkpoint
    from nanospeaker_b200 import MoEBlock
    m = MoEBlock(64, 8, d_ff=192, top_k=2, n_shared=1).to(torch.bfloat16).cuda()
    m.combine_mode = combine
    x = torch.randn(300, 64, device="cuda").bfloat16()
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    m(xa).float().square().mean().backward()
    ga = m.W_in.grad.clone()
    m.zero_grad()
    checkpoint(m, xb, use_reentrant=True).float().square().mean().backward()
    assert _same(xa.grad, xb.grad, combine) and _same(ga, m.W_in.grad, combine)


def test_opcheck_and_fake_kernels():
    """torch.library's audit of schema, fake kernel and autograd registration
    (tests/test_moe_kernel.py:224-239)."""
    from nanospeaker_b200 import MoEBlock, moe_dispatch, moe_experts, router_topk
    idx = torch.randint(0, 4, (10, 2), device="cuda")
    torch.library.opcheck(moe_dispatch, (idx, 4))
    logits = torch.randn(10, 4, device="cuda", requires_grad=True)
    torch.library.opcheck(router_topk, (logits, 2, True, True))
    m = MoEBlock(64, 4, d_ff=192, n_shared=1).to(torch.bfloat16).cuda()
    x = torch.randn(10, 64, device="cuda").bfloat16()
    with torch.no_grad():
        w, idx, _ = m.router(x)
        # one shared expert = expert id 4 that every token is routed to with weight 1
        idx = torch.cat([idx, torch.full((10, 1), 4, device="cuda")], 1)
        w = torch.cat([w, torch.ones(10, 1, device="cuda", dtype=w.dtype)], 1)
    plan = moe_dispatch(idx, 5)
    rg = lambda t: t.detach().clone().requires_grad_(True)
    torch.library.opcheck(moe_experts, (rg(x), rg(m.W_in), rg(m.W_out), rg(w), rg(m.W_sh_in),
                                        rg(m.W_sh_out), *plan, "silu", True),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def _block_logits(m, xc):
    """The logits the block op routes on: its own router GEMM (bf16 out, fp32 accumulate) against
    the zero-padded router weight, bit for bit."""
    from nanospeaker_b200 import kernels
    from nanospeaker_b200.moe_kernel import _router_ld
    d, e = m.router.W.shape
    wp = xc.new_zeros((1, d, _router_ld(e)))
    wp[0, :, :e] = m.router.W
    return kernels.down_gemm(xc, wp, None, None, 1, None, None, 0)[0][:, :e].float()


def test_config3_decode_20_stacked_blocks_T64():
    """BASELINE config 3: 20 stacked blocks (independent weights) on T=64 tokens, forward only.
    Every block's output is checked against the oracle on the same input (identical logits), and
    the residual chain is carried on the GPU so the 20 launches see realistic inputs."""
    T, layers = 64, 20
    xc = None
    for layer in range(layers):
        x, m, o = _model_shape_pair(T, train=False, seed=100 + layer)
        with torch.no_grad():
            if xc is None:
                xc = x.cuda()
            out = m(xc)
            assert m._use_kernel(xc)
            xin = xc.cpu()
            o.logits_override = _block_logits(m, xc).cpu()
            ref = o(xin)
            assert torch.equal(m.expert_counts.cpu().long(), o.expert_counts), layer
            assert int(m.expert_counts.sum()) == T * 6
            assert rel_l2(out.cpu(), ref) < TOL, layer
            nxt = xc.float() + out.float()
            xc = (nxt / nxt.std()).to(torch.bfloat16)           # residual, kept at unit scale
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


def test_config4_prefill_forward_T131072_token_slices():
    """BASELINE config 4 (one GPU's view): T=131072 forward. Tokens are independent through the
    block, so slices of the big batch must equal the oracle run on those tokens alone."""
    T = 131072
    x, m, o = _model_shape_pair(T, train=False, seed=9)
    with torch.no_grad():
        xc = x.cuda()
        out = m(xc)
        counts = m.expert_counts.cpu().long()
        assert int(counts.sum()) == T * 6
        logits = _block_logits(m, xc)
        assert torch.equal(counts, torch.bincount(O.canonical_topk(logits.cpu(), 6).reshape(-1),
                                                  minlength=76))
        for lo in (0, 65536 - 128, T - 256):
            sl = slice(lo, lo + 256)
            o.logits_override = logits[sl].cpu()
            ref = o(x[sl])
            assert rel_l2(out[sl].cpu(), ref) < TOL, lo
        # the same rows come out bit-identical when their tokens are run as a small batch of their
        # own order-preserving subset (slot order inside an expert run is by token index)
        m.combine_mode = "store"
        big = m(xc)
        small = m(xc[:4096])
        assert rel_l2(small, big[:4096].float()) < 1e-6
        assert rel_l2(out, big) < ATOMIC_TOL        # the default (atomic) combine against it
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")
    assert torch.isfinite(out.float()).all()


def test_stacked_decoder_graph_replay_equals_eager_stack():
    """The graph-replayed stack of blocks (decode-shaped batch) gives the eager stack's bits, for
    several inputs through the same captured graph."""
    from nanospeaker_b200.decode import StackedMoEDecoder
    blocks = [_model_shape_pair(64, train=False, seed=200 + i)[1] for i in range(4)]
    stack = StackedMoEDecoder(blocks)
    for seed in (1, 2, 3):
        torch.manual_seed(seed)
        x = torch.randn(64, 576, device="cuda").bfloat16()
        want = stack.eager(x)
        got = stack.step(x)
        assert torch.equal(got, want)
        # the runner's six-launch block (residual inside the combine's fp32 sum, cached padded
        # router weight) against the blocks' own forward chained with a bf16 add
        # (block by block on the same input: chained, a rounding difference may flip a routing
        # decision further down the stack)
        from nanospeaker_b200 import moe_kernel as MK
        with torch.no_grad():
            for b in blocks:
                b.combine_mode = "store"
                ref = (x + b(x)).float()
                for mode, tol in (("store", 4e-3), ("atomic", 6e-3)):
                    fast = MK.moe_block_inference(x, *stack._fast_args(b, x), residual=x,
                                                  combine=mode)
                    assert rel_l2(fast.float(), ref) < tol, mode
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


def test_graphed_block_replays_the_blocks_training_step():
    """GraphedMoEBlock: forward and backward captured once per shape and replayed behind the module
    interface. Against the block called directly, over several steps with changing inputs and an
    in-place weight update in between: output, balance loss, counts and every gradient."""
    from nanospeaker_b200 import GraphedMoEBlock
    x0, m, _ = _model_shape_pair(1024, train=True, seed=6)
    m.combine_mode = "store"                     # bitwise comparable
    g = GraphedMoEBlock(m)
    params = dict(m.named_parameters())
    for step in range(3):
        torch.manual_seed(20 + step)
        x = torch.randn(4, 256, 576, device="cuda").bfloat16()      # leading dims kept
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        for p in params.values():
            p.grad = None
        out_a = g(xa)
        (out_a.float().square().mean() + g.aux_loss).backward()
        got = {n: p.grad.clone() for n, p in params.items()}
        aux_a, counts_a = g.aux_loss.detach().clone(), g.expert_counts.clone()
        for p in params.values():
            p.grad = None
        out_b = m(xb)
        (out_b.float().square().mean() + m.aux_loss).backward()
        assert out_a.shape == x.shape and torch.equal(out_a, out_b)
        assert torch.equal(counts_a.long(), m.expert_counts.long())
        assert abs(float(aux_a) - float(m.aux_loss)) < 1e-6
        assert torch.equal(xa.grad, xb.grad)
        for n, p in params.items():
            assert torch.equal(got[n], p.grad), n
        with torch.no_grad():                    # an optimizer step in place: the graphs see it
            for p in params.values():
                p.add_(0.01 * torch.randn_like(p))
    assert len(g._graphed) == 1
    with torch.no_grad():                        # no autograd: the block's own inference path
        assert g(x).shape == x.shape
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


def test_exploration_noise_runs_inside_the_whole_block_op():
    """Training with router.noise_std > 0 (the opening stretch of the reference's run,
    src/model/router.py:76-77, src/train/train.py:298-300) stays on the whole-block op: the noise is
    drawn in torch and handed to the op, which adds it to the logits in the router kernel and again
    in the router's backward. Against the oracle routed on identical noisy logits: output, balance
    loss, counts and all six gradients; a second call draws fresh noise."""
    T = 2048
    x, m, o = _model_shape_pair(T, train=True, seed=8)
    m.router.noise_std = 0.5
    xc = x.cuda().requires_grad_(True)
    torch.manual_seed(77)
    out = m(xc)
    assert m._whole_block_ok(xc)
    (out.float().square().mean() + m.aux_loss).backward()
    torch.manual_seed(77)                     # the same draw the module made
    noise = torch.randn(T, 76, device="cuda", dtype=torch.float32) * 0.5
    o.logits_override = (_block_logits(m, xc.detach()) + noise).cpu()
    xo = x.clone().requires_grad_(True)
    ref = o(xo)
    (ref.float().square().mean() + o.aux_loss).backward()
    assert torch.equal(m.expert_counts.cpu().long(), o.expert_counts)
    noiseless = O.canonical_topk(_block_logits(m, xc.detach()).cpu(), 6)
    assert not torch.equal(torch.bincount(noiseless.reshape(-1), minlength=76), o.expert_counts)
    assert rel_l2(out.detach().cpu(), ref.detach()) < TOL
    assert abs(float(m.aux_loss) - float(o.aux_loss)) < 1e-4
    for name, a, b in [("dx", xc.grad, xo.grad), ("dW_in", m.W_in.grad, o.W_in.grad),
                       ("dW_out", m.W_out.grad, o.W_out.grad),
                       ("dW_sh_in", m.W_sh_in.grad, o.W_sh_in.grad),
                       ("dW_sh_out", m.W_sh_out.grad, o.W_sh_out.grad),
                       ("d_router", m.router.W.grad, o.router_W.grad)]:
        assert rel_l2(a.cpu(), b) < (2e-2 if name == "d_router" else TOL), name
    with torch.no_grad():
        counts = m.expert_counts.clone()
        m(xc)
        assert not torch.equal(counts, m.expert_counts)      # fresh noise, other routing
        m.eval()                                             # no noise outside training
        a, b = m(xc), m(xc)
        assert rel_l2(a, b) < ATOMIC_TOL
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")


@pytest.mark.parametrize("n_shared,noise_std,T", [(2, 0.0, 2048), (0, 0.0, 1000), (2, 0.5, 300)])
def test_one_call_per_direction_equals_the_stage_sequence(n_shared, noise_std, T):
    """The whole-block op's training form is issued by one call into the library per direction
    (moe_b200_block_fwd / moe_b200_block_bwd, host code over the same stage entry points, three
    streams inside the backward). Against the stage-by-stage sequence from Python on the same
    inputs: the routing plan bit-equal, everything numeric within the atomic combine's ordering
    noise; with and without shared experts, with exploration noise, T off the tile grid; through
    the registered op as well as the autograd node eager calls use."""
    from nanospeaker_b200 import MoEBlock, moe_kernel as MK, kernels
    torch.manual_seed(31 + T)
    m = MoEBlock(576, 76, d_ff=192, top_k=6, n_shared=n_shared, capacity_factor=None)
    with torch.no_grad():
        m.router.W.copy_(torch.randn(576, 76) * 0.02)
        for p_ in (m.W_in, m.W_out) + ((m.W_sh_in, m.W_sh_out) if n_shared else ()):
            p_.copy_(torch.randn_like(p_) * p_.shape[1] ** -0.5)
    m = m.to(torch.bfloat16).cuda().train()
    m.router.noise_std = noise_std
    m.router.logit_bias = torch.randn(76, device="cuda") * 0.27
    x = torch.randn(T, 576, device="cuda").bfloat16()
    assert MK._ONE_CALL
    res = {}
    try:
        for mode in (True, False, "one stream"):
            MK._ONE_CALL = bool(mode)
            MK._DEBUG_ONE_STREAM = mode == "one stream"   # the backward's branches in line
            xc = x.clone().requires_grad_(True)
            for p in m.parameters():
                p.grad = None
            torch.manual_seed(5)                          # the same exploration noise in both runs
            out = m(xc)
            (out.float().square().mean() + m.aux_loss).backward()
            res[mode] = dict(out=out.detach(), aux=m.aux_loss.detach().clone(),
                             counts=m.expert_counts.clone(), dx=xc.grad,
                             **{n: p.grad.clone() for n, p in m.named_parameters()
                                if p.grad is not None})
    finally:
        MK._ONE_CALL, MK._DEBUG_ONE_STREAM = True, False
    for k_ in res[True]:
        if k_ not in ("counts", "aux"):
            assert rel_l2(res["one stream"][k_], res[True][k_]) < ATOMIC_TOL, k_
    a, b = res[True], res[False]
    assert a.keys() == b.keys() and "router.W" in a and ("W_sh_in" in a) == bool(n_shared)
    assert torch.equal(a["counts"], b["counts"])
    assert abs(float(a["aux"]) - float(b["aux"])) < 1e-5
    for k in a:
        if k not in ("counts", "aux"):
            assert rel_l2(a[k], b[k]) < ATOMIC_TOL, k
    # the registered op takes the same path: plan tensors bit-equal with the stage sequence
    cast = lambda t: None if t is None else t.detach()
    args = (x, cast(m.router.W), m.router.logit_bias.float().contiguous(), cast(m.W_in),
            cast(m.W_out), cast(m.W_sh_in), cast(m.W_sh_out), 6, True, True, 0.01, "silu", True,
            None, True, None, False)
    with torch.no_grad():
        one = torch.ops.moe_b200.moe_block(*args)
        MK._ONE_CALL = False
        try:
            seq = torch.ops.moe_b200.moe_block(*args)
        finally:
            MK._ONE_CALL = True
    live = int(one[12].item())
    assert live == int(seq[12].item())
    for i in (2, 10, 11, 13):                              # counts, offsets, counts_all, inv_ids
        assert torch.equal(one[i], seq[i]), i
    assert torch.equal(one[8][:live], seq[8][:live])       # sorted_ids
    assert torch.equal(one[9][: live // 128], seq[9][: live // 128])
    assert torch.equal(one[5], seq[5]) and torch.equal(one[6], seq[6])   # logits, weights
    assert rel_l2(one[0], seq[0]) < ATOMIC_TOL
    kernels.check_status("cuda")


@pytest.mark.parametrize("T", [1, 64, 129, 2048])
def test_one_call_inference_block_equals_the_stage_sequence(T):
    """moe_b200_block_infer (one call per layer of a decode stack) against the same launches issued
    one by one: bit-identical with the deterministic combine, residual included."""
    from nanospeaker_b200 import moe_kernel as MK, kernels
    x, m, _ = _model_shape_pair(T, train=False, seed=T)
    xc = x.cuda()
    wp = MK.pad_router_weight(m.router.W.detach(), xc.dtype)
    args = (wp, None, m.W_in.detach(), m.W_out.detach(), m.W_sh_in.detach(), m.W_sh_out.detach(),
            76, 6, True, "silu")
    assert MK._ONE_CALL
    one = MK.moe_block_inference(xc, *args, residual=xc, combine="store")
    one_atomic = MK.moe_block_inference(xc, *args, residual=None, combine="atomic")
    MK._ONE_CALL = False
    try:
        seq = MK.moe_block_inference(xc, *args, residual=xc, combine="store")
        seq_plain = MK.moe_block_inference(xc, *args, residual=None, combine="store")
    finally:
        MK._ONE_CALL = True
    assert torch.equal(one, seq)
    assert rel_l2(one_atomic, seq_plain) < ATOMIC_TOL
    kernels.check_status("cuda")


def test_global_balance_loss_shares_sum_to_the_loss_of_the_whole_batch():
    """Tokens sharded over two ranks (run one after the other on this GPU; the count exchange is a
    hook that adds the other rank's counts): each rank's aux_loss is its share of the balance loss
    of the concatenated batch, and its gradient with respect to the rank's own tokens is the
    oracle's gradient of that global loss."""
    from nanospeaker_b200 import moe_kernel as MK
    T = 1024
    x, m, o = _model_shape_pair(2 * T, train=True, seed=12)
    shards = [x[:T].cuda(), x[T:].cuda()]
    try:
        local = []
        for xs in shards:                       # pass 1: every rank's own counts
            with torch.no_grad():
                m(xs)
            local.append(m.expert_counts.clone())
        shares, grads = [], []
        for r, xs in enumerate(shards):         # pass 2: with the exchange
            other = local[1 - r]
            MK.set_aux_reduce(lambda c, other=other: c.add_(other.to(c.dtype)))
            xr = xs.clone().requires_grad_(True)
            m(xr)
            shares.append(m.aux_loss.detach().float().cpu())
            m.aux_loss.backward()
            grads.append(xr.grad.float().cpu())
    finally:
        MK.set_aux_reduce(None)
    logits = torch.cat([_block_logits(m, s) for s in shards]).cpu()
    o.logits_override = logits
    xo = x.clone().requires_grad_(True)
    o(xo)
    o.aux_loss.backward()
    assert torch.equal((local[0] + local[1]).cpu().long(), o.expert_counts)
    assert abs(float(shares[0] + shares[1]) - float(o.aux_loss)) < 1e-5
    assert rel_l2(torch.cat(grads), xo.grad.float()) < 2e-2
