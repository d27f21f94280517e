"""GPU parity of the fused FFN sublayer (RMSNorm kernel -> whole-block op with the residual in its
combine -> block backward -> RMSNorm backward with the residual gradient folded in) against the
reference's golden vectors and, at nanoSpeaker's shape, against the CPU oracle."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2


def test_rmsnorm_kernels_against_the_closed_form():
    from nanospeaker_b200 import kernels as K
    torch.manual_seed(3)
    for T, D in ((1000, 576), (7, 64), (300, 2048)):
        x = (torch.randn(T, D) * 1.5).bfloat16()
        gamma = (1 + 0.2 * torch.randn(D)).bfloat16()
        dh = torch.randn(T, D).bfloat16()
        add = torch.randn(T, D).bfloat16()
        h, rstd = K.rmsnorm(x.cuda(), gamma.cuda(), 1e-6)
        ref_h = O.rmsnorm(x.float(), gamma.float(), 1e-6)
        assert rel_l2(h.cpu(), ref_h) < 5e-3
        ref_r = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        assert torch.allclose(rstd.cpu(), ref_r, rtol=1e-5)
        dx, dgamma = K.rmsnorm_bwd(dh.cuda(), x.cuda(), rstd, gamma.cuda(), add=add.cuda())
        ref_dx, ref_dg = O.rmsnorm_backward(dh, x, gamma, 1e-6)
        assert rel_l2(dx.cpu(), ref_dx + add.float()) < 5e-3
        assert rel_l2(dgamma.cpu(), ref_dg) < 1e-4
        dx0, _ = K.rmsnorm_bwd(dh.cuda(), x.cuda(), rstd, gamma.cuda())
        assert rel_l2(dx0.cpu(), ref_dx) < 5e-3
    K.check_status("cuda")


def test_fused_sublayer_matches_reference_golden():
    from nanospeaker_b200 import MoEBlock
    from nanospeaker_b200.sublayer import MoEFFNSublayer
    g = load_golden("sublayer_bf16_train")
    d_model, n_experts, d_ff, top_k, n_shared, tokens = g["meta"].tolist()
    ffn = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                   capacity_factor=None, normalize_weights=True)
    sub = MoEFFNSublayer(ffn, float(g["epsilon"])).to(torch.bfloat16)
    with torch.no_grad():
        sub.norm_gamma.copy_(g["gamma"])
        ffn.router.W.copy_(g["router_W"])
        ffn.W_in.copy_(g["W_in"])
        ffn.W_out.copy_(g["W_out"])
        ffn.W_sh_in.copy_(g["W_sh_in"])
        ffn.W_sh_out.copy_(g["W_sh_out"])
    sub = sub.cuda().train()
    x = g["x"].cuda().requires_grad_(True)
    assert sub._fused_ok(x), "fused path was not taken"
    out, aux = sub(x)
    (out.float().square().mean() + aux).backward()
    assert rel_l2(out.detach().cpu(), g["out"]) < TOL
    assert abs(float(aux) - float(g["aux_loss"])) < 1e-4
    for got, key in [(x.grad, "grad_x"), (sub.norm_gamma.grad, "grad_gamma"),
                     (ffn.W_in.grad, "grad_W_in"), (ffn.W_out.grad, "grad_W_out"),
                     (ffn.W_sh_in.grad, "grad_W_sh_in"), (ffn.W_sh_out.grad, "grad_W_sh_out"),
                     (ffn.router.W.grad, "grad_router_W")]:
        assert rel_l2(got.cpu(), g[key]) < (2e-2 if key in ("grad_router_W", "grad_gamma") else TOL), key


def test_fused_sublayer_equals_its_unfused_composition_at_model_shape():
    """x + block(rmsnorm(x)) through the fused node against the same three steps through separate
    autograd nodes (torch rms_norm, the block module, a torch add) on identical inputs."""
    from nanospeaker_b200 import MoEBlock
    from nanospeaker_b200.sublayer import MoEFFNSublayer
    torch.manual_seed(4)
    D, E, k, S, T = 576, 76, 6, 2, 4096
    ffn = MoEBlock(D, E, d_ff=192, top_k=k, n_shared=S, capacity_factor=None)
    with torch.no_grad():
        ffn.router.W.copy_(torch.randn(D, E) * 0.02)
        ffn.W_in.copy_(torch.randn(E, D, 256) * D ** -0.5)
        ffn.W_out.copy_(torch.randn(E, 128, D) * 128 ** -0.5)
        ffn.W_sh_in.copy_(torch.randn(S, D, 256) * D ** -0.5)
        ffn.W_sh_out.copy_(torch.randn(S, 128, D) * 128 ** -0.5)
    sub = MoEFFNSublayer(ffn).to(torch.bfloat16).cuda().train()
    with torch.no_grad():
        sub.norm_gamma.copy_(1 + 0.1 * torch.randn(D))
    x = (torch.randn(T, D) * 2).bfloat16().cuda()
    gout = torch.randn(T, D).bfloat16().cuda()

    xa = x.clone().requires_grad_(True)
    out, aux = sub(xa)
    torch.autograd.backward([out, aux], [gout, torch.ones((), device="cuda")])
    fused = {n: p.grad.clone() for n, p in sub.named_parameters()}
    for p in sub.parameters():
        p.grad = None

    xb = x.clone().requires_grad_(True)
    h = torch.nn.functional.rms_norm(xb, (D,), sub.norm_gamma, sub.epsilon)
    ref = xb + ffn(h)
    torch.autograd.backward([ref, ffn.aux_loss], [gout, torch.ones((), device="cuda")])
    assert rel_l2(out.detach(), ref.detach().float()) < TOL
    assert rel_l2(xa.grad, xb.grad.float()) < TOL
    for n, p in sub.named_parameters():
        assert rel_l2(fused[n], p.grad.float()) < 2e-2, n
    from nanospeaker_b200 import kernels
    kernels.check_status("cuda")
