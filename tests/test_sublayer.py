"""The FFN sublayer  x + ffn(rmsnorm(x)) : the oracle's restatement against golden vectors produced
by the unmodified reference (RMSNorm + MoEBlock as Block.forward wires them), the closed-form
RMSNorm backward against autograd, and the module's torch fallback on CPU."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import moe_oracle as O


def _oracle_from_golden(g):
    d_model, n_experts, d_ff, top_k, n_shared, tokens = g["meta"].tolist()
    dt = g["x"].dtype
    blk = O.OracleBlock(d_model, n_experts, d_ff, top_k, n_shared).to(dt)
    sub = O.OracleSublayer(blk, float(g["epsilon"])).to(dt)
    with torch.no_grad():
        sub.gamma.copy_(g["gamma"])
        blk.router_W.copy_(g["router_W"])
        blk.W_in.copy_(g["W_in"])
        blk.W_out.copy_(g["W_out"])
        blk.W_sh_in.copy_(g["W_sh_in"])
        blk.W_sh_out.copy_(g["W_sh_out"])
    return sub.train()


@pytest.mark.parametrize("case", ["sublayer_fp32_train", "sublayer_bf16_train"])
def test_oracle_sublayer_matches_reference_golden(case):
    g = load_golden(case)
    sub = _oracle_from_golden(g)
    x = g["x"].clone().requires_grad_(True)
    assert torch.equal(O.rmsnorm(x.detach(), sub.gamma.detach(), sub.eps), g["h"])
    out, aux = sub(x)
    (out.float().square().mean() + aux).backward()
    fp32 = g["x"].dtype == torch.float32
    tol = 1e-6 if fp32 else 1e-2
    assert rel_l2(out.detach(), g["out"]) < tol
    assert abs(float(aux) - float(g["aux_loss"])) < 1e-5
    for got, key in [(x.grad, "grad_x"), (sub.gamma.grad, "grad_gamma"),
                     (sub.block.router_W.grad, "grad_router_W"), (sub.block.W_in.grad, "grad_W_in"),
                     (sub.block.W_out.grad, "grad_W_out"), (sub.block.W_sh_in.grad, "grad_W_sh_in"),
                     (sub.block.W_sh_out.grad, "grad_W_sh_out")]:
        assert rel_l2(got, g[key]) < (tol if fp32 else 2e-2), key


def test_rmsnorm_backward_closed_form_matches_autograd():
    torch.manual_seed(0)
    x = (torch.randn(37, 96, dtype=torch.float64) * 2).requires_grad_(True)
    gamma = (1 + 0.3 * torch.randn(96, dtype=torch.float64)).requires_grad_(True)
    dh = torch.randn(37, 96, dtype=torch.float64)
    O.rmsnorm(x, gamma, 1e-6).backward(dh)
    dx, dgamma = O.rmsnorm_backward(dh.float(), x.detach().float(), gamma.detach().float(), 1e-6)
    assert rel_l2(dx, x.grad.float()) < 1e-5
    assert rel_l2(dgamma, gamma.grad.float()) < 1e-5


def test_module_fallback_on_cpu_matches_golden():
    from nanospeaker_b200 import MoEBlock
    from nanospeaker_b200.sublayer import MoEFFNSublayer
    g = load_golden("sublayer_fp32_train")
    d_model, n_experts, d_ff, top_k, n_shared, tokens = g["meta"].tolist()
    ffn = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                   capacity_factor=None, normalize_weights=True)
    sub = MoEFFNSublayer(ffn, float(g["epsilon"])).train()
    with torch.no_grad():
        sub.norm_gamma.copy_(g["gamma"])
        ffn.router.W.copy_(g["router_W"])
        ffn.W_in.copy_(g["W_in"])
        ffn.W_out.copy_(g["W_out"])
        ffn.W_sh_in.copy_(g["W_sh_in"])
        ffn.W_sh_out.copy_(g["W_sh_out"])
    x = g["x"].clone().requires_grad_(True)
    out, aux = sub(x)
    (out.float().square().mean() + aux).backward()
    assert rel_l2(out.detach(), g["out"]) < 1e-5
    assert rel_l2(x.grad, g["grad_x"]) < 1e-5
    assert rel_l2(sub.norm_gamma.grad, g["grad_gamma"]) < 1e-5
