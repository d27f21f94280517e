"""Host-side behaviour of the drop-in module, on CPU: constructor validation, parameter layout,
the eager ragged path against the dense cross-check and against the oracle, and the gates that
decide when the CUDA kernels run. Mirrors what tests/test_moe.py of the reference pins."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import moe_oracle as O


def make(**kw):
    from nanospeaker_b200 import MoEBlock
    args = dict(d_model=32, n_experts=8, d_ff=64, fused=False, capacity_factor=None)
    args.update(kw)
    return MoEBlock(**args)


@pytest.mark.parametrize("top_k", [1, 2, 8])
@pytest.mark.parametrize("n_shared", [0, 2])
def test_sparse_equals_dense_in_fp64(top_k, n_shared):
    m = make(top_k=top_k, n_shared=n_shared).double()
    x = torch.randn(3, 17, 32, dtype=torch.double)
    with torch.no_grad():
        assert torch.allclose(m(x), m.dense_forward(x), atol=1e-12)
    assert int(m.expert_counts.sum()) == 3 * 17 * top_k


def test_matches_reference_golden_on_cpu():
    from nanospeaker_b200 import MoEBlock
    g = load_golden("block_fp32_train")
    d_model, n_experts, d_ff, top_k, n_shared, *_ = g["meta"].tolist()
    m = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                 capacity_factor=None)
    with torch.no_grad():
        m.router.W.copy_(g["router_W"]); m.W_in.copy_(g["W_in"]); m.W_out.copy_(g["W_out"])
        m.W_sh_in.copy_(g["W_sh_in"]); m.W_sh_out.copy_(g["W_sh_out"])
    m.train(True)
    x = g["x"].clone().requires_grad_(True)
    out = m(x)
    (out.float().square().mean() + m.aux_loss).backward()
    assert torch.equal(out, g["out"])
    assert torch.equal(m.expert_counts, g["plan_counts"])
    # (the gradient's k contributions per token are summed in this module's own order: equal to
    # fp32 rounding, not bit for bit; the oracle is what is pinned bitwise)
    assert rel_l2(x.grad, g["grad_x"]) < 1e-6 and rel_l2(m.W_in.grad, g["grad_W_in"]) < 1e-6
    assert rel_l2(m.router.W.grad, g["grad_router_W"]) < 1e-5
    experts, order, token_idx, counts = m._plan(g["topk_idx"])
    assert torch.equal(order, g["plan_order"]) and torch.equal(token_idx, g["plan_token_idx"])


def test_constructor_validation():
    with pytest.raises(ValueError): make(n_shared=-1)
    with pytest.raises(ValueError): make(capacity_factor=0)
    with pytest.raises(ValueError): make(top_k=9)
    with pytest.raises(ValueError): make(n_experts=0)
    with pytest.raises(ValueError): make(d_ff=1)
    with pytest.raises(ValueError): make(activation="nope")
    with pytest.raises(ValueError): make()(torch.randn(4, 31))
    assert make(activation="SiLU").activation == "silu"


def test_parameter_layout_and_state_dict():
    m = make(d_model=576, n_experts=76, d_ff=192, top_k=6, n_shared=2)
    assert m.d_hidden == 128
    assert m.W_in.shape == (76, 576, 256) and m.W_out.shape == (76, 128, 576)
    assert m.W_sh_in.shape == (2, 576, 256) and m.W_sh_out.shape == (2, 128, 576)
    assert m.router.W.shape == (576, 76)
    assert set(m.state_dict()) == {"router.W", "W_in", "W_out", "W_sh_in", "W_sh_out"}
    b = make(bias=True, n_shared=1)
    assert {"b_in", "b_out", "b_sh_in", "b_sh_out"} <= set(b.state_dict())
    assert "edges" not in m.state_dict()


def test_kernel_gate_on_cpu_and_auto_capacity():
    from nanospeaker_b200 import AUTO_CAPACITY, kernel_supported, shapes_supported
    m = make(capacity_factor="auto")
    assert m.capacity_factor == AUTO_CAPACITY           # no kernels on CPU -> padded fallback cap
    assert not m._use_kernel(torch.zeros(1, 32))
    assert not kernel_supported(torch.zeros(1))
    assert shapes_supported(576, 128, 76, 6, 2)
    assert not shapes_supported(32, 42, 8, 2)           # d_hidden the tiles do not cover
    assert not shapes_supported(576, 128, 300, 6)
    assert make(activation=lambda t: t)._kernel_act is None


def test_router_contract():
    m = make(top_k=3)
    m.eval()
    x = torch.randn(40, 32)
    w, idx, probs = m.router(x)
    assert probs is None and idx.dtype == torch.int64
    assert torch.allclose(w.sum(-1), torch.ones(40), atol=1e-6)
    m.train()
    w2, idx2, probs2 = m.router(x)
    assert probs2 is not None and torch.equal(idx, idx2) and torch.allclose(w, w2, atol=1e-6)
    m(x)
    assert m.aux_loss > 0
    m.eval(); m(x)
    assert float(m.aux_loss) == 0.0
    m.train(); m.router.noise_std = 1.0
    a, b = m.router(x)[1], m.router(x)[1]
    assert not torch.equal(a, b)


def test_fused_forward_rejects_cpu_and_unknown_activations():
    from nanospeaker_b200 import fused_moe_forward
    m = make(d_model=64, d_ff=192)
    x = torch.randn(4, 64)
    w, idx, _ = m.router(x)
    with pytest.raises(ValueError, match="no kernel"):
        fused_moe_forward(x, m.W_in, m.W_out, w, idx, None, None, "softplus")
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_moe_forward(x, m.W_in, m.W_out, w, idx, None, None, "silu")


def test_eager_path_equals_oracle_block_bf16():
    g = load_golden("block_bf16_train")
    from nanospeaker_b200 import MoEBlock
    d_model, n_experts, d_ff, top_k, n_shared, *_ = g["meta"].tolist()
    m = MoEBlock(d_model, n_experts, d_ff=d_ff, top_k=top_k, n_shared=n_shared,
                 capacity_factor=None).to(torch.bfloat16)
    with torch.no_grad():
        m.router.W.copy_(g["router_W"]); m.W_in.copy_(g["W_in"]); m.W_out.copy_(g["W_out"])
        m.W_sh_in.copy_(g["W_sh_in"]); m.W_sh_out.copy_(g["W_sh_out"])
    m.train(True)
    out = m(g["x"])
    assert torch.equal(out, g["out"])
