"""The CPU oracle against the golden vectors produced by the unmodified reference
(tests/golden/make_golden.py), and against the reference imported live when a checkout exists."""
import os
import sys

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import moe_oracle as O

# checkout of the reference project, where one is named (live cross-checks are skipped otherwise)
REF = os.environ.get("NANOSPEAKER_REF", "")
BLOCK_CASES = ["block_fp32_eval", "block_fp32_train", "block_bf16_train", "block_bf16_eval_gelu"]


def _block_from_golden(g):
    d_model, n_experts, d_ff, top_k, n_shared, tokens, train, normalize = g["meta"].tolist()
    m = O.OracleBlock(d_model, n_experts, d_ff, top_k, n_shared, activation=g["activation"],
                      normalize_weights=bool(normalize))
    dt = g["x"].dtype
    m = m.to(dt)
    with torch.no_grad():
        m.router_W.copy_(g["router_W"])
        m.W_in.copy_(g["W_in"])
        m.W_out.copy_(g["W_out"])
        if n_shared:
            m.W_sh_in.copy_(g["W_sh_in"])
            m.W_sh_out.copy_(g["W_sh_out"])
    m.train(bool(train))
    return m


@pytest.mark.parametrize("case", BLOCK_CASES)
def test_router_and_plan_match_golden(case):
    g = load_golden(case)
    m = _block_from_golden(g)
    logits, w, idx, probs = m.route(g["x"])
    assert torch.equal(logits, g["logits"])
    assert torch.equal(idx, g["topk_idx"])
    assert torch.equal(w, g["topk_w"])
    if "probs" in g:
        assert torch.equal(probs, g["probs"])
    experts, order, token_idx, counts = O.plan(idx, m.n_experts)
    assert torch.equal(experts, g["plan_experts"])
    assert torch.equal(order, g["plan_order"])
    assert torch.equal(token_idx, g["plan_token_idx"])
    assert torch.equal(counts, g["plan_counts"])
    # the canonical tie rule picks the same experts wherever torch.topk had no freedom, and the
    # same values everywhere
    tied = O.tied_rows(logits.detach(), m.top_k)
    canon = O.canonical_topk(logits.detach(), m.top_k)
    assert torch.equal(canon[~tied], idx[~tied])
    assert torch.equal(logits.detach().gather(1, canon), logits.detach().gather(1, idx))


@pytest.mark.parametrize("case", BLOCK_CASES)
def test_block_output_matches_golden(case):
    g = load_golden(case)
    m = _block_from_golden(g)
    with torch.no_grad():
        out = m(g["x"])
    assert torch.equal(out, g["out"]), rel_l2(out, g["out"])
    assert torch.allclose(m.aux_loss.float(), g["aux_loss"], atol=1e-7)
    if "dense_out" in g:
        w, idx = g["topk_w"], g["topk_idx"]
        dense = O.dense_forward(g["x"], m.W_in, m.W_out, w, idx, m.activation, m.W_sh_in,
                                m.W_sh_out)
        assert torch.equal(dense, g["dense_out"])


@pytest.mark.parametrize("case", ["block_fp32_train", "block_bf16_train"])
def test_block_gradients_match_golden(case):
    g = load_golden(case)
    m = _block_from_golden(g)
    x = g["x"].clone().requires_grad_(True)
    out = m(x)
    (out.float().square().mean() + m.aux_loss).backward()
    pairs = [(x.grad, "grad_x"), (m.router_W.grad, "grad_router_W"), (m.W_in.grad, "grad_W_in"),
             (m.W_out.grad, "grad_W_out"), (m.W_sh_in.grad, "grad_W_sh_in"),
             (m.W_sh_out.grad, "grad_W_sh_out")]
    for got, key in pairs:
        assert torch.equal(got, g[key]), (key, rel_l2(got, g[key]))


def test_closed_form_backward_matches_golden_fp32():
    """experts_backward / router_backward (the formulas the CUDA kernels implement) reproduce the
    reference's autograd gradients."""
    g = load_golden("block_fp32_train")
    m = _block_from_golden(g)
    x = g["x"]
    T, D = x.shape
    logits, w, idx, probs = m.route(x)
    out = g["out"]
    d_out = 2.0 * out / out.numel()
    dx, dw_in, dw_out, dtw, dsi, dso = O.experts_backward(
        d_out, x, m.W_in.detach(), m.W_out.detach(), w.detach(), idx, "silu",
        m.W_sh_in.detach(), m.W_sh_out.detach())
    assert rel_l2(dw_in, g["grad_W_in"]) < 1e-5
    assert rel_l2(dw_out, g["grad_W_out"]) < 1e-5
    assert rel_l2(dsi, g["grad_W_sh_in"]) < 1e-5
    assert rel_l2(dso, g["grad_W_sh_out"]) < 1e-5
    counts = g["plan_counts"]
    f = counts.float() / counts.sum()
    d_probs = (m.aux_loss_coef * m.n_experts * f / T).expand(T, -1)
    dl = O.router_backward(logits.detach(), idx, dtw, d_probs, True, True)
    d_router = x.t() @ dl
    assert rel_l2(d_router, g["grad_router_W"]) < 1e-5
    dx_total = dx + dl @ m.router_W.detach().t()
    assert rel_l2(dx_total, g["grad_x"]) < 1e-5


@pytest.mark.parametrize("case", ["routing_e76_k6_fp32", "routing_e76_k6_bf16"])
def test_routing_at_model_width_matches_golden(case):
    g = load_golden(case)
    tokens, n_experts, top_k, _ = g["meta"].tolist()
    logits, ref_idx = g["logits"], g["topk_idx"]
    canon = O.canonical_topk(logits, top_k)
    tied = O.tied_rows(logits, top_k)
    # bit-equal wherever torch.topk had no freedom
    assert torch.equal(canon[~tied], ref_idx[~tied])
    # on tied rows: the same VALUES are selected, in the same order
    assert torch.equal(logits.gather(1, canon), logits.gather(1, ref_idx))
    if case.endswith("bf16"):
        assert tied.any(), "bf16-derived logits are expected to produce exact ties"
    _, order, token_idx, counts = O.plan(ref_idx, n_experts)
    assert torch.equal(order, g["plan_order"])
    assert torch.equal(token_idx, g["plan_token_idx"])
    assert torch.equal(counts, g["plan_counts"])


def test_padded_dispatch_layout_invariants():
    """The invariants the reference asserts on its dispatch op (tests/test_moe_kernel.py:197-216),
    on the oracle's padded layout, plus stability."""
    idx = torch.randint(0, 8, (50, 2))
    sids, eids, offs, counts, npp, inv = O.dispatch(idx, 8)
    m = idx.numel()
    assert sids.numel() == O.l_cap(m, 8)
    assert torch.equal(sids[inv.long()], torch.arange(m, dtype=torch.int32))
    assert torch.equal(counts.long(), torch.bincount(idx.reshape(-1), minlength=8))
    assert int(npp) == int(((counts + 127) // 128 * 128).sum())
    flat = idx.reshape(-1)
    for e in range(8):
        run = sids[int(offs[e]): int(offs[e]) + int(counts[e])].long()
        assert (flat[run] == e).all()
        assert (run[1:] > run[:-1]).all()          # stable: ascending pair id inside a run
        assert (sids[int(offs[e]) + int(counts[e]): int(offs[e + 1])] == m).all()
    _, order, _, _ = O.plan(idx, 8)
    assert torch.equal(sids[sids < m].long(), order)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src", "model")),
                    reason="no checkout of the reference on this machine")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("train", [False, True])
def test_oracle_matches_live_reference_at_model_shape(dtype, train):
    """nanoSpeaker's real block shape (E=76, k=6, D=576, d_ff=192, S=2) on fresh random inputs:
    the oracle and the imported reference agree bit for bit, forward and backward."""
    sys.path.insert(0, REF)
    try:
        from src.model.moe import MoEBlock as RefBlock
    finally:
        sys.path.remove(REF)
    torch.manual_seed(11)
    ref = RefBlock(576, 76, d_ff=192, top_k=6, n_shared=2, capacity_factor=None, fused=False,
                   kernel=False).to(dtype)
    ref.train(train)
    m = O.OracleBlock(576, 76, 192, 6, 2).to(dtype)
    m.train(train)
    with torch.no_grad():
        m.router_W.copy_(ref.router.W)
        m.W_in.copy_(ref.W_in)
        m.W_out.copy_(ref.W_out)
        m.W_sh_in.copy_(ref.W_sh_in)
        m.W_sh_out.copy_(ref.W_sh_out)
    x = torch.randn(256, 576).to(dtype)
    xa, xb = x.clone().requires_grad_(train), x.clone().requires_grad_(train)
    with torch.set_grad_enabled(train):
        oa, ob = ref(xa), m(xb)
    assert torch.equal(oa, ob)
    assert torch.equal(ref.expert_counts, m.expert_counts)
    if train:
        (oa.float().square().mean() + ref.aux_loss).backward()
        (ob.float().square().mean() + m.aux_loss).backward()
        assert torch.equal(xa.grad, xb.grad)
        assert torch.equal(ref.W_in.grad, m.W_in.grad)
        assert torch.equal(ref.W_out.grad, m.W_out.grad)
        assert torch.equal(ref.router.W.grad, m.router_W.grad)
        assert torch.equal(ref.W_sh_in.grad, m.W_sh_in.grad)


@pytest.mark.parametrize("case", ["block_fp32_train_bias", "block_bf16_train_bias"])
def test_expert_biases_match_golden(case):
    """experts_forward with per-expert biases (src/model/moe.py:295-305) on the reference's own
    routing: the reference's output, and through autograd its bias and weight gradients."""
    g = load_golden(case)
    leaf = lambda k: g[k].clone().requires_grad_(True)
    names = ("x", "W_in", "W_out", "W_sh_in", "W_sh_out", "b_in", "b_out", "b_sh_in", "b_sh_out")
    p = {k: leaf(k) for k in names}
    assert float(g["b_sh_in"].abs().sum()) > 0 and float(g["b_sh_out"].abs().sum()) > 0
    out = O.experts_forward(p["x"], p["W_in"], p["W_out"], g["topk_w"], g["topk_idx"], "silu",
                            p["W_sh_in"], p["W_sh_out"], p["b_in"], p["b_out"], p["b_sh_in"],
                            p["b_sh_out"])
    fp32 = g["x"].dtype == torch.float32
    assert rel_l2(out, g["out"]) < (1e-6 if fp32 else 1e-2)
    out.float().square().mean().backward()       # the balance loss does not reach these gradients
    for k in names[1:]:
        assert rel_l2(p[k].grad, g["grad_" + k]) < (1e-5 if fp32 else 2e-2), k


def real_shape_oracle(g):
    """The oracle block at nanoSpeaker's real shape with the weights the real-shape golden was
    generated from (they are re-drawn from the stored seed; the fingerprint says whether this
    torch build draws the same numbers)."""
    D, E, d_ff, k, S, tokens, seed, stride = g["meta"].tolist()
    w = O.seeded_block_weights(seed, D, E, 2 * d_ff // 3, S)
    fp = torch.tensor([int(w[key].view(torch.int16).long().sum()) for key in
                       ("router_W", "W_in", "W_out", "W_sh_in", "W_sh_out")], dtype=torch.int64)
    if not torch.equal(fp, g["weights_fingerprint"]):
        pytest.skip("this torch build draws other random numbers than the golden's generator")
    o = O.OracleBlock(D, E, d_ff, k, S).to(torch.bfloat16)
    with torch.no_grad():
        o.router_W.copy_(w["router_W"])
        for key in ("W_in", "W_out", "W_sh_in", "W_sh_out"):
            getattr(o, key).copy_(w[key])
    return o.train(), w, stride


def test_oracle_matches_the_reference_at_nanospeakers_real_shape():
    """d_model 576, 76 + 2 experts, top-6, bf16, training mode, 256 tokens: the reference's output,
    balance loss and gradients (golden generated by the unmodified reference), bit for bit."""
    g = load_golden("block_real_shape_bf16_train")
    o, _, stride = real_shape_oracle(g)
    x = g["x"].clone().requires_grad_(True)
    logits, w, idx, probs = o.route(x)
    assert torch.equal(logits.detach(), g["logits"]) and torch.equal(idx, g["topk_idx"])
    assert torch.equal(w.detach(), g["topk_w"])
    # every token's selected set is the same under the canonical tie rule: results cannot depend
    # on how ties are broken
    canon = O.canonical_topk(logits.detach(), o.top_k)
    assert torch.equal(canon.sort(1).values, idx.sort(1).values)
    out = o(x)
    assert torch.equal(out.detach(), g["out"])
    assert torch.equal(o.expert_counts, g["plan_counts"])
    assert float(o.aux_loss) == float(g["aux_loss"])
    (out.float().square().mean() + o.aux_loss).backward()
    assert torch.equal(x.grad, g["grad_x"])
    assert torch.equal(o.router_W.grad, g["grad_router_W"])
    assert torch.equal(o.W_sh_in.grad, g["grad_W_sh_in"])
    assert torch.equal(o.W_sh_out.grad, g["grad_W_sh_out"])
    for key in ("W_in", "W_out"):
        grad = getattr(o, key).grad
        assert torch.equal(grad.reshape(-1)[::stride], g[f"grad_{key}_strided"]), key
        assert torch.allclose(grad.float().flatten(1).norm(dim=1), g[f"grad_{key}_norms"])


def _muon_golden():
    g = load_golden("muon_newton_schulz")
    t = O.seeded_muon_inputs()
    fp = torch.tensor([int(v.view(torch.int16).long().sum()) for v in t.values()], dtype=torch.int64)
    if not torch.equal(fp, g["fingerprint"]):
        pytest.skip("this torch build draws other random numbers than the golden's generator")
    return g, t


def test_newton_schulz_and_muon_step_match_the_reference():
    """oracle.newton_schulz5 / muon_step against the reference's zeropower_via_newtonschulz5 and two
    steps of its Muon optimizer (golden from src/train/optim.py), bit for bit."""
    g, t = _muon_golden()
    for tag, _ in O.MUON_SHAPES:
        assert torch.equal(O.newton_schulz5(t[f"g_{tag}"]), g[f"ns_{tag}"]), tag
        w, buf = t[f"w_{tag}"].clone(), torch.zeros_like(t[f"w_{tag}"])
        for step in range(2):
            O.muon_step(w, t[f"grad_{tag}_{step}"], buf)
        assert torch.equal(w.reshape(-1)[::7], g[f"w_{tag}_after"]), tag
        # the orthogonal factor: singular values pulled towards 1
        sv = torch.linalg.svdvals(g[f"ns_{tag}"][0].float())
        assert 0.6 < float(sv.min()) and float(sv.max()) < 1.3
