"""Muon's batched Newton-Schulz on the stacked expert weights (nanospeaker_b200/muon.py) against the
oracle's restatement of src/train/optim.py:27-105 and the golden the reference produced."""
import pytest
import torch

from conftest import rel_l2
from oracle import moe_oracle as O
from test_oracle import _muon_golden


def test_torch_path_matches_the_reference_golden_on_cpu():
    from nanospeaker_b200.muon import Muon, newton_schulz5
    g, t = _muon_golden()
    for tag, _ in O.MUON_SHAPES:
        assert torch.equal(newton_schulz5(t[f"g_{tag}"]), g[f"ns_{tag}"]), tag
        w = torch.nn.Parameter(t[f"w_{tag}"].clone())
        opt = Muon([w], lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5)
        for step in range(2):
            w.grad = t[f"grad_{tag}_{step}"].clone()
            opt.step()
        assert torch.equal(w.detach().reshape(-1)[::7], g[f"w_{tag}_after"]), tag
        assert opt.update_norm_ratio() > 0
    one = newton_schulz5(t["g_out"][0])            # a single matrix
    assert torch.equal(one, g["ns_out"][0])


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(78, 576, 256), (78, 128, 576), (3, 256, 576), (2, 128, 256)])
def test_kernel_newton_schulz_matches_the_oracle(shape):
    """The stacked weight-gradient shapes of the block (dW_in and dW_sh_in together: 78 x [576, 256],
    dW_out: 78 x [128, 576]) through the grouped tcgen05 GEMMs: against the oracle's bf16 iteration
    and the fp32 iteration. Five bf16 Newton-Schulz steps are noisy by themselves: the reference's
    own bf16 result sits 2.5e-2 (rel-L2) from the fp32 iteration on these inputs, and the kernels
    round in fewer places (one rounding per a X + b Y), so the bars are 4e-2 against the bf16
    oracle and 3e-2 against fp32; plus the defining property (singular values near 1)."""
    from nanospeaker_b200 import kernels
    from nanospeaker_b200.muon import _kernel_ok, newton_schulz5
    torch.manual_seed(5)
    g = (torch.randn(*shape) * 0.02).bfloat16()
    assert _kernel_ok(g.cuda())
    before = kernels.LAUNCHES
    got = newton_schulz5(g.cuda()).cpu()
    assert kernels.LAUNCHES - before >= 2 + 5 * 5        # no per-expert loop: 5 launches an iteration
    want = O.newton_schulz5(g)
    assert got.shape == g.shape and got.dtype == torch.bfloat16
    assert rel_l2(got, want) < 4e-2
    # fp32 iteration on the same bf16 input
    x = g.float()
    tall = shape[1] > shape[2]
    x = x.mT if tall else x
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(5):
        a = x @ x.mT
        x = 3.4445 * x + (-4.7750 * a + 2.0315 * (a @ a)) @ x
    x = x.mT if tall else x
    assert rel_l2(got, x) < 3e-2
    sv = torch.linalg.svdvals(got[0].float())
    assert 0.6 < float(sv.min()) and float(sv.max()) < 1.3
    kernels.check_status("cuda")


@pytest.mark.gpu
def test_muon_step_on_the_blocks_gradients():
    """One optimizer step on a block's stacked expert weights with the gradients its backward left,
    on the GPU (kernel Newton-Schulz) against the oracle's step on the CPU."""
    from nanospeaker_b200 import MoEBlock
    from nanospeaker_b200.muon import Muon
    torch.manual_seed(1)
    m = MoEBlock(576, 8, d_ff=192, top_k=2, n_shared=1, capacity_factor=None)
    m = m.to(torch.bfloat16).cuda()
    x = torch.randn(512, 576, device="cuda").bfloat16()
    (m(x).float().square().mean() + m.aux_loss).backward()
    params = [m.W_in, m.W_out, m.W_sh_in, m.W_sh_out]
    ref = [(p.detach().cpu().clone(), p.grad.cpu().clone()) for p in params]
    opt = Muon(params, lr=0.02)
    opt.step()
    for p, (w, gr) in zip(params, ref):
        decayed = w.float() * (1 - 0.02 * 0.1)
        delta = O.muon_step(w, gr, torch.zeros_like(w))          # updates w in place
        # (these gradients have rank <= rows per expert < 256: the iteration amplifies rounding
        # noise in the near-null directions, so the applied step is compared loosely)
        assert rel_l2(p.detach().cpu(), w) < 1e-2                # the updated weights
        assert rel_l2(p.detach().cpu().float() - decayed, delta.float()) < 0.2    # the applied step
    assert 0 < opt.update_norm_ratio() < 1
