"""GPU parity of the integer / fp32 routing kernels against the CPU oracle: bit-exact expert
selection (given identical fp32 logits) and bit-exact dispatch plan. Calls go through the C ABI."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def K():
    from nanospeaker_b200 import kernels
    return kernels


SPELLINGS = [(True, True), (True, False), (False, True), (False, False)]  # (normalize, full)


@pytest.mark.parametrize("case", ["routing_e76_k6_fp32", "routing_e76_k6_bf16"])
@pytest.mark.parametrize("normalize,full", SPELLINGS)
def test_router_topk_golden(case, normalize, full):
    g = load_golden(case)
    _, n_experts, top_k, _ = g["meta"].tolist()
    logits = g["logits"]
    w, idx, probs = K().router_topk(logits.cuda(), top_k, normalize, full, full)
    idx, w = idx.cpu(), w.cpu()
    canon = O.canonical_topk(logits, top_k)
    assert torch.equal(idx, canon)                       # bit-exact under the stated tie rule
    tied = O.tied_rows(logits, top_k)
    assert torch.equal(idx[~tied], g["topk_idx"][~tied])  # == torch.topk of the reference run
    assert torch.equal(logits.gather(1, idx), logits.gather(1, g["topk_idx"]))
    ref_w, _, ref_p = O.router_select(logits, top_k, normalize, full, idx=canon)
    assert (w - ref_w).abs().max() < 1e-6                # fp32 tolerance: 1e-6 absolute
    if full:
        assert (probs.cpu() - ref_p).abs().max() < 1e-6


@pytest.mark.parametrize("T,E,k", [(1, 1, 1), (3, 8, 8), (257, 200, 16), (64, 256, 6), (777, 5, 1)])
@pytest.mark.parametrize("normalize,full", SPELLINGS)
def test_router_topk_shapes_and_backward(T, E, k, normalize, full):
    logits = torch.randn(T, E) * 2
    w, idx, probs = K().router_topk(logits.cuda(), k, normalize, full, full)
    canon = O.canonical_topk(logits, k)
    assert torch.equal(idx.cpu(), canon)
    ref_w, _, _ = O.router_select(logits, k, normalize, full, idx=canon)
    assert (w.cpu() - ref_w).abs().max() < 1e-6
    d_w = torch.randn(T, k)
    d_p = torch.randn(T, E) * 0.1 if full else None
    dl = K().router_topk_bwd(logits.cuda(), idx, d_w.cuda(), None if d_p is None else d_p.cuda(),
                             normalize, full).cpu()
    ref = O.router_backward(logits, canon, d_w, d_p, normalize, full)
    assert (dl - ref).abs().max() < 2e-6 * max(1.0, float(ref.abs().max()))


def test_router_ties_go_to_the_lowest_index():
    logits = torch.zeros(6, 76)
    logits[5, 0] = float("nan")
    logits[1, 40] = 1.0
    logits[2] = float("-inf")
    logits[3, 7] = float("nan")         # torch orders NaN above everything
    logits[4, ::2] = -0.0               # -0.0 ties with +0.0
    _, idx, _ = K().router_topk(logits.cuda(), 6, True, False, False)
    idx = idx.cpu()
    assert idx[0].tolist() == [0, 1, 2, 3, 4, 5]
    assert idx[1].tolist() == [40, 0, 1, 2, 3, 4]
    assert idx[2].tolist() == [0, 1, 2, 3, 4, 5]
    assert idx[3].tolist() == [7, 0, 1, 2, 3, 4]
    assert idx[4].tolist() == [0, 1, 2, 3, 4, 5]
    assert idx[5].tolist() == [0, 1, 2, 3, 4, 5]


def _check_dispatch(idx, E):
    got = [t.cpu() for t in K().dispatch(idx.cuda(), E)]
    K().check_status("cuda")
    ref = O.dispatch(idx, E)
    names = ["sorted_ids", "expert_ids", "pad_offsets", "counts", "n_post_pad", "inv_ids"]
    live_tiles = int(ref[4]) // 128
    for name, a, b in zip(names, got, ref):
        if name == "expert_ids":
            a, b = a[:live_tiles], b[:live_tiles]
        assert a.dtype == torch.int32 and torch.equal(a, b), name
    m = idx.numel()
    _, order, token_idx, counts = O.plan(idx, E)
    sids = got[0]
    assert torch.equal(sids[sids < m].long(), order)            # == MoEBlock._plan's permutation
    assert torch.equal(sids[sids < m].long() // idx.shape[1], token_idx)


@pytest.mark.parametrize("T,E,k", [(50, 8, 2), (1, 8, 1), (3, 8, 8), (127, 8, 2), (128, 8, 2),
                                   (129, 8, 2), (4096, 76, 6), (5000, 256, 16), (2, 200, 3)])
def test_dispatch_matches_stable_sort(T, E, k):
    logits = torch.randn(T, E)
    _check_dispatch(logits.topk(k, -1).indices, E)


def test_dispatch_collapsed_router_and_empty_experts():
    """Every token on the same experts: most runs empty, one long ragged one
    (the case of tests/test_moe_kernel.py:104-110)."""
    _check_dispatch(torch.zeros(200, 1, dtype=torch.long), 8)
    _check_dispatch(torch.tensor([[7, 3]]).repeat(1000, 1), 8)
    idx = torch.randint(0, 4, (600, 2)) * 19          # only experts 0, 19, 38, 57 of 76
    _check_dispatch(idx, 76)


def test_dispatch_model_scale_skewed():
    """BASELINE config 2's size (T=16384, E=76, k=6) with a skewed router."""
    torch.manual_seed(1)
    logits = torch.randn(16384, 76) * 0.5 + torch.randn(76) * 1.5
    _check_dispatch(logits.topk(6, -1).indices, 76)


def test_dispatch_handles_no_pairs():
    sids, eids, offs, counts, npp, inv = K().dispatch(
        torch.zeros(0, 2, dtype=torch.long, device="cuda"), 8)
    assert sids.numel() == 0 and int(npp) == 0 and int(counts.sum()) == 0 and inv.numel() == 0
    assert offs.tolist() == [0] * 9


def test_dispatch_flags_out_of_range_expert():
    idx = torch.tensor([[0, 9]], device="cuda")
    K().dispatch(idx, 8)
    with pytest.raises(RuntimeError, match="expert id"):
        K().check_status("cuda")
    K().check_status("cuda")  # cleared by the failed check


@pytest.mark.parametrize("T,E,k,S,full,norm", [(777, 76, 6, 2, True, True), (64, 76, 6, 2, False, True),
                                              (300, 8, 2, 0, True, False), (129, 200, 8, 1, True, True)])
def test_router_fused_matches_router_topk_on_the_same_logits(T, E, k, S, full, norm):
    """The whole-block router kernels (bf16 logits with a padded row stride + fp32 bias, shared
    experts appended, column sums) against the fp32 stand-alone router on identical values."""
    from nanospeaker_b200 import kernels as K
    torch.manual_seed(E + k)
    ld = (E + 63) // 64 * 64
    logits = torch.zeros(T, ld, device="cuda", dtype=torch.bfloat16)
    logits[:, :E] = torch.randn(T, E, device="cuda").bfloat16()
    bias = torch.randn(E, device="cuda") * 0.3
    w_all, idx_all, colsum = K.router_fused(logits, bias, E, k, S, norm, full)
    ref_logits = logits[:, :E].float() + bias
    w, idx, probs = K.router_topk(ref_logits, k, norm, full, True)
    assert torch.equal(idx_all[:, :k], idx)                                # bit-exact selection
    assert torch.equal(idx_all[:, k:], torch.arange(E, E + S, device="cuda").expand(T, S))
    assert torch.equal(w_all[:, k:].float(), torch.ones(T, S, device="cuda"))
    assert torch.allclose(w_all[:, :k].float(), w, atol=4e-3, rtol=8e-3)   # bf16 rounding of w
    if full:
        assert torch.allclose(colsum, probs.sum(0), rtol=1e-4, atol=1e-4)
        counts = torch.bincount(idx.reshape(-1), minlength=E).int()
        aux = K.balance_loss(colsum, counts, E, T, 1e-2)
        share = counts.float() / counts.sum()
        ref_aux = 1e-2 * E * (share * probs.mean(0)).sum()
        assert abs(float(aux) - float(ref_aux)) < 1e-5
        # backward: d(logits) of  sum(w * g) + aux  from both kernels
        g = torch.randn(T, k + S, device="cuda").bfloat16()
        d_aux = torch.ones(1, device="cuda")
        dl = K.router_fused_bwd(logits, bias, idx_all, g, E, k, S, norm, full, d_aux, counts, 1e-2, ld)
        d_probs = (1e-2 * E / T) * share.expand(T, E).contiguous()
        ref_dl = K.router_topk_bwd(ref_logits, idx, g[:, :k].float(), d_probs, norm, full)
        assert torch.all(dl[:, E:] == 0)
        assert rel_l2(dl[:, :E].float(), ref_dl) < 1e-2
    K.check_status("cuda")


@pytest.mark.parametrize("T,E,k,S", [(16384, 76, 6, 2), (1000, 76, 6, 1), (129, 8, 2, 0),
                                     (1, 200, 8, 2), (40000, 16, 3, 2)])
def test_router_dispatch_equals_router_fused_then_dispatch(T, E, k, S):
    """The two-launch router + dispatch of the whole-block path against the separate entry points:
    every output bit for bit."""
    from nanospeaker_b200 import kernels as K
    torch.manual_seed(T + E)
    ld = (E + 63) // 64 * 64
    logits = torch.zeros(T, ld, device="cuda", dtype=torch.bfloat16)
    logits[:, :E] = torch.randn(T, E, device="cuda").bfloat16()
    bias = torch.randn(E, device="cuda") * 0.3
    w_all, idx_all, colsum = K.router_fused(logits, bias, E, k, S, True, True)
    ref = K.dispatch(idx_all, E + S)
    got = K.router_dispatch(logits, bias, E, k, S, True, True)
    assert torch.equal(got[0], w_all) and torch.equal(got[1], idx_all)
    assert torch.allclose(got[2], colsum, rtol=1e-5, atol=1e-4)       # atomics: order may differ
    live = int(ref[4])
    assert int(got[7]) == live
    assert torch.equal(got[3][:live], ref[0][:live])                  # sorted_ids
    assert torch.equal(got[4][: live // 128], ref[1][: live // 128])  # expert_ids
    for a, b in ((5, 2), (6, 3), (8, 5)):                             # pad_offsets, counts, inv_ids
        assert torch.equal(got[a], ref[b])
    K.check_status("cuda")
