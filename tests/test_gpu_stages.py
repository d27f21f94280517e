"""GPU parity of the data-movement and grouped-GEMM stages, each against plain fp32 CPU math on the
same seeded inputs. Movement is bit-exact; GEMM stages are bf16-out / fp32-accumulate and are held
to rel-L2 <= 5e-3 (the bar for the whole block is 1e-2)."""
import pytest
import torch

from conftest import rel_l2
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
TOL = 5e-3


def K():
    from nanospeaker_b200 import kernels
    return kernels


def _setup(T, E, k, D, H=128, skew=0.0, seed=0):
    torch.manual_seed(seed)
    logits = torch.randn(T, E) + skew * torch.randn(E)
    idx = logits.topk(k, -1).indices
    plan = O.dispatch(idx, E)
    x = torch.randn(T, D).bfloat16()
    w_in = (torch.randn(E, D, 2 * H) * D ** -0.5).bfloat16()
    w_out = (torch.randn(E, H, D) * H ** -0.5).bfloat16()
    tw = torch.rand(T, k).bfloat16()
    return idx, plan, x, w_in, w_out, tw


def _slot_rows(src, sids, k, nl, M):
    """CPU permute: src[pair // k] per live slot, zeros in pad slots."""
    s = sids[:nl].long()
    live = s < M
    rows = src[(s // k).clamp(max=src.shape[0] - 1)].clone()
    rows[~live] = 0
    return rows, live


def _per_expert(a, w, offs, transpose=False):
    out = torch.zeros(a.shape[0], w.shape[1] if transpose else w.shape[2])
    for e in range(w.shape[0]):
        lo, hi = int(offs[e]), int(offs[e + 1])
        if hi > lo:
            wf = w[e].float()
            out[lo:hi] = a[lo:hi].float() @ (wf.t() if transpose else wf)
    return out


CASES = [(300, 8, 2, 576, 0.0), (1, 8, 1, 64, 0.0), (129, 4, 2, 96, 0.0), (2048, 76, 6, 576, 1.0)]


@pytest.mark.parametrize("T,E,k,D,skew", CASES)
def test_permute_and_combine_are_bit_exact(T, E, k, D, skew):
    idx, (sids, eids, offs, counts, npp, inv), x, _, _, _ = _setup(T, E, k, D, skew=skew)
    nl, M = int(npp), T * k
    g = lambda t: t.cuda()
    xs = K().permute(g(x), k, g(sids), g(npp)).cpu()
    ref, _ = _slot_rows(x, sids, k, nl, M)
    assert torch.equal(xs[:nl], ref)

    y = torch.randn(sids.numel(), D).bfloat16()
    e1, e2 = torch.randn(T, D).bfloat16(), torch.randn(T, D).bfloat16()
    for extras in [(None, None), (e1, None), (e1, e2)]:
        out = K().combine(g(y), g(inv), T, k, *[None if e is None else g(e) for e in extras]).cpu()
        acc = torch.zeros(T, D)
        for j in range(k):
            acc += y[inv.view(T, k)[:, j].long()].float()
        for e in extras:
            if e is not None:
                acc += e.float()
        assert torch.equal(out, acc.bfloat16())


@pytest.mark.parametrize("T,E,k,D,skew", CASES)
def test_forward_gemm_stages(T, E, k, D, skew):
    H = 128
    idx, (sids, eids, offs, counts, npp, inv), x, w_in, w_out, tw = _setup(T, E, k, D, skew=skew)
    nl, M = int(npp), T * k
    g = lambda t: t.cuda()
    xs_ref, live = _slot_rows(x, sids, k, nl, M)
    xs = torch.zeros(sids.numel(), D, dtype=torch.bfloat16)
    xs[:nl] = xs_ref
    a1_ref = _per_expert(xs_ref, w_in, offs)
    hid0, a1 = K().up_gemm(g(xs), g(w_in), g(eids), g(npp), 0, 0, True)
    assert rel_l2(a1.cpu()[:nl], a1_ref) < TOL
    # rows gathered inside the kernel (no permuted copy) give the same bits as the permuted input
    hid_g, a1_g = K().up_gemm(g(x), g(w_in), g(eids), g(npp), 0, 0, True, gather=(g(sids), k))
    assert torch.equal(hid_g[:nl], hid0[:nl]) and torch.equal(a1_g[:nl], a1[:nl])
    for name, act in [("silu", 0), ("gelu", 1), ("relu", 2), ("sigmoid", 3), ("tanh", 4)]:
        hid, raw = K().up_gemm(g(xs), g(w_in), g(eids), g(npp), 0, act, False)
        assert raw is None
        gate, up = a1_ref.chunk(2, -1)
        assert rel_l2(hid.cpu()[:nl], O.ACTS[name](gate) * up) < TOL, name
    gate, up = a1_ref.chunk(2, -1)
    hid_b = torch.zeros(sids.numel(), H, dtype=torch.bfloat16)
    hid_b[:nl] = (torch.nn.functional.silu(gate) * up).bfloat16()
    twf = tw.reshape(-1)
    wslot = torch.where(live, twf[sids[:nl].long().clamp(max=M - 1)].float(), torch.zeros(()))
    y = K().down_gemm(g(hid_b), g(w_out), g(eids), g(npp), 0, g(sids), g(twf), M).cpu()
    y_ref = _per_expert(hid_b[:nl], w_out, offs) * wslot[:, None]
    assert rel_l2(y[:nl], y_ref) < TOL
    assert (y[:nl][~live] == 0).all()                 # pad slots carry exact zeros
    K().check_status("cuda")


@pytest.mark.parametrize("T,E,k,D,skew", CASES)
def test_backward_gemm_stages(T, E, k, D, skew):
    H = 128
    idx, (sids, eids, offs, counts, npp, inv), x, w_in, w_out, tw = _setup(T, E, k, D, skew=skew,
                                                                            seed=3)
    nl, M, cap = int(npp), T * k, sids.numel()
    g = lambda t: t.cuda()
    twf = tw.reshape(-1)
    xs_ref, live = _slot_rows(x, sids, k, nl, M)
    wslot = torch.where(live, twf[sids[:nl].long().clamp(max=M - 1)].float(), torch.zeros(()))
    dout = torch.randn(T, D).bfloat16()
    douts_ref, _ = _slot_rows(dout, sids, k, nl, M)
    pad = lambda t, w: torch.cat([t, torch.zeros(cap - nl, w, dtype=t.dtype)])
    a1_b = pad(_per_expert(xs_ref, w_in, offs).bfloat16(), 2 * H)

    da1, hidw, dtw = K().dhidden_glu_bwd(g(pad(douts_ref, D)), g(w_out), g(eids), g(npp), 0,
                                         g(sids), g(twf), M, g(a1_b), 0, True)
    da1_g, hidw_g, dtw_g = K().dhidden_glu_bwd(g(dout), g(w_out), g(eids), g(npp), 0, g(sids),
                                               g(twf), M, g(a1_b), 0, True, gather_top_k=k)
    assert torch.equal(da1_g[:nl], da1[:nl]) and torch.equal(hidw_g[:nl], hidw[:nl])
    assert torch.equal(dtw_g, dtw)
    G = _per_expert(douts_ref, w_out, offs, transpose=True)
    gate, up = a1_b[:nl].float().chunk(2, -1)
    sg = torch.sigmoid(gate)
    act, dact = gate * sg, sg * (1 + gate * (1 - sg))
    dh = wslot[:, None] * G
    assert rel_l2(da1.cpu()[:nl], torch.cat([dh * up * dact, dh * act], -1)) < TOL
    assert rel_l2(hidw.cpu()[:nl], act * up * wslot[:, None]) < TOL
    dtw_ref = torch.zeros(M)
    dtw_ref[sids[:nl][live].long()] = (G * act * up).sum(-1)[live]
    assert rel_l2(dtw.cpu(), dtw_ref) < TOL

    da1_in = pad((torch.randn(nl, 2 * H) * live[:, None]).bfloat16(), 2 * H)
    ydx = K().dx_gemm(g(da1_in), g(w_in), g(eids), g(npp), 0).cpu()
    assert rel_l2(ydx[:nl], _per_expert(da1_in[:nl], w_in, offs, transpose=True)) < TOL

    xs_b = pad(xs_ref, D)
    dw_in = K().wgrad(g(xs_b), g(da1_in), g(offs), E).cpu()
    dw_out = K().wgrad(g(pad((act * up).bfloat16(), H)), g(pad(douts_ref, D)), g(offs), E).cpu()
    dw_in_g = K().wgrad(g(x), g(da1_in), g(offs), E, gather=("a", g(sids), k)).cpu()
    dw_out_g = K().wgrad(g(pad((act * up).bfloat16(), H)), g(dout), g(offs), E,
                         gather=("b", g(sids), k)).cpu()
    assert torch.equal(dw_in_g, dw_in) and torch.equal(dw_out_g, dw_out)
    for e in range(E):
        lo, hi = int(offs[e]), int(offs[e + 1])
        if hi == lo:
            assert (dw_in[e] == 0).all() and (dw_out[e] == 0).all()   # empty expert: exact zeros
    ref_in = torch.stack([xs_ref[int(offs[e]):int(offs[e + 1])].float().t()
                          @ da1_in[int(offs[e]):int(offs[e + 1])].float() for e in range(E)])
    ref_out = torch.stack([(act * up).bfloat16()[int(offs[e]):int(offs[e + 1])].float().t()
                           @ douts_ref[int(offs[e]):int(offs[e + 1])].float() for e in range(E)])
    assert rel_l2(dw_in, ref_in) < TOL
    assert rel_l2(dw_out, ref_out) < TOL
    K().check_status("cuda")


@pytest.mark.parametrize("T", [1, 5, 127, 128, 129, 1000, 3000])
def test_shared_expert_schedule_on_unpermuted_tokens(T):
    """Fixed-group schedule: all S weight matrices over the rows in token order, any row count,
    out-of-range rows masked; forward and backward stages, incl. split-K weight gradients."""
    D, H, S = 576, 128, 2
    x = torch.randn(T, D).bfloat16()
    dout = torch.randn(T, D).bfloat16()
    wsi = (torch.randn(S, D, 2 * H) * D ** -0.5).bfloat16()
    wso = (torch.randn(S, H, D) * H ** -0.5).bfloat16()
    g = lambda t: t.cuda()
    hid, raw = K().up_gemm(g(x), g(wsi), None, None, S, 0, True)
    y = K().down_gemm(hid, g(wso), None, None, S, None, None, 0)
    da1, hidw, _ = K().dhidden_glu_bwd(g(dout), g(wso), None, None, S, None, None, 0, raw, 0, False)
    ydx = K().dx_gemm(da1, g(wsi), None, None, S)
    dwi = K().wgrad(g(x), da1, None, S, b_grouped=True)
    dwo = K().wgrad(hidw, g(dout), None, S, a_grouped=True)
    dwi_small_chunks = K().wgrad(g(x), da1, None, S, ks_rows=64, b_grouped=True)
    assert hid.shape == (S, T, H) and y.shape == (S, T, D) and dwi.shape == (S, D, 2 * H)
    for s in range(S):
        a1_ref = x.float() @ wsi[s].float()
        gate, up = a1_ref.chunk(2, -1)
        assert rel_l2(raw[s].cpu(), a1_ref) < TOL
        assert rel_l2(hid[s].cpu(), torch.nn.functional.silu(gate) * up) < TOL
        assert rel_l2(y[s].cpu(), hid[s].cpu().float() @ wso[s].float()) < TOL
        gb, ub = raw[s].cpu().float().chunk(2, -1)
        sg = torch.sigmoid(gb)
        act, dact = gb * sg, sg * (1 + gb * (1 - sg))
        G = dout.float() @ wso[s].float().t()
        assert rel_l2(da1[s].cpu(), torch.cat([G * ub * dact, G * act], -1)) < TOL
        assert rel_l2(hidw[s].cpu(), act * ub) < TOL
        assert rel_l2(ydx[s].cpu(), da1[s].cpu().float() @ wsi[s].float().t()) < TOL
        assert rel_l2(dwi[s].cpu(), x.float().t() @ da1[s].cpu().float()) < TOL
        assert rel_l2(dwi_small_chunks[s].cpu(), x.float().t() @ da1[s].cpu().float()) < TOL
        assert rel_l2(dwo[s].cpu(), hidw[s].cpu().float().t() @ dout.float()) < TOL
    K().check_status("cuda")


@pytest.mark.parametrize("T,S", [(1, 1), (127, 2), (300, 2), (1000, 3), (2048, 2)])
def test_group_summed_gemms_store_the_shared_experts_share(T, S):
    """out[t] = sum_g A[offsets[g] + t] @ B_g with plain stores: the shared experts' share of the
    block's output and of dX, read from token-ordered runs at device-side offsets (runs padded to
    128 rows, neighbours holding other data), any token count; and it composes with the routed
    experts' atomic adds that follow it on the same buffer."""
    D, H = 576, 128
    torch.manual_seed(T + S)
    run = (T + 127) // 128 * 128
    first = 256                                  # rows of other runs in front
    rows = first + S * run + 128
    hid = torch.randn(rows, H).bfloat16()
    da1 = (torch.randn(rows, 2 * H) * 0.1).bfloat16()
    wso = (torch.randn(S, H, D) * H ** -0.5).bfloat16()
    wsi = (torch.randn(S, D, 2 * H) * D ** -0.5).bfloat16()
    offs = torch.tensor([first + g * run for g in range(S)], dtype=torch.int32)
    g = lambda t: t.cuda()
    y = K().down_gemm_sum(g(hid), g(wso), g(offs), T)
    dx = K().dx_gemm_sum(g(da1), g(wsi), g(offs), T)
    assert y.shape == (T, D) and dx.shape == (T, D)
    y_ref = sum(hid[int(o):int(o) + T].float() @ wso[i].float() for i, o in enumerate(offs))
    dx_ref = sum(da1[int(o):int(o) + T].float() @ wsi[i].float().t() for i, o in enumerate(offs))
    assert rel_l2(y.cpu(), y_ref) < TOL
    assert rel_l2(dx.cpu(), dx_ref) < TOL
    # a caller-provided buffer is overwritten, not added to
    buf = torch.full((T, D), 7.0, dtype=torch.bfloat16, device="cuda")
    K().down_gemm_sum(g(hid), g(wso), g(offs), T, out=buf)
    assert torch.equal(buf, y)
    K().check_status("cuda")


def test_wgrad_split_k_is_deterministic_and_chunk_size_independent():
    """A hot expert (thousands of rows) is split over many CTAs; the partials are summed in chunk
    order, so two runs agree bit for bit and chunk sizes only move fp32 rounding."""
    torch.manual_seed(4)
    T, E, k, D, H = 6000, 8, 2, 192, 128
    idx = torch.stack([torch.zeros(T, dtype=torch.long), torch.randint(1, E, (T,))], 1)
    sids, eids, offs, counts, npp, inv = O.dispatch(idx, E)
    nl, cap = int(npp), sids.numel()
    a = torch.zeros(cap, D).bfloat16()
    b = torch.zeros(cap, 2 * H).bfloat16()
    live = sids[:nl] < T * k
    a[:nl] = (torch.randn(nl, D) * live[:, None]).bfloat16()
    b[:nl] = (torch.randn(nl, 2 * H) * live[:, None]).bfloat16()
    g = lambda t: t.cuda()
    r1 = K().wgrad(g(a), g(b), g(offs), E, ks_rows=1024)
    r2 = K().wgrad(g(a), g(b), g(offs), E, ks_rows=1024)
    r3 = K().wgrad(g(a), g(b), g(offs), E, ks_rows=128)
    assert torch.equal(r1, r2)
    ref = torch.stack([a[int(offs[e]):int(offs[e + 1])].float().t()
                       @ b[int(offs[e]):int(offs[e + 1])].float() for e in range(E)])
    assert rel_l2(r1.cpu(), ref) < TOL and rel_l2(r3.cpu(), ref) < TOL
    K().check_status("cuda")


def test_entry_points_reject_bad_arguments():
    x = torch.randn(4, 100, device="cuda").bfloat16()          # d_model % 8 != 0
    with pytest.raises(RuntimeError, match="shape|covered"):
        K().permute(x, 2, torch.zeros(128, dtype=torch.int32, device="cuda"),
                    torch.zeros(1, dtype=torch.int32, device="cuda"))
    w = torch.randn(2, 64, 128, device="cuda").bfloat16()       # d_hidden 64: not covered
    with pytest.raises(RuntimeError, match="not covered"):
        K().up_gemm(torch.randn(128, 64, device="cuda").bfloat16(), w, None, None, 1, 0, False)
    with pytest.raises(RuntimeError, match="CUDA"):
        K().router_topk(torch.randn(4, 8), 2, True, False, False)   # CPU tensor: no fallback


@pytest.mark.parametrize("T,E,S,k,D", [(300, 8, 2, 2, 576), (129, 4, 1, 2, 96), (2048, 76, 2, 6, 576)])
def test_shared_experts_read_token_rows_in_place(T, E, S, k, D):
    """The shared experts' runs are the token-major matrix itself: with token_rows the up GEMM, the
    dHidden GEMM and both weight gradients give the same bits as on fully permuted buffers, although
    the permute stopped at the first shared run (rows of those runs hold garbage). T not a multiple
    of 128 makes the last tile of a shared run read past the matrix (zero rows)."""
    H, ks = 128, k + S
    torch.manual_seed(T + S)
    idx = torch.cat([torch.randn(T, E).topk(k, -1).indices,
                     torch.arange(E, E + S).expand(T, S)], 1)
    sids, eids, offs, counts, npp, inv = [t.cuda() for t in O.dispatch(idx, E + S)]
    g = lambda *shape, s=1.0: (torch.randn(*shape, device="cuda") * s).bfloat16()
    x, dout = g(T, D), g(T, D)
    w_in, w_sh_in = g(E, D, 2 * H, s=D ** -0.5), g(S, D, 2 * H, s=D ** -0.5)
    w_out, w_sh_out = g(E, H, D, s=H ** -0.5), g(S, H, D, s=H ** -0.5)
    tw = torch.rand(T * ks, device="cuda").bfloat16()
    nl, M = int(npp), T * ks
    first_shared = offs[E:E + 1]
    assert int(first_shared) < nl

    def poisoned(src):
        part = K().permute(src, ks, sids, first_shared)
        part[int(first_shared):] = float("nan")       # whatever the allocator left there
        return part

    xs_full, douts_full = K().permute(x, ks, sids, npp), K().permute(dout, ks, sids, npp)
    hid0, a10 = K().up_gemm(xs_full, w_in, eids, npp, 0, 0, True, w_extra=w_sh_in)
    hid1, a11 = K().up_gemm(poisoned(x), w_in, eids, npp, 0, 0, True, w_extra=w_sh_in,
                            token_rows=(x, offs))
    assert torch.equal(hid0[:nl], hid1[:nl]) and torch.equal(a10[:nl], a11[:nl])

    args = (w_out, eids, npp, 0, sids, tw, M, a10, 0, True)
    ref = K().dhidden_glu_bwd(douts_full, *args, w_extra=w_sh_out)
    got = K().dhidden_glu_bwd(poisoned(dout), *args, w_extra=w_sh_out, token_rows=(dout, offs))
    for a, b in zip(ref, got):
        assert torch.equal(a[:nl] if a.shape[0] != M else a, b[:nl] if b.shape[0] != M else b)

    da1, hidw = ref[0], ref[1]
    for ks_rows in (0, 64):
        ref_in = K().wgrad(xs_full, da1, offs, E + S, ks_rows, n_extra=S)
        got_in = K().wgrad(poisoned(x), da1, offs, E + S, ks_rows, n_extra=S, token_rows=("a", x))
        ref_out = K().wgrad(hidw, douts_full, offs, E + S, ks_rows, n_extra=S)
        got_out = K().wgrad(hidw, poisoned(dout), offs, E + S, ks_rows, n_extra=S,
                            token_rows=("b", dout))
        for a, b in zip(ref_in + ref_out, got_in + got_out):
            assert torch.equal(a, b)
    K().check_status("cuda")


@pytest.mark.parametrize("T,E,k,D,skew", CASES)
def test_accumulating_down_and_dx_gemms_match_store_then_combine(T, E, k, D, skew):
    """The GEMMs that add their rows straight into the token-major result (bf16 atomics) against
    fp32 CPU math: out[t] = sum_j w * hid @ W_out (+ what the accumulator held), dx[t] = sum_j
    da1 @ W_in^T; also against the store-then-reduce pair on the GPU, and with a per-expert bias."""
    idx, (sids, eids, offs, counts, npp, inv), x, w_in, w_out, tw = _setup(T, E, k, D, skew=skew)
    nl, M = int(npp), T * k
    g = lambda t: t.cuda()
    torch.manual_seed(3)
    hid = (torch.randn(sids.numel(), 128) * 0.5).bfloat16()
    s = sids[:nl].long()
    live = s < M
    hid[:nl][~live] = 0                                   # pad rows are zero rows
    tok = (s // k).clamp(max=T - 1)
    wrow = torch.where(live, tw.reshape(-1)[s.clamp(max=M - 1)].float(), torch.zeros(()))
    bias = (torch.randn(E, D) * 0.1).bfloat16()
    eid_row = eids.long().repeat_interleave(128)[:nl]
    for b in (None, bias):
        y = _per_expert(hid[:nl], w_out, offs)
        if b is not None:
            y = y + b.float()[eid_row]
        y = y * wrow[:, None]
        init = torch.randn(T, D).bfloat16()
        want = init.float().index_add(0, tok[live], y[live])
        acc = g(init).clone()
        K().down_gemm_acc(g(hid), g(w_out), g(eids), g(npp), 0, g(sids), g(tw.reshape(-1)), M, k,
                          acc, bias=None if b is None else g(b))
        assert rel_l2(acc.cpu(), want) < TOL
        ys = K().down_gemm(g(hid), g(w_out), g(eids), g(npp), 0, g(sids), g(tw.reshape(-1)), M,
                           bias=None if b is None else g(b))
        ref = K().combine(ys, g(inv), T, k, g(init))
        assert rel_l2(acc, ref) < TOL
    da1 = (torch.randn(sids.numel(), 256) * 0.5).bfloat16()
    da1[:nl][~live] = 0
    ydx = _per_expert(da1[:nl], w_in, offs, transpose=True)
    want = torch.zeros(T, D).index_add(0, tok[live], ydx[live])
    acc = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    K().dx_gemm_acc(g(da1), g(w_in), g(eids), g(npp), 0, g(sids), M, k, acc)
    assert rel_l2(acc.cpu(), want) < TOL
    K().check_status("cuda")


def test_accumulating_gemms_on_the_fixed_schedule_add_every_group_to_the_same_rows():
    """Fixed schedule: row r of every group lands on row r of the accumulator (how the router's
    share of dx joins the experts'); exact against the storing kernels for one group."""
    torch.manual_seed(0)
    T, D, S = 300, 576, 2
    a = (torch.randn(S, T, 128) * 0.5).bfloat16().cuda()
    w = (torch.randn(S, 128, D) * 0.1).bfloat16().cuda()
    y = K().down_gemm(a, w, None, None, S, None, None, 0)            # [S, T, D]
    acc = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    K().down_gemm_acc(a, w, None, None, S, None, None, 0, 1, acc)
    assert rel_l2(acc, y.float().sum(0)) < TOL
    one = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    K().down_gemm_acc(a[:1], w[:1], None, None, 1, None, None, 0, 1, one)
    assert torch.equal(one, y[0])
    wt = (torch.randn(1, D, 128) * 0.1).bfloat16().cuda()
    ydx = K().dx_gemm(a[:1], wt, None, None, 1)
    one.zero_()
    K().dx_gemm_acc(a[:1], wt, None, None, 1, None, 0, 1, one)
    assert torch.equal(one, ydx[0])
    K().check_status("cuda")
