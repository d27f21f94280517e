"""Tensor-level wrappers around the C ABI: allocate outputs with torch, pass raw device pointers and
the current CUDA stream, raise on any error code. One function per entry point of
include/moe_b200.h; `moe_kernel.py` composes them into the differentiable ops.
"""
from typing import Optional, Tuple

import torch

from . import _lib

ALIGN_M = 128  # rows every expert's run is padded to (src/model/moe_kernel.py:71 uses the same)

# Gate activations the epilogues implement; ids as in src/model/moe_kernel.py:75.
KERNEL_ACTIVATIONS = {"silu": 0, "swish": 0, "gelu": 1, "relu": 2, "sigmoid": 3, "tanh": 4}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("moe_b200 kernels take CUDA tensors only; there is no CPU path")


# Number of CUDA kernels this module has launched (every entry point launches a fixed number).
LAUNCHES = 0


def _count(n: int) -> None:
    global LAUNCHES
    LAUNCHES += n


_status_words = {}


def status_word(device) -> torch.Tensor:
    """The per-device int32 status word kernels write problems into (0 = none seen)."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[key] = w
    return w


def check_status(device) -> None:
    """Synchronising read of the status word; raises if a kernel flagged a problem."""
    w = status_word(device)
    code = int(w.item())
    if code:
        w.zero_()
        what = {1: "a bounded wait inside a GEMM kernel ran out",
                2: "an expert id outside [0, n_experts) reached the dispatch"}.get(code, "unknown")
        raise RuntimeError(f"moe_b200 device status {code}: {what}")


def l_cap(n_pairs: int, n_experts: int) -> int:
    """Worst-case padded pair count (pure arithmetic, safe without a GPU)."""
    live = min(n_experts, n_pairs)
    return (n_pairs + live * (ALIGN_M - 1) + ALIGN_M - 1) // ALIGN_M * ALIGN_M


def router_topk(logits: torch.Tensor, top_k: int, normalize: bool, full_softmax: bool,
                want_probs: bool) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """fp32 logits [T, E] -> (topk_w fp32 [T, k], topk_idx int64 [T, k], probs fp32 [T, E] | None)."""
    _need_cuda(logits)
    logits = logits.contiguous()
    t, e = logits.shape
    w = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
    idx = torch.empty((t, top_k), dtype=torch.int64, device=logits.device)
    probs = torch.empty_like(logits) if want_probs else None
    _lib.check(_lib.load().moe_b200_router_topk(
        logits.data_ptr(), t, e, top_k, int(normalize), int(full_softmax), w.data_ptr(),
        idx.data_ptr(), _lib.ptr(probs), _stream(logits)), "moe_b200_router_topk")
    _count(1 if t else 0)
    return w, idx, probs


def router_topk_bwd(logits, topk_idx, d_topk_w, d_probs, normalize: bool,
                    full_softmax: bool) -> torch.Tensor:
    _need_cuda(logits, topk_idx, d_topk_w, d_probs)
    logits = logits.contiguous()
    t, e = logits.shape
    k = topk_idx.shape[-1]
    d_topk_w = d_topk_w.to(torch.float32).contiguous()
    d_probs = None if d_probs is None else d_probs.to(torch.float32).contiguous()
    out = torch.empty_like(logits)
    _lib.check(_lib.load().moe_b200_router_topk_bwd(
        logits.data_ptr(), topk_idx.contiguous().data_ptr(), d_topk_w.data_ptr(),
        _lib.ptr(d_probs), t, e, k, int(normalize), int(full_softmax), out.data_ptr(),
        _stream(logits)), "moe_b200_router_topk_bwd")
    _count(1 if t else 0)
    return out


def router_fused(logits, bias, n_experts: int, top_k: int, n_shared: int, normalize: bool,
                 full_softmax: bool, noise=None):
    """bf16 logits [T, ld] (+ fp32 bias [E]) -> (w_all bf16 [T, k+S], idx_all int64 [T, k+S],
    colsum fp32 [E] or None). The last S columns are the shared experts (id E+s, weight 1)."""
    _need_cuda(logits)
    t, ld = logits.shape
    ks = top_k + n_shared
    w_all = torch.empty((t, ks), dtype=logits.dtype, device=logits.device)
    idx_all = torch.empty((t, ks), dtype=torch.int64, device=logits.device)
    colsum = (torch.zeros(n_experts, dtype=torch.float32, device=logits.device)
              if full_softmax else None)
    _lib.check(_lib.load().moe_b200_router_fused(
        logits.data_ptr(), ld, _lib.ptr(bias), _lib.ptr(_noise(noise, t, n_experts)), t, n_experts,
        top_k, n_shared, int(normalize), int(full_softmax), w_all.data_ptr(), idx_all.data_ptr(),
        _lib.ptr(colsum), _stream(logits)), "moe_b200_router_fused")
    _count(1 if t else 0)
    return w_all, idx_all, colsum


def _noise(noise, n_tokens: int, n_experts: int):
    """Exploration noise as the kernels read it: fp32 [n_tokens, n_experts], contiguous."""
    if noise is None:
        return None
    assert tuple(noise.shape) == (n_tokens, n_experts) and noise.dtype == torch.float32
    assert noise.is_contiguous()
    return noise


def router_dispatch(logits, bias, n_experts: int, top_k: int, n_shared: int, normalize: bool,
                    full_softmax: bool, noise=None):
    """router_fused + dispatch in two launches (the router kernel leaves the dispatch's per-block
    histograms; one launch when the batch fits one block of 128 tokens): -> (w_all, idx_all, colsum | None, sorted_ids, expert_ids, pad_offsets, counts,
    n_post_pad, inv_ids) with counts / pad_offsets over the n_experts + n_shared experts."""
    _need_cuda(logits)
    t, ld = logits.shape
    ks, n_all = top_k + n_shared, n_experts + n_shared
    dev, i32 = logits.device, torch.int32
    lib = _lib.load()
    m = t * ks
    cap = l_cap(m, n_all)
    w_all = torch.empty((t, ks), dtype=logits.dtype, device=dev)
    idx_all = torch.empty((t, ks), dtype=torch.int64, device=dev)
    colsum = torch.zeros(n_experts, dtype=torch.float32, device=dev) if full_softmax else None
    sids = torch.empty(cap, dtype=i32, device=dev)
    eids = torch.empty(cap // ALIGN_M, dtype=i32, device=dev)
    offs = torch.empty(n_all + 1, dtype=i32, device=dev)
    counts = torch.empty(n_all, dtype=i32, device=dev)
    npp = torch.empty(1, dtype=i32, device=dev)
    inv = torch.empty(m, dtype=i32, device=dev)
    nbytes = lib.moe_b200_router_dispatch_scratch_bytes(t, n_all)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.check(lib.moe_b200_router_dispatch(
        logits.data_ptr(), ld, _lib.ptr(bias), _lib.ptr(_noise(noise, t, n_experts)), t, n_experts,
        top_k, n_shared, int(normalize),
        int(full_softmax), w_all.data_ptr(), idx_all.data_ptr(), _lib.ptr(colsum), sids.data_ptr(),
        eids.data_ptr(), offs.data_ptr(), counts.data_ptr(), npp.data_ptr(), inv.data_ptr(),
        scratch.data_ptr(), nbytes, status_word(dev).data_ptr(), _stream(logits)),
        "moe_b200_router_dispatch")
    # up to 128 tokens of a shape the four-lanes-per-token kernel takes: one launch does both passes
    one = (t <= 128 and top_k <= 8 and n_experts <= 96 and ld % 8 == 0
           and ld >= (64 if n_experts <= 64 else 96))
    _count(1 if one else 2)
    return w_all, idx_all, colsum, sids, eids, offs, counts, npp, inv


def router_fused_bwd(logits, bias, idx_all, dw_all, n_experts: int, top_k: int, n_shared: int,
                     normalize: bool, full_softmax: bool, d_aux, counts, aux_coef: float,
                     ld_out: int, noise=None) -> torch.Tensor:
    """-> d(logits) bf16 [T, ld_out], zero in the pad columns."""
    _need_cuda(logits, idx_all, dw_all)
    t, ld = logits.shape
    out = torch.empty((t, ld_out), dtype=logits.dtype, device=logits.device)
    _lib.check(_lib.load().moe_b200_router_fused_bwd(
        logits.data_ptr(), ld, _lib.ptr(bias), _lib.ptr(_noise(noise, t, n_experts)),
        idx_all.data_ptr(), dw_all.data_ptr(), t,
        n_experts, top_k, n_shared, int(normalize), int(full_softmax), _lib.ptr(d_aux),
        _lib.ptr(counts), float(aux_coef), out.data_ptr(), ld_out, _stream(logits)),
        "moe_b200_router_fused_bwd")
    _count(1 if t else 0)
    return out


def balance_loss(colsum, counts, n_experts: int, n_tokens: int, aux_coef: float) -> torch.Tensor:
    """0-dim fp32: aux_coef * E * sum_e share_e * mean_t probs[t, e], from the column sums."""
    aux = torch.empty((), dtype=torch.float32, device=colsum.device)
    _lib.check(_lib.load().moe_b200_balance_loss(
        colsum.data_ptr(), counts.data_ptr(), n_experts, n_tokens, float(aux_coef),
        aux.data_ptr(), _stream(colsum)), "moe_b200_balance_loss")
    _count(1)
    return aux


def dispatch(topk_idx: torch.Tensor, n_experts: int, capacity: int = 0, n_capped: int = -1):
    """int64 topk_idx [T, k] -> (sorted_ids, expert_ids, pad_offsets, counts, n_post_pad, inv_ids).
    capacity > 0: every expert below n_capped (default: all) keeps the first `capacity` pairs of its
    run; dropped pairs get inv_ids = -1 and no slot, counts still reports the routing decisions."""
    _need_cuda(topk_idx)
    flat = topk_idx.reshape(-1).contiguous()
    if flat.dtype != torch.int64:
        flat = flat.to(torch.int64)
    m = flat.numel()
    dev, i32 = flat.device, torch.int32
    cap = l_cap(m, n_experts)
    lib = _lib.load()
    sids = torch.empty(cap, dtype=i32, device=dev)
    eids = torch.empty(cap // ALIGN_M, dtype=i32, device=dev)
    offs = torch.empty(n_experts + 1, dtype=i32, device=dev)
    counts = torch.empty(n_experts, dtype=i32, device=dev)
    npp = torch.empty(1, dtype=i32, device=dev)
    inv = torch.empty(m, dtype=i32, device=dev)
    nbytes = lib.moe_b200_dispatch_scratch_bytes(m, n_experts)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _lib.check(lib.moe_b200_dispatch(
        flat.data_ptr(), m, n_experts, sids.data_ptr(), eids.data_ptr(), offs.data_ptr(),
        counts.data_ptr(), npp.data_ptr(), inv.data_ptr(), scratch.data_ptr(), nbytes, capacity,
        n_experts if n_capped < 0 else n_capped, status_word(dev).data_ptr(), _stream(flat)),
        "moe_b200_dispatch")
    _count(3 if m else 1)
    return sids, eids, offs, counts, npp, inv


def permute(x: torch.Tensor, top_k: int, sorted_ids: torch.Tensor,
            n_post_pad: torch.Tensor) -> torch.Tensor:
    """x [T, D] -> xs [l_cap, D] in slot order; rows at or past n_post_pad are left unwritten."""
    _need_cuda(x)
    t, d = x.shape
    cap = sorted_ids.numel()
    xs = torch.empty((cap, d), dtype=x.dtype, device=x.device)
    _lib.check(_lib.load().moe_b200_permute(
        x.data_ptr(), t, d, top_k, sorted_ids.data_ptr(), n_post_pad.data_ptr(), cap,
        xs.data_ptr(), _stream(x)), "moe_b200_permute")
    _count(1 if cap and t else 0)
    return xs


def combine(y: torch.Tensor, inv_ids: torch.Tensor, n_tokens: int, top_k: int,
            extra: Optional[torch.Tensor] = None,
            extra2: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(y)
    d = y.shape[1]
    out = torch.empty((n_tokens, d), dtype=y.dtype, device=y.device)
    _lib.check(_lib.load().moe_b200_combine(
        y.data_ptr(), inv_ids.data_ptr(), n_tokens, top_k, d, _lib.ptr(extra), _lib.ptr(extra2),
        out.data_ptr(), _stream(y)), "moe_b200_combine")
    _count(1 if n_tokens else 0)
    return out


def segment_colsum(buf, expert_ids, n_post_pad, n_groups: int, sorted_ids=None, pair_w=None,
                   n_pairs: int = 0, token_rows=None) -> torch.Tensor:
    """fp32 [n_groups, width]: per expert the column sums of its run's rows of the slot-ordered
    buf [rows, width], each row weighted by pair_w[sorted_ids[row]] when pair_w is given.
    token_rows=(matrix, pad_offsets, first_group): the runs from first_group on read their rows
    from the token-major matrix (row = slot - start of the run) instead of from buf."""
    _need_cuda(buf)
    rows, width = buf.shape
    out = torch.zeros((n_groups, width), dtype=torch.float32, device=buf.device)
    alt, offs, first = token_rows if token_rows is not None else (None, None, 0)
    _lib.check(_lib.load().moe_b200_segment_colsum(
        buf.data_ptr(), rows, width, expert_ids.data_ptr(), n_post_pad.data_ptr(), _lib.ptr(offs),
        n_groups, _lib.ptr(sorted_ids), _lib.ptr(pair_w), n_pairs, _lib.ptr(alt),
        alt.shape[0] if alt is not None else 0, first, out.data_ptr(), _stream(buf)),
        "moe_b200_segment_colsum")
    _count(1 if rows else 0)
    return out


def group_sumsq(x: torch.Tensor) -> torch.Tensor:
    """fp32 [G]: sum of squares of every x[g] (x [G, ...] bf16, contiguous)."""
    _need_cuda(x)
    g = x.shape[0]
    out = torch.zeros(g, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().moe_b200_group_sumsq(x.data_ptr(), g, x[0].numel(), out.data_ptr(),
                                                _stream(x)), "moe_b200_group_sumsq")
    _count(1)
    return out


def axpby(x: torch.Tensor, alpha: float, y=None, beta: float = 0.0, sumsq=None, eps: float = 0.0,
          out=None) -> torch.Tensor:
    """alpha * s_g * x + beta * y (fp32 arithmetic, bf16 result), s_g = 1 / (sqrt(sumsq[g]) + eps)
    per leading-dim group when sumsq is given."""
    _need_cuda(x, y)
    out = torch.empty_like(x) if out is None else out
    _lib.check(_lib.load().moe_b200_axpby(
        x.data_ptr(), _lib.ptr(y), out.data_ptr(), x.shape[0], x[0].numel(), float(alpha),
        float(beta), _lib.ptr(sumsq), float(eps), _stream(x)), "moe_b200_axpby")
    _count(1)
    return out


def _stack(n_fixed: int, rows: int, width: int, like: torch.Tensor) -> torch.Tensor:
    shape = (rows, width) if n_fixed == 0 else (n_fixed, rows, width)
    return torch.empty(shape, dtype=like.dtype, device=like.device)


def _extra(w_extra):
    return (0, 0) if w_extra is None else (w_extra.data_ptr(), w_extra.shape[0])


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float):
    """x [T, D] bf16, gamma [D] bf16 -> (h = x * rstd * gamma [T, D] bf16, rstd [T] fp32)."""
    _need_cuda(x, gamma)
    t, d = x.shape
    h = torch.empty_like(x)
    rstd = torch.empty(t, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().moe_b200_rmsnorm(
        x.data_ptr(), gamma.data_ptr(), t, d, float(eps), h.data_ptr(), rstd.data_ptr(),
        _stream(x)), "moe_b200_rmsnorm")
    _count(1 if t else 0)
    return h, rstd


def rmsnorm_bwd(dh, x, rstd, gamma, add=None):
    """-> (dx [T, D] bf16 including `add` (the residual branch's gradient) when given,
    dgamma [D] fp32)."""
    _need_cuda(dh, x, rstd, gamma)
    t, d = x.shape
    dx = torch.empty_like(x)
    dgamma = torch.zeros(d, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().moe_b200_rmsnorm_bwd(
        dh.data_ptr(), x.data_ptr(), rstd.data_ptr(), gamma.data_ptr(), _lib.ptr(add), t, d,
        dx.data_ptr(), dgamma.data_ptr(), _stream(x)), "moe_b200_rmsnorm_bwd")
    _count(1 if t else 0)
    return dx, dgamma


def copy_cols(src: torch.Tensor, dst_ld: int) -> torch.Tensor:
    """[rows, cols] 16-bit matrix -> [rows, dst_ld]: zero-padded columns (dst_ld > cols) or the
    first dst_ld columns (dst_ld < cols)."""
    _need_cuda(src)
    assert src.dim() == 2 and src.element_size() == 2 and src.stride(1) == 1
    rows, cols = src.shape
    dst = torch.empty((rows, dst_ld), dtype=src.dtype, device=src.device)
    _lib.check(_lib.load().moe_b200_copy_cols(
        src.data_ptr(), rows, min(cols, dst_ld), src.stride(0), dst.data_ptr(), dst_ld,
        _stream(src)), "moe_b200_copy_cols")
    _count(1 if rows else 0)
    return dst


def up_gemm(a, w_in, expert_ids, n_post_pad, n_fixed: int, act: int, want_raw: bool,
            gather=None, w_extra=None, token_rows=None, bias=None, pad_offsets=None):
    """a x w_in [G, D, 2H] -> (act(g)*u [rows, H], raw [g|u] [rows, 2H] | None).
    a is slot-ordered [rows, D]; or, with gather=(sorted_ids, top_k), the token-major x [T, D] whose
    rows the kernel gathers itself (rows = len(sorted_ids)). n_fixed = S > 0 applies weight
    matrices 0..S-1 to all rows of a; outputs are then [S, rows, .]. w_extra is an optional second
    weight stack for expert ids >= G (the shared experts on the routed schedule).
    token_rows=(x, pad_offsets): the experts of the second stack read their rows from the token-major
    x [T, D] (row = slot - start of the expert's run) instead of from a, whose rows in those runs
    need not have been written.
    pad_offsets (the dispatch's run starts; implied by token_rows): lets the routed schedule run on
    CTA pairs that share each weight tile."""
    _need_cuda(a, w_in)
    tok, offs = token_rows if token_rows is not None else (None, pad_offsets)
    d = a.shape[1]
    xp, xn = _extra(w_extra)
    sids, top_k = gather if gather is not None else (None, 0)
    rows = sids.numel() if gather is not None else a.shape[0]
    n_pairs = a.shape[0] * top_k
    g, _, h2 = w_in.shape
    h = h2 // 2
    hid = _stack(n_fixed, rows, h, a)
    raw = _stack(n_fixed, rows, h2, a) if want_raw else None
    _lib.check(_lib.load().moe_b200_up_gemm(
        a.data_ptr(), rows, d, w_in.data_ptr(), g, xp, xn, h, _lib.ptr(expert_ids),
        _lib.ptr(n_post_pad), n_fixed, _lib.ptr(sids), top_k, n_pairs, act, hid.data_ptr(), _lib.ptr(raw),
        _lib.ptr(tok), tok.shape[0] if tok is not None else 0, _lib.ptr(offs), _lib.ptr(bias),
        status_word(a.device).data_ptr(), _stream(a)), "moe_b200_up_gemm")
    _count(1 if rows else 0)
    return hid, raw


def down_gemm(hid, w_out, expert_ids, n_post_pad, n_fixed: int, sorted_ids, pair_w,
              n_pairs: int, w_extra=None, bias=None, out=None) -> torch.Tensor:
    """hid [rows, K] (or [S, rows, K]) x w_out [G, K, D] -> y, scaled per row by
    pair_w[sorted_ids[row]] on the routed schedule."""
    _need_cuda(hid, w_out)
    rows, k = hid.shape[-2:]
    g, _, d = w_out.shape
    y = _stack(n_fixed, rows, d, hid) if out is None else out   # out: a caller-owned [rows, D] buffer
    xp, xn = _extra(w_extra)
    _lib.check(_lib.load().moe_b200_down_gemm(
        hid.data_ptr(), rows, k, w_out.data_ptr(), g, xp, xn, d, _lib.ptr(expert_ids),
        _lib.ptr(n_post_pad), n_fixed, _lib.ptr(sorted_ids), _lib.ptr(pair_w), n_pairs,
        y.data_ptr(), _lib.ptr(bias), status_word(hid.device).data_ptr(), _stream(hid)),
        "moe_b200_down_gemm")
    _count(1 if rows else 0)
    return y


def down_gemm_acc(hid, w_out, expert_ids, n_post_pad, n_fixed: int, sorted_ids, pair_w,
                  n_pairs: int, top_k: int, acc: torch.Tensor, w_extra=None, bias=None) -> torch.Tensor:
    """The down GEMM fused with the combine: every live row of (hid x w_out[e]) * pair_w is added
    (bf16 atomics) to row sorted_ids[row] // top_k of acc [T, D], which the caller has filled with
    zeros or another summand. Fixed schedule: row r of every group goes to row r of acc."""
    _need_cuda(hid, w_out, acc)
    rows, k = hid.shape[-2:]
    g, _, d = w_out.shape
    assert acc.is_contiguous() and acc.shape[1] == d and acc.dtype == hid.dtype
    xp, xn = _extra(w_extra)
    _lib.check(_lib.load().moe_b200_down_gemm_acc(
        hid.data_ptr(), rows, k, w_out.data_ptr(), g, xp, xn, d, _lib.ptr(expert_ids),
        _lib.ptr(n_post_pad), n_fixed, _lib.ptr(sorted_ids), _lib.ptr(pair_w), n_pairs, top_k,
        acc.data_ptr(), acc.shape[0], _lib.ptr(bias), status_word(hid.device).data_ptr(),
        _stream(hid)), "moe_b200_down_gemm_acc")
    _count(1 if rows else 0)
    return acc


def down_gemm_sum(hid, w_out, run_offsets, n_tokens: int, out=None) -> torch.Tensor:
    """out [T, D] = sum_g hid[run_offsets[g] + t] @ w_out[g] (plain stores): the shared experts'
    share of the block's output, written as the initial value of the atomic combine's accumulator.
    run_offsets: int32 device tensor [S], the starts of the groups' token-ordered runs in hid."""
    _need_cuda(hid, w_out)
    rows, k = hid.shape
    g, _, d = w_out.shape
    if out is None:
        out = torch.empty((n_tokens, d), dtype=hid.dtype, device=hid.device)
    assert run_offsets.dtype == torch.int32 and run_offsets.numel() >= g and out.is_contiguous()
    _lib.check(_lib.load().moe_b200_down_gemm_sum(
        hid.data_ptr(), rows, k, w_out.data_ptr(), g, d, run_offsets.data_ptr(), n_tokens,
        out.data_ptr(), status_word(hid.device).data_ptr(), _stream(hid)), "moe_b200_down_gemm_sum")
    _count(1)
    return out


def dx_gemm_sum(da1, w_in, run_offsets, n_tokens: int, out=None) -> torch.Tensor:
    """out [T, D] = sum_g da1[run_offsets[g] + t] @ w_in[g]^T (plain stores): the shared experts'
    share of dX as the initial value of the accumulator dx_gemm_acc adds the routed rows to."""
    _need_cuda(da1, w_in)
    rows, h2 = da1.shape
    g, d, _ = w_in.shape
    if out is None:
        out = torch.empty((n_tokens, d), dtype=da1.dtype, device=da1.device)
    assert run_offsets.dtype == torch.int32 and run_offsets.numel() >= g and out.is_contiguous()
    _lib.check(_lib.load().moe_b200_dx_gemm_sum(
        da1.data_ptr(), rows, h2 // 2, w_in.data_ptr(), g, d, run_offsets.data_ptr(), n_tokens,
        out.data_ptr(), status_word(da1.device).data_ptr(), _stream(da1)), "moe_b200_dx_gemm_sum")
    _count(1)
    return out


def dx_gemm_acc(da1, w_in, expert_ids, n_post_pad, n_fixed: int, sorted_ids, n_pairs: int,
                top_k: int, acc: torch.Tensor, w_extra=None, pad_offsets=None) -> torch.Tensor:
    """The dX GEMM fused with the combine: row `row` of da1 x w_in[e]^T is added to row
    sorted_ids[row] // top_k of acc [T, D] (fixed schedule: row r of every group to row r).
    pad_offsets (the dispatch's run starts): lets the routed schedule run on CTA pairs."""
    _need_cuda(da1, w_in, acc)
    rows, h2 = da1.shape[-2:]
    g, d, _ = w_in.shape
    assert acc.is_contiguous() and acc.shape[1] == d and acc.dtype == da1.dtype
    xp, xn = _extra(w_extra)
    _lib.check(_lib.load().moe_b200_dx_gemm_acc(
        da1.data_ptr(), rows, h2 // 2, w_in.data_ptr(), g, xp, xn, d, _lib.ptr(expert_ids),
        _lib.ptr(n_post_pad), n_fixed, _lib.ptr(sorted_ids), n_pairs, top_k, acc.data_ptr(),
        acc.shape[0], _lib.ptr(pad_offsets), status_word(da1.device).data_ptr(), _stream(da1)),
        "moe_b200_dx_gemm_acc")
    _count(1 if rows else 0)
    return acc


def dhidden_glu_bwd(douts, w_out, expert_ids, n_post_pad, n_fixed: int, sorted_ids, pair_w,
                    n_pairs: int, a1, act: int, want_dtw: bool, gather_top_k: int = 0,
                    w_extra=None, token_rows=None, dtw_out=None):
    """-> (da1 [.., rows, 2H], hidw [.., rows, H], dtw [n_pairs] | None). douts is slot-ordered
    [rows, D], or with gather_top_k > 0 the token-major dOut [T, D] gathered through sorted_ids.
    token_rows=(dout, pad_offsets): as for up_gemm, for the rows of douts."""
    _need_cuda(douts, w_out, a1)
    tok, offs = token_rows if token_rows is not None else (None, None)
    d = douts.shape[1]
    rows = sorted_ids.numel() if gather_top_k else douts.shape[0]
    g, h, _ = w_out.shape
    da1 = _stack(n_fixed, rows, 2 * h, douts)
    hidw = _stack(n_fixed, rows, h, douts)
    dtw = None
    if want_dtw:
        dtw = dtw_out if dtw_out is not None else torch.empty(n_pairs, dtype=douts.dtype,
                                                              device=douts.device)
    xp, xn = _extra(w_extra)
    _lib.check(_lib.load().moe_b200_dhidden_glu_bwd(
        douts.data_ptr(), rows, d, w_out.data_ptr(), g, xp, xn, h, _lib.ptr(expert_ids),
        _lib.ptr(n_post_pad), n_fixed, _lib.ptr(sorted_ids), gather_top_k, _lib.ptr(pair_w),
        n_pairs, a1.data_ptr(), act, da1.data_ptr(), hidw.data_ptr(), _lib.ptr(dtw),
        _lib.ptr(tok), tok.shape[0] if tok is not None else 0, _lib.ptr(offs),
        status_word(douts.device).data_ptr(), _stream(douts)), "moe_b200_dhidden_glu_bwd")
    _count(1 if rows else 0)
    return da1, hidw, dtw


def dx_gemm(da1, w_in, expert_ids, n_post_pad, n_fixed: int, w_extra=None, out=None) -> torch.Tensor:
    """da1 [.., rows, 2H] x w_in[e]^T -> ydx [.., rows, D]."""
    _need_cuda(da1, w_in)
    rows, h2 = da1.shape[-2:]
    g, d, _ = w_in.shape
    ydx = _stack(n_fixed, rows, d, da1) if out is None else out
    xp, xn = _extra(w_extra)
    _lib.check(_lib.load().moe_b200_dx_gemm(
        da1.data_ptr(), rows, h2 // 2, w_in.data_ptr(), g, xp, xn, d, _lib.ptr(expert_ids),
        _lib.ptr(n_post_pad), n_fixed, ydx.data_ptr(), status_word(da1.device).data_ptr(),
        _stream(da1)), "moe_b200_dx_gemm")
    _count(1 if rows else 0)
    return ydx


def wgrad(a, b, pad_offsets, n_groups: int, ks_rows: int = 0, a_grouped: bool = False,
          b_grouped: bool = False, gather=None, n_extra: int = 0, token_rows=None):
    """dw[e] = a_e^T @ b_e over run e's rows -> [G, Mdim, Ndim]. Routed schedule: a [rows, Mdim],
    b [rows, Ndim] in slot order plus pad_offsets. Fixed schedule (pad_offsets None): every group
    spans all rows; a / b are [G, rows, .] when *_grouped, else shared by the groups.
    ks_rows = rows per split-K chunk (0: chosen by the library).
    gather=("a" | "b", sorted_ids, top_k): that operand is token-major [T, .] and gathered inside
    the kernel (routed schedule only).
    n_extra > 0: the last n_extra groups are returned as a second tensor (dw, dw_extra).
    token_rows=("a" | "b", m): the last n_extra runs read that operand from the token-major matrix m
    (row = slot - start of the run) instead of from the slot-ordered buffer."""
    _need_cuda(a, b)
    alt_which, alt = (0, None) if token_rows is None else (1 if token_rows[0] == "a" else 2, token_rows[1])
    import ctypes
    which, sids, top_k = 0, None, 0
    if gather is not None:
        which = 1 if gather[0] == "a" else 2
        sids, top_k = gather[1], gather[2]
    slot_op = b if which == 1 else a
    rows = slot_op.shape[-2]
    m_dim, n_dim = a.shape[-1], b.shape[-1]
    n_pairs = (a if which == 1 else b).shape[0] * top_k if which else 0
    routed = pad_offsets is not None
    lib = _lib.load()
    pb = ctypes.c_size_t(0)
    _lib.check(lib.moe_b200_wgrad_scratch_bytes(m_dim, n_dim, rows, n_groups, int(routed),
                                                ks_rows, ctypes.byref(pb)),
               "moe_b200_wgrad_scratch_bytes")
    partials = torch.empty(max(pb.value, 32), dtype=torch.uint8, device=a.device)
    n_first = n_groups - n_extra
    dw = torch.empty((n_first, m_dim, n_dim), dtype=a.dtype, device=a.device)
    dw_extra = (torch.empty((n_extra, m_dim, n_dim), dtype=a.dtype, device=a.device)
                if n_extra else None)
    _lib.check(lib.moe_b200_wgrad(
        a.data_ptr(), int(a_grouped), m_dim, b.data_ptr(), int(b_grouped), n_dim, rows,
        _lib.ptr(pad_offsets), n_groups, ks_rows, _lib.ptr(sids), top_k, n_pairs, which,
        dw.data_ptr(), n_first, _lib.ptr(dw_extra), partials.data_ptr(), pb.value,
        _lib.ptr(alt), alt.shape[0] if alt is not None else 0, alt_which,
        status_word(a.device).data_ptr(), _stream(a)), "moe_b200_wgrad")
    _count(2 if rows > (ks_rows or 256) else 1)
    return (dw, dw_extra) if n_extra else dw


# ---------------------------------------------------------------- the whole block in one call
def block_fwd(x, router_w, logit_bias, noise, w_in, w_out, w_sh_in, w_sh_out, top_k: int,
              normalize: bool, full_softmax: bool, aux_coef: float, act: int, ld: int):
    """moe_b200_block_fwd: the training forward of the whole block issued by one C call. Returns
    (out, aux, counts, xs, a1, logits, w_all, idx_all, sorted_ids, expert_ids, pad_offsets,
    counts_all, n_post_pad, inv_ids, router_w_padded [1, D, ld])."""
    import ctypes
    _need_cuda(x, w_in, w_out)
    t, d = x.shape
    e_n, _, h2 = w_in.shape
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    ks, n_all = top_k + s_n, e_n + s_n
    cap = l_cap(t * ks, n_all)
    dev, i32 = x.device, torch.int32
    new = lambda shape, dtype=x.dtype: torch.empty(shape, dtype=dtype, device=dev)
    out, aux, counts = new((t, d)), new((), torch.float32), new((e_n,), i32)
    xs, a1, logits = new((cap, d)), new((cap, h2)), new((t, ld))
    w_all, idx_all = new((t, ks)), new((t, ks), torch.int64)
    sids, eids, offs = new((cap,), i32), new((cap // ALIGN_M,), i32), new((n_all + 1,), i32)
    counts_all, npp, inv = new((n_all,), i32), new((1,), i32), new((t * ks,), i32)
    wp = new((1, d, ld))
    lib = _lib.load()
    nbytes = lib.moe_b200_block_fwd_scratch_bytes(t, d, h2 // 2, e_n, s_n, top_k)
    scratch = new((nbytes,), torch.uint8)
    n_l = ctypes.c_int32(0)
    _lib.check(lib.moe_b200_block_fwd(
        x.data_ptr(), t, d, router_w.data_ptr(), _lib.ptr(logit_bias),
        _lib.ptr(_noise(noise, t, e_n)), w_in.data_ptr(), w_out.data_ptr(), e_n, h2 // 2,
        _lib.ptr(w_sh_in), _lib.ptr(w_sh_out), s_n, top_k, int(normalize), int(full_softmax),
        float(aux_coef), act, out.data_ptr(), aux.data_ptr(), counts.data_ptr(), xs.data_ptr(),
        a1.data_ptr(), logits.data_ptr(), w_all.data_ptr(), idx_all.data_ptr(), sids.data_ptr(),
        eids.data_ptr(), offs.data_ptr(), counts_all.data_ptr(), npp.data_ptr(), inv.data_ptr(),
        wp.data_ptr(), scratch.data_ptr(), nbytes, ctypes.byref(n_l),
        status_word(dev).data_ptr(), _stream(x)), "moe_b200_block_fwd")
    _count(n_l.value)
    return (out, aux, counts, xs, a1, logits, w_all, idx_all, sids, eids, offs, counts_all, npp,
            inv, wp)


def block_infer(x, router_w_padded, logit_bias, w_in, w_out, w_sh_in, w_sh_out, top_k: int,
                normalize: bool, act: int, residual, atomic: bool) -> torch.Tensor:
    """moe_b200_block_infer: the inference forward of the whole block (+ residual) by one C call."""
    import ctypes
    _need_cuda(x, w_in, w_out)
    t, d = x.shape
    e_n, _, h2 = w_in.shape
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    out = torch.empty_like(x)
    lib = _lib.load()
    nbytes = lib.moe_b200_block_infer_scratch_bytes(t, d, h2 // 2, e_n, s_n, top_k)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    n_l = ctypes.c_int32(0)
    _lib.check(lib.moe_b200_block_infer(
        x.data_ptr(), t, d, router_w_padded.data_ptr(), _lib.ptr(logit_bias), w_in.data_ptr(),
        w_out.data_ptr(), e_n, h2 // 2, _lib.ptr(w_sh_in), _lib.ptr(w_sh_out), s_n, top_k,
        int(normalize), act, _lib.ptr(residual), int(atomic), out.data_ptr(), scratch.data_ptr(),
        nbytes, ctypes.byref(n_l), status_word(x.device).data_ptr(), _stream(x)),
        "moe_b200_block_infer")
    _count(n_l.value)
    return out


def block_bwd(grad_out, grad_aux, x, logit_bias, noise, w_in, w_out, w_sh_in, w_sh_out, xs, a1,
              logits, w_all, idx_all, sids, eids, offs, counts_all, npp, wp, top_k: int,
              normalize: bool, full_softmax: bool, aux_coef: float, act: int, side_streams):
    """moe_b200_block_bwd: the whole backward issued by one C call (three streams inside).
    Returns (dx, d_router [D, E], dw_in, dw_out, dw_sh_in | None, dw_sh_out | None)."""
    import ctypes
    _need_cuda(grad_out, x)
    t, d = x.shape
    e_n, _, h2 = w_in.shape
    s_n = 0 if w_sh_in is None else w_sh_in.shape[0]
    dev = x.device
    new = lambda shape, dtype=x.dtype: torch.empty(shape, dtype=dtype, device=dev)
    dx, d_router = new((t, d)), new((d, e_n))
    dw_in, dw_out = torch.empty_like(w_in), torch.empty_like(w_out)
    dw_sh_in = torch.empty_like(w_sh_in) if s_n else None
    dw_sh_out = torch.empty_like(w_sh_out) if s_n else None
    lib = _lib.load()
    nbytes = lib.moe_b200_block_bwd_scratch_bytes(t, d, h2 // 2, e_n, s_n, top_k)
    scratch = new((nbytes,), torch.uint8)
    sa, sb = side_streams if side_streams is not None else (None, None)
    # (buffers of this stream are used on the side streams too: the call joins them back into
    # this stream before it returns, so whatever reuses the memory later is ordered after them)
    n_l = ctypes.c_int32(0)
    _lib.check(lib.moe_b200_block_bwd(
        grad_out.data_ptr(), _lib.ptr(grad_aux), x.data_ptr(), t, d, _lib.ptr(logit_bias),
        _lib.ptr(_noise(noise, t, e_n)), w_in.data_ptr(), w_out.data_ptr(), e_n, h2 // 2,
        _lib.ptr(w_sh_in), _lib.ptr(w_sh_out), s_n, top_k, int(normalize), int(full_softmax),
        float(aux_coef), act, xs.data_ptr(), a1.data_ptr(), logits.data_ptr(), w_all.data_ptr(),
        idx_all.data_ptr(), sids.data_ptr(), eids.data_ptr(), offs.data_ptr(),
        counts_all.data_ptr(), npp.data_ptr(), wp.data_ptr(), dx.data_ptr(), d_router.data_ptr(),
        dw_in.data_ptr(), dw_out.data_ptr(), _lib.ptr(dw_sh_in), _lib.ptr(dw_sh_out),
        scratch.data_ptr(), nbytes, sa.cuda_stream if sa is not None else None,
        sb.cuda_stream if sb is not None else None, ctypes.byref(n_l),
        status_word(dev).data_ptr(), _stream(x)), "moe_b200_block_bwd")
    _count(n_l.value)
    return dx, d_router, dw_in, dw_out, dw_sh_in, dw_sh_out


# ---------------------------------------------------------------- expert parallelism, peer memory
def _ptr_array(ptrs):
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*ptrs) if ptrs is not None else None


def ep_plan(cnt_all, bounds, rank: int, n_local: int, cap_tiles: int):
    """cnt_all [G, E] int32, bounds [G+1] int32 (both on the device) -> (owner_of [E], send_row0 [E],
    own_offs [n_local+1], own_counts [n_local], own_npp [1], own_eids [cap_tiles])."""
    _need_cuda(cnt_all, bounds)
    g, e = cnt_all.shape
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=cnt_all.device)
    owner_of, send_row0 = i32(e), i32(e)
    own_offs, own_counts, own_npp, own_eids = i32(n_local + 1), i32(max(n_local, 1)), i32(1), i32(cap_tiles)
    _lib.check(_lib.load().moe_b200_ep_plan(
        cnt_all.data_ptr(), bounds.data_ptr(), g, e, rank, owner_of.data_ptr(),
        send_row0.data_ptr(), own_offs.data_ptr(), own_counts.data_ptr(), own_npp.data_ptr(),
        own_eids.data_ptr(), cap_tiles, _stream(cnt_all)), "moe_b200_ep_plan")
    _count(1)
    return owner_of, send_row0, own_offs, own_counts, own_npp, own_eids


def ep_pair_map(idx_all, inv_ids, local_offs, owner_of, send_row0, n_experts: int, n_ranks: int):
    _need_cuda(idx_all)
    t, k_all = idx_all.shape
    pair_rank = torch.empty(t * k_all, dtype=torch.int32, device=idx_all.device)
    pair_row = torch.empty_like(pair_rank)
    _lib.check(_lib.load().moe_b200_ep_pair_map(
        idx_all.data_ptr(), inv_ids.data_ptr(), local_offs.data_ptr(), owner_of.data_ptr(),
        send_row0.data_ptr(), t, k_all, n_experts, n_ranks, pair_rank.data_ptr(),
        pair_row.data_ptr(), _stream(idx_all)), "moe_b200_ep_pair_map")
    _count(1 if t else 0)
    return pair_rank, pair_row


def ep_push_rows(src, k_all: int, sorted_ids, n_live_slots, pair_rank, pair_row, dst_rows,
                 dst_sid=None, dst_w=None, w_all=None, first_slot=None) -> None:
    """dst_* are lists of device pointers (ints), one per rank; first_slot (1-element int32 device
    tensor) is where the walk over the slots starts before it wraps around."""
    _need_cuda(src)
    t, d = src.shape
    _lib.check(_lib.load().moe_b200_ep_push_rows(
        src.data_ptr(), t, d, k_all, sorted_ids.data_ptr(), n_live_slots.data_ptr(),
        _lib.ptr(first_slot), sorted_ids.numel(), pair_rank.data_ptr(), pair_row.data_ptr(), _ptr_array(dst_rows),
        _ptr_array(dst_sid), _ptr_array(dst_w), len(dst_rows), _lib.ptr(w_all), _stream(src)),
        "moe_b200_ep_push_rows")
    _count(1 if t else 0)


def ep_pad_fix(own_offs, own_counts, n_local: int, rows, sid=None, sentinel: int = 0) -> None:
    _need_cuda(rows)
    _lib.check(_lib.load().moe_b200_ep_pad_fix(
        own_offs.data_ptr(), own_counts.data_ptr(), n_local, rows.data_ptr(), rows.shape[1],
        _lib.ptr(sid), sentinel, _stream(rows)), "moe_b200_ep_pad_fix")
    _count(1 if n_local else 0)


def ep_pull_combine(y_ptrs, pair_rank, pair_row, n_tokens: int, k_all: int, d_model: int, like,
                    extra=None) -> torch.Tensor:
    out = torch.empty((n_tokens, d_model), dtype=like.dtype, device=like.device)
    _lib.check(_lib.load().moe_b200_ep_pull_combine(
        _ptr_array(y_ptrs), len(y_ptrs), pair_rank.data_ptr(), pair_row.data_ptr(), n_tokens,
        k_all, d_model, _lib.ptr(extra), out.data_ptr(), _stream(like)), "moe_b200_ep_pull_combine")
    _count(1 if n_tokens else 0)
    return out


def ep_pull_vec(v_ptrs, pair_rank, pair_row, n_tokens: int, k_all: int, top_k: int, like):
    out = torch.empty((n_tokens, k_all), dtype=like.dtype, device=like.device)
    _lib.check(_lib.load().moe_b200_ep_pull_vec(
        _ptr_array(v_ptrs), len(v_ptrs), pair_rank.data_ptr(), pair_row.data_ptr(), n_tokens,
        k_all, top_k, out.data_ptr(), _stream(like)), "moe_b200_ep_pull_vec")
    _count(1 if n_tokens else 0)
    return out
