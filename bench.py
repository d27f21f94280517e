"""Benchmark of the MoE block on B200: tokens/s of one forward+backward of the block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): BASELINE config 2 -- T=16384 tokens (8 x 2048), d_model 576, 76 routed + 2 shared
SwiGLU experts (d_expert 128), top-6 softmax routing, bf16 with fp32 accumulation, training mode,
per-expert logit bias ~N(0, 0.27) so the expert load has CV ~ 1. One step = router, dispatch,
permute, grouped GEMMs, combine, shared experts and the full backward (dx, dW_in, dW_out,
dW_sh_*, d_router). With N > 1 every rank runs the same per-GPU workload on its own token shard
(weak scaling; tokens are independent, so the block's data path needs no collective).

Prints ONE JSON line (rank 0). `value` times K steps with inputs resident in HBM; `e2e` times
the same step through MoEBlock.forward/backward with the step's input copied from pinned host
memory and the loss read back. `--impl reference` times the CPU oracle (the reference's
pure-PyTorch path restated, see oracle/moe_oracle.py) on the host cores instead.

Side workloads, one JSON line each, not the headline (`--workload`): `decode` (20 stacked blocks,
T=64, one CUDA graph), `prefill` (T=131072 forward), `sublayer` (x + ffn(rmsnorm(x))), `ep` (experts
partitioned over the ranks under torchrun: `--ep-impl push | nccl`, `--routing uniform | hotspot`),
`ep-loopback` (the same step with virtual ranks on one GPU). `--skew literal1.5` switches the
headline's routing bias to the literal N(0, 1.5).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D_MODEL, N_EXPERTS, TOP_K, N_SHARED, D_FF, D_HIDDEN = 576, 76, 6, 2, 192, 128
TOKENS = 16384
# Per-expert logit bias N(0, std), seed 1. With router W ~ N(0, 0.02) the logits have std 0.48, so
# std 0.27 gives the expert-load CV ~ 1 that the workload describes (the default, and the headline);
# the literal std 1.5 gives CV ~ 3 with more than half of the experts empty (--skew literal1.5).
SKEWS = {"cv1": 0.27, "literal1.5": 1.5}
SKEW_NAME = "cv1"
BIAS_STD = SKEWS[SKEW_NAME]
N_INPUT_SETS = 8         # x / dOut pairs cycled through so successive steps do not hit L2
METRIC = "MoE-block tokens/s (fwd+bwd)"

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels that have
# been captured with ncu on this workload; see profiles/ncu_block_kernels_T16384.md and
# profiles/ncu_dW_in_dHidden_permute_T16384.md.
NCU_TRAFFIC_BYTES = {"permute (routed rows; shared experts read x in place)": 82.0e6,
                     "wgrad_in (gemm + reduce)": 243.2e6, "dhidden+glu_bwd": 285.7e6}
# (filled from the ncu summaries under profiles/; a kernel without a capture reports null)

FLOP_PER_TOKEN_FWD_BWD = 10_879_488   # 3 * (routed up 1 769 472 + down 884 736 + shared 884 736 + router 87 552)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


def init_weights(seed=0):
    """Draw order: x sets, router W, W_in, W_out, W_sh_in, W_sh_out, then the routing bias."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)
    w = {
        "router_W": rn(D_MODEL, N_EXPERTS) * 0.02,
        "W_in": rn(N_EXPERTS, D_MODEL, 2 * D_HIDDEN) * D_MODEL ** -0.5,
        "W_out": rn(N_EXPERTS, D_HIDDEN, D_MODEL) * D_HIDDEN ** -0.5,
        "W_sh_in": rn(N_SHARED, D_MODEL, 2 * D_HIDDEN) * D_MODEL ** -0.5,
        "W_sh_out": rn(N_SHARED, D_HIDDEN, D_MODEL) * D_HIDDEN ** -0.5,
    }
    bias = torch.randn(N_EXPERTS, generator=torch.Generator().manual_seed(1)) * BIAS_STD
    return {k: v.bfloat16() for k, v in w.items()}, bias


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))


    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) == 6] or \
               [r for _, r in self.rows if len(r) == 6]
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(names, r[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------- CPU arm
def cpu_steps(tokens, steps, warmup, threads):
    """Forward+backward of the oracle block on the host cores; returns (seconds per step, tokens)."""
    from oracle import moe_oracle as O
    torch.set_num_threads(threads)
    w, bias = init_weights()
    m = O.OracleBlock(D_MODEL, N_EXPERTS, D_FF, TOP_K, N_SHARED).to(torch.bfloat16)
    with torch.no_grad():
        m.router_W.copy_(w["router_W"])
        m.W_in.copy_(w["W_in"])
        m.W_out.copy_(w["W_out"])
        m.W_sh_in.copy_(w["W_sh_in"])
        m.W_sh_out.copy_(w["W_sh_out"])
    m.routing_bias = bias
    m.train()
    g = torch.Generator().manual_seed(2)
    x = torch.randn(tokens, D_MODEL, generator=g).bfloat16()
    dout = torch.randn(tokens, D_MODEL, generator=g).bfloat16()

    def step():
        for p in m.parameters():
            p.grad = None
        xi = x.clone().requires_grad_(True)
        out = m(xi)
        torch.autograd.backward([out, m.aux_loss], [dout, torch.ones(())])

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) / max(steps, 1)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    tokens = TOKENS
    # bound the run: one probe step decides how large a sample each step can be
    t_probe = cpu_steps(2048, 1, 1, threads)
    budget = 150.0 / max(args.steps + args.warmup, 1)
    while tokens > 2048 and t_probe * (tokens / 2048) > budget:
        tokens //= 2
    sec = cpu_steps(tokens, args.steps, args.warmup, threads)
    value = tokens / sec * 1.0
    sample = (f"{tokens} of {TOKENS} tokens per step, fwd+bwd, bf16, "
              f"torch {torch.__version__} CPU, {threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(args.gpus, tokens),
                       reference_scope="the CPU arm runs on rank 0's host cores only and its "
                                       "tokens/s does not depend on n_gpus: at n_gpus > 1 the "
                                       "ratio compares N GPUs with ONE host, not like for like"),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus, tokens_per_gpu=TOKENS):
    return {
        "workload": "BASELINE config 2: dropless MoE block fwd+bwd, T=16384 (8x2048) per GPU, "
                    "d_model 576, 76 routed + 2 shared SwiGLU experts, d_expert 128, top-6",
        "tokens_per_gpu": tokens_per_gpu, "global_tokens": tokens_per_gpu * n_gpus,
        "skew": f"{SKEW_NAME}: per-expert logit bias N(0,{BIAS_STD}), seed 1",
        "parallelism": f"token-sharded replicas x{n_gpus}: no collective on the data path" +
                       ("; the weight gradients are all-reduced over the ranks every step, "
                        "inside the timed region" if n_gpus > 1 else ""),
        "l2": f"{N_INPUT_SETS} input/dOut sets cycled (302 MB) and ~1 GB of intermediates per "
              "step, both beyond the 126 MB L2; no explicit flush",
    }


# --------------------------------------------------------------------------------- GPU arm
class _MeanLoss(torch.autograd.Function):
    """loss = mean(out) in fp32, the end-to-end loop's scalar. The loss is the root of the graph, so
    its incoming gradient is exactly 1 and d loss / d out is the constant 1 / numel: the backward
    hands out that constant tensor (kept per shape) instead of PyTorch's expand + divide + cast
    kernels, which cost the bench 30 us per step of glue that is not the block."""
    _const = {}

    @staticmethod
    def forward(ctx, out):
        ctx.key = (tuple(out.shape), out.dtype, out.device)
        if ctx.key not in _MeanLoss._const:
            _MeanLoss._const[ctx.key] = torch.full(out.shape, 1.0 / out.numel(), dtype=out.dtype,
                                                   device=out.device)
        return out.mean(dtype=torch.float32)

    @staticmethod
    def backward(ctx, grad):
        return _MeanLoss._const[ctx.key]


def mean_loss(out):
    return _MeanLoss.apply(out)


def build_block(device):
    from nanospeaker_b200 import MoEBlock
    w, bias = init_weights()
    m = MoEBlock(D_MODEL, N_EXPERTS, d_ff=D_FF, top_k=TOP_K, n_shared=N_SHARED,
                 capacity_factor=None).to(torch.bfloat16)
    with torch.no_grad():
        m.router.W.copy_(w["router_W"])
        m.W_in.copy_(w["W_in"])
        m.W_out.copy_(w["W_out"])
        m.W_sh_in.copy_(w["W_sh_in"])
        m.W_sh_out.copy_(w["W_sh_out"])
    m = m.to(device).train()
    m.router.logit_bias = bias.to(device)
    return m


def build_stages(m, x):
    """Every kernel of the step as a standalone callable with its algorithmic work per launch.
    Operands are rotated through 3 buffer copies so a launch does not find its input in L2."""
    from nanospeaker_b200 import kernels as K
    T, D, H, E, k, S = x.shape[0], D_MODEL, D_HIDDEN, N_EXPERTS, TOP_K, N_SHARED
    with torch.no_grad():
        w, idx, _ = m.router(x)
        logits = (x @ m.router.W).float() + m.router.logit_bias
        # the block dispatches the shared experts as experts E..E+S-1 that every token visits
        ids = torch.arange(E, E + S, device=x.device)
        idx_all = torch.cat([idx, ids.expand(T, S)], 1)
        w_all = torch.cat([w, w.new_ones((T, S))], 1)
        ka, Ea = k + S, E + S
        M = T * ka
        sids, eids, offs, counts, npp, inv = K.dispatch(idx_all, Ea)
        tw = w_all.reshape(-1).contiguous()
        copies = lambda t: [t.clone() for _ in range(3)]
        xr = copies(x)
        gather = (sids, ka)
        # as in the block op: the permute stops at the first shared run, the shared experts read
        # their rows from the token-major matrix itself
        live = offs[E:E + 1]
        Mr = T * k                                   # routed pairs: the rows the permute copies
        xs = copies(K.permute(x, ka, sids, npp))
        hid0, a1 = K.up_gemm(xs[0], m.W_in, eids, npp, 0, 0, True, w_extra=m.W_sh_in)
        hid = copies(hid0)
        y = copies(K.down_gemm(hid[0], m.W_out, eids, npp, 0, sids, tw, M, w_extra=m.W_sh_out))
        acc = [torch.zeros_like(x) for _ in range(3)]
        da1 = copies(K.dhidden_glu_bwd(xs[0], m.W_out, eids, npp, 0, sids, tw, M, a1, 0, True,
                                       w_extra=m.W_sh_out)[0])
        from nanospeaker_b200.moe_kernel import _router_ld
        ld = _router_ld(E)
        wp = x.new_zeros((1, D, ld))
        wp[0, :, :E] = m.router.W
        logits_p = K.down_gemm(x, wp, None, None, 1, None, None, 0)[0]
        bias = m.router.logit_bias
        _, _, colsum = K.router_fused(logits_p, bias, E, k, S, True, True)
        dtw = w_all.clone()
        d_aux = torch.ones(1, device=x.device)
        dl = copies(K.router_fused_bwd(logits_p, bias, idx_all, dtw, E, k, S, True, True, d_aux,
                                       counts, 1e-2, ld))

        gamma = torch.ones(D, device=x.device, dtype=x.dtype)
        _, rstd = K.rmsnorm(x, gamma, 1e-6)

        GE, TF = "hbm", "tensor"
        # One entry per kernel launch of the block op's forward + backward, in launch order.
        # M counts routed and shared pairs alike: (k + S) * T rows go through every expert GEMM.
        stages = [
            # name, bound, work per launch (bytes or flop), launches per step, callable(i)
            ("router GEMM x@W (padded to %d cols)" % ld, TF, 2.0 * T * D * E, 1,
             lambda i: K.down_gemm(xr[i % 3], wp, None, None, 1, None, None, 0)),
            ("router top-k + dispatch (2 kernels)", GE, T * ld * 2 + T * ka * 10 + M * 8 + M * 4 * 3, 1,
             lambda i: K.router_dispatch(logits_p, bias, E, k, S, True, True)),
            ("router_fused alone (top-k, softmax, colsum)", GE, T * ld * 2 + T * ka * 10, 0,
             lambda i: K.router_fused(logits_p, bias, E, k, S, True, True)),
            ("dispatch alone (histogram, plan + scatter)", GE, M * 8 * 2 + M * 4 * 3, 0,
             lambda i: K.dispatch(idx_all, Ea)),
            # compulsory traffic: x read once (its k + S re-reads hit L2), every slot row written
            ("permute (routed rows; shared experts read x in place)", GE,
             T * D * 2 + Mr * D * 2 + Mr * 4, 2,
             lambda i: K.permute(xr[i % 3], ka, sids, live)),
            ("permute, every row (without the shared-row shortcut)", GE,
             T * D * 2 + M * D * 2 + M * 4, 0,
             lambda i: K.permute(xr[i % 3], ka, sids, npp)),
            ("up_gemm+glu (+a1 saved)", TF, 2.0 * M * D * 2 * H, 1,
             lambda i: K.up_gemm(xs[i % 3], m.W_in, eids, npp, 0, 0, True, w_extra=m.W_sh_in,
                                 token_rows=(xr[i % 3], offs))),
            ("up_gemm+glu (gathered rows, inference)", TF, 2.0 * M * D * 2 * H, 0,
             lambda i: K.up_gemm(xr[i % 3], m.W_in, eids, npp, 0, 0, False, gather=gather,
                                 w_extra=m.W_sh_in)),
            # the step's default: the shared experts' rows (token-ordered, weight 1) are summed by a
            # plain-store GEMM that gives the token-major result its first value; the routed
            # experts' rows are then added to it in the down / dX GEMMs' epilogues (bf16 atomics in L2)
            ("down_gemm shared experts (stores; first value of out)", TF, 2.0 * T * S * H * D, 1,
             lambda i: K.down_gemm_sum(hid[i % 3], m.W_sh_out, offs[E:], T, out=acc[i % 3])),
            ("down_gemm+scale+combine (routed rows, atomic adds into out)", TF,
             2.0 * T * k * H * D, 1,
             lambda i: K.down_gemm_acc(hid[i % 3], m.W_out, eids, offs[E:E + 1], 0, sids, tw, M, ka,
                                       acc[i % 3])),
            # the store-then-reduce alternative (combine mode "store"): not part of the default step
            ("down_gemm+scale (stores per-pair rows)", TF, 2.0 * M * H * D, 0,
             lambda i: K.down_gemm(hid[i % 3], m.W_out, eids, npp, 0, sids, tw, M,
                                   w_extra=m.W_sh_out)),
            ("combine (store mode)", GE, M * D * 2 + M * 4 + T * D * 2, 0,
             lambda i: K.combine(y[i % 3], inv, T, ka)),
            ("balance_loss", GE, E * 8, 1, lambda i: K.balance_loss(colsum, counts, E, T, 1e-2)),
            ("dhidden+glu_bwd", TF, 2.0 * M * D * H, 1,
             lambda i: K.dhidden_glu_bwd(xs[i % 3], m.W_out, eids, npp, 0, sids, tw, M, a1, 0,
                                         True, w_extra=m.W_sh_out,
                                         token_rows=(xr[i % 3], offs))),
            ("dhidden+glu_bwd (gathered rows)", TF, 2.0 * M * D * H, 0,
             lambda i: K.dhidden_glu_bwd(xr[i % 3], m.W_out, eids, npp, 0, sids, tw, M, a1, 0,
                                         True, gather_top_k=ka, w_extra=m.W_sh_out)),
            ("dx_gemm shared experts (stores; first value of dx)", TF, 2.0 * T * S * 2 * H * D, 1,
             lambda i: K.dx_gemm_sum(da1[i % 3], m.W_sh_in, offs[E:], T, out=acc[i % 3])),
            ("dx_gemm+combine (routed rows, atomic adds into dx)", TF, 2.0 * T * k * 2 * H * D, 1,
             lambda i: K.dx_gemm_acc(da1[i % 3], m.W_in, eids, offs[E:E + 1], 0, sids, M, ka,
                                     acc[i % 3], pad_offsets=offs[:E + 1])),
            ("dx_gemm (stores per-pair rows)", TF, 2.0 * M * 2 * H * D, 0,
             lambda i: K.dx_gemm(da1[i % 3], m.W_in, eids, npp, 0, w_extra=m.W_sh_in)),
            ("wgrad_in (gemm + reduce)", TF, 2.0 * M * D * 2 * H, 1,
             lambda i: K.wgrad(xs[i % 3], da1[i % 3], offs, Ea, n_extra=S,
                               token_rows=("a", xr[i % 3]))),
            ("wgrad_out (gemm + reduce)", TF, 2.0 * M * H * D, 1,
             lambda i: K.wgrad(hid[i % 3], xs[i % 3], offs, Ea, n_extra=S,
                               token_rows=("b", xr[i % 3]))),
            ("wgrad_in (gathered rows)", TF, 2.0 * M * D * 2 * H, 0,
             lambda i: K.wgrad(xr[i % 3], da1[i % 3], offs, Ea, gather=("a", sids, ka), n_extra=S)),
            ("wgrad_out (gathered rows)", TF, 2.0 * M * H * D, 0,
             lambda i: K.wgrad(hid[i % 3], xr[i % 3], offs, Ea, gather=("b", sids, ka), n_extra=S)),
            ("rmsnorm forward (FFN sublayer only)", GE, 2 * T * D * 2, 0,
             lambda i: K.rmsnorm(xr[i % 3], gamma, 1e-6)),
            ("rmsnorm backward + residual gradient (FFN sublayer only)", GE, 4 * T * D * 2, 0,
             lambda i: K.rmsnorm_bwd(xr[(i + 1) % 3], xr[i % 3], rstd, gamma, add=xr[(i + 2) % 3])),
            ("router_fused_bwd", GE, T * ld * 2 * 2 + T * ka * 10, 1,
             lambda i: K.router_fused_bwd(logits_p, bias, idx_all, dtw, E, k, S, True, True,
                                          d_aux, counts, 1e-2, ld)),
            ("router wgrad x^T@dl (gemm + reduce)", TF, 2.0 * T * D * E, 1,
             lambda i: K.wgrad(xr[i % 3], dl[i % 3], None, 1)),
            ("router dx dl@W^T (atomic adds into dx)", TF, 2.0 * T * D * E, 1,
             lambda i: K.dx_gemm_acc(dl[i % 3].unsqueeze(0), wp, None, None, 1, None, 0, 1,
                                     acc[i % 3])),
        ]
    return stages


def gemm_stage_bytes(T, ld):
    """Compulsory HBM bytes per launch of the GEMM stages: every operand read once, every output
    written once (bf16). The GEMMs of this block sit below the ridge of the measured roofline
    (about 250 flop per byte), so this floor, not the tensor peak, is what bounds them."""
    D, H, k, S = D_MODEL, D_HIDDEN, TOP_K, N_SHARED
    M, G = T * (k + S), N_EXPERTS + S
    w_in, w_out = G * D * 2 * H * 2, G * H * D * 2
    return {
        "router GEMM": T * D * 2 + D * ld * 2 + T * ld * 2,
        "up_gemm+glu (+a1 saved)": M * D * 2 + w_in + M * 3 * H * 2,
        "up_gemm+glu (gathered rows, inference)": T * D * 2 + w_in + M * H * 2,
        "down_gemm+scale (stores": M * H * 2 + w_out + M * D * 2,
        # atomic variants: no per-pair rows; the token-major result is read and written once in HBM
        "down_gemm+scale+combine": T * k * H * 2 + N_EXPERTS * H * D * 2 + 2 * T * D * 2,
        "dx_gemm+combine": T * k * 2 * H * 2 + N_EXPERTS * D * 2 * H * 2 + 2 * T * D * 2,
        "down_gemm shared experts": T * S * H * 2 + S * H * D * 2 + T * D * 2,
        "dx_gemm shared experts": T * S * 2 * H * 2 + S * D * 2 * H * 2 + T * D * 2,
        "dhidden+glu_bwd": M * D * 2 + M * 2 * H * 2 + w_out + M * 3 * H * 2 + M * 2,
        "dx_gemm (stores": M * 2 * H * 2 + w_in + M * D * 2,
        "wgrad_in (gemm + reduce)": M * D * 2 + M * 2 * H * 2 + w_in,
        "wgrad_out (gemm + reduce)": M * H * 2 + M * D * 2 + w_out,
    }


def stage_rooflines(m, x, pk):
    """Time every kernel of the step alone (CUDA events on the current stream) and put each next
    to its algorithmic work."""
    GE = "hbm"
    stages = build_stages(m, x)
    from nanospeaker_b200.moe_kernel import _router_ld
    floor_bytes = gemm_stage_bytes(x.shape[0], _router_ld(N_EXPERTS))
    with torch.no_grad():
        out = []
        for name, bound, work, per_step, fn in stages:
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
            # n launches captured in a CUDA graph and replayed: the host cost of a call (argument
            # checks, output allocation) would otherwise hide the device time of the small kernels
            n = 12
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(n):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / n * 1e3
            del g
            if bound == GE:
                ach, peak, unit = work / us / 1e3, pk["hbm_gbs"], "GB/s"
            else:
                ach, peak, unit = work / us / 1e6, pk["bf16_tflops"], "TFLOP/s"
            out.append({"kernel": name, "bound": bound, "us": round(us, 2),
                        "launches_per_step": per_step, "achieved": round(ach, 1), "peak": peak,
                        "unit": unit, "frac": round(ach / peak, 4)})
            hb = next((b for key, b in floor_bytes.items() if name.startswith(key)), None)
            if hb is not None:      # a GEMM stage: its HBM byte floor beside the tensor fraction
                out[-1]["hbm_bytes"] = hb
                out[-1]["hbm_gbs"] = round(hb / us / 1e3, 1)
                out[-1]["hbm_frac"] = round(hb / us / 1e3 / pk["hbm_gbs"], 4)
    return out


def run_ours(args):
    import torch.distributed as dist
    from nanospeaker_b200 import kernels as K

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE block has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()

    m = build_block(dev)
    if args.profile_stage:
        # for `ncu -k ...`: launch one stage's kernel a few times on the bench workload and leave
        x = torch.randn(TOKENS, D_MODEL, generator=torch.Generator().manual_seed(100)).bfloat16()
        hits = [s for s in build_stages(m, x.to(dev)) if args.profile_stage in s[0]]
        if not hits:
            raise SystemExit(f"no stage matches {args.profile_stage!r}")
        with torch.no_grad():
            for i in range(3):
                hits[0][4](i)
        torch.cuda.synchronize()
        K.check_status(dev)
        print(json.dumps({"profiled_stage": hits[0][0], "launches": 3}))
        return
    g = torch.Generator().manual_seed(100 + rank)      # every rank has its own token shard
    host_x = [torch.randn(TOKENS, D_MODEL, generator=g).bfloat16().pin_memory()
              for _ in range(N_INPUT_SETS)]
    dev_x = [h.to(dev) for h in host_x]
    dev_dout = [torch.randn(TOKENS, D_MODEL, generator=g).bfloat16().to(dev)
                for _ in range(N_INPUT_SETS)]
    one = torch.ones((), device=dev)
    params = list(m.parameters())

    def step(i):
        for p in params:
            p.grad = None
        x = dev_x[i % N_INPUT_SETS].detach().requires_grad_(True)
        out = m(x)
        torch.autograd.backward([out, m.aux_loss], [dev_dout[i % N_INPUT_SETS], one])
        if world > 1 and not args.no_grad_allreduce:
            from nanospeaker_b200.parallel import all_reduce_gradients
            all_reduce_gradients(params)

    # The step has no host sync and no data-dependent shape, so the whole forward+backward is
    # captured once into a CUDA graph and replayed: the ~60 launches of a step then cost one
    # submission instead of ~1 ms of Python and launch overhead.
    static_x = dev_x[0].clone().requires_grad_(True)
    static_dout = dev_dout[0].clone()

    def capture(with_loss, static_x=static_x, static_dout=static_dout):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                for p in params:
                    p.grad = None
                static_x.grad = None
                out = m(static_x)
                if with_loss:
                    (mean_loss(out) + m.aux_loss).backward()
                else:
                    torch.autograd.backward([out, m.aux_loss], [static_dout, one])
        torch.cuda.current_stream().wait_stream(side)
        # Drop every reference to earlier autograd graphs (the block keeps its last aux_loss):
        # their AccumulateGrad nodes are tied to the stream they ran on and would pull that
        # stream into the capture.
        del out
        m.aux_loss = torch.zeros((), device=dev)
        for p in params:
            p.grad = None
        static_x.grad = None
        graph = torch.cuda.CUDAGraph()
        l0 = K.LAUNCHES
        with torch.cuda.graph(graph):
            out = m(static_x)
            if with_loss:
                loss = mean_loss(out) + m.aux_loss
                loss.backward()
            else:
                loss = None
                torch.autograd.backward([out, m.aux_loss], [static_dout, one])
        # the gradients this graph writes (its own static tensors, rewritten by every replay)
        grads = [p.grad for p in params if p.grad is not None]
        return graph, loss, K.LAUNCHES - l0, grads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms, t0, time.time()

    torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
    warmup = max(args.warmup, 3)
    use_graph = not args.no_graph
    # N > 1: the data-parallel training step. Every rank's weight gradients (34.6 MB in bf16) are
    # summed over the ranks inside the timed region: the step's graph is replayed, then the flattened
    # bucket is all-reduced on a communication stream under the NEXT step's compute (what a trainer
    # does between two micro-steps) -- by device-to-device copies through peer memory (up to 4
    # ranks) or by NCCL (--grad-allreduce-impl); the barrier that ends the timed region waits for
    # the last one. --no-grad-allreduce times the bare replicas instead.
    with_comm = world > 1 and not args.no_grad_allreduce
    eager_ms, _, _ = timed(step, args.steps, warmup)
    if use_graph:
        # value: one graph per resident input set (the sets are cycled so that no step finds its
        # input in L2); nothing but the graph replay is inside a timed step
        # (the graphs hold raw pointers: their input tensors must stay alive next to them)
        value_x = [dev_x[i].clone().requires_grad_(True) for i in range(N_INPUT_SETS)]
        graph_sets = [capture(False, value_x[i], dev_dout[i]) for i in range(N_INPUT_SETS)]
        per_step_launches = graph_sets[0][2]

        comm_stream = torch.cuda.Stream()
        computed = torch.cuda.Event()
        flattened = {}    # per graph / gradient-buffer set: its last flatten copy
        n_grad = sum(g.numel() for g in graph_sets[0][3])
        bucket = torch.empty(n_grad, dtype=torch.bfloat16, device=dev)
        peer_ar = None
        impl = args.grad_allreduce_impl
        if impl == "auto":
            impl = "peer" if world <= 4 else "nccl"
        if with_comm and impl == "peer":
            # the sum through peer memory and the copy engines (parallel.PeerGradAllReduce): no
            # collective kernel sits on SMs the persistent GEMMs want; NCCL if it cannot be set up
            try:
                from nanospeaker_b200.parallel import PeerGradAllReduce
                peer_ar = PeerGradAllReduce(n_grad, dev)
            except Exception as exc:       # symmetric memory unavailable on this box
                if rank == 0:
                    print(f"peer-memory all-reduce unavailable ({exc}); using NCCL", file=sys.stderr)

        def reduce_grads(grads, key):
            """Flatten this step's gradients into the bucket and all-reduce it, on the
            communication stream. Every graph owns its gradient buffers, so the compute stream
            does not wait here: a graph waits for ITS last flatten copy before it is replayed
            again (`before_replay`), several steps later."""
            computed.record()
            with torch.cuda.stream(comm_stream):
                comm_stream.wait_event(computed)
                if peer_ar is not None:
                    peer_ar.fill(grads)
                else:
                    torch.cat([g.reshape(-1) for g in grads], out=bucket)
                flattened.setdefault(key, torch.cuda.Event()).record(comm_stream)
                if peer_ar is not None:
                    peer_ar()
                else:
                    dist.all_reduce(bucket)

        def before_replay(key):
            if key in flattened:
                torch.cuda.current_stream().wait_event(flattened[key])

        def replica_step(i):
            graph_sets[i % N_INPUT_SETS][0].replay()

        def value_step(i):
            if with_comm:
                before_replay(("value", i % N_INPUT_SETS))
            graph_sets[i % N_INPUT_SETS][0].replay()
            if with_comm:
                reduce_grads(graph_sets[i % N_INPUT_SETS][3], ("value", i % N_INPUT_SETS))

        # e2e: two input buffers / graphs in ping-pong. The pinned-host -> device copy of step i+1
        # runs on a copy stream while step i computes (what an input pipeline does), and the loss
        # of step i is copied to pinned host memory on that stream too and read by the host one
        # step later (what a logging training loop does), so the device never waits for the host.
        e2e_x = [static_x, dev_x[1].clone().requires_grad_(True)]
        e2e_graphs = [capture(with_loss=True, static_x=bx) for bx in e2e_x]
        copy_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
        copied = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        loss_read = [torch.cuda.Event(), torch.cuda.Event()]
        loss_host = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]

        def prefetch(i):
            b = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[b])       # the graph that read this buffer is done
                e2e_x[b].detach().copy_(host_x[i % N_INPUT_SETS], non_blocking=True)
                copied[b].record(copy_stream)

        state = {"next": None, "pending": None}

        def e2e_step(i):
            b = i % 2
            if state["next"] != i:                        # first step of a run: nothing prefetched
                prefetch(i)
                state["pending"] = None
            torch.cuda.current_stream().wait_event(copied[b])
            if with_comm:
                before_replay(("e2e", b))
            e2e_graphs[b][0].replay()
            consumed[b].record()
            if with_comm:
                reduce_grads(e2e_graphs[b][3], ("e2e", b))
            prefetch(i + 1)                               # H2D of the next step's input
            with torch.cuda.stream(d2h_stream):           # D2H of this step's loss
                d2h_stream.wait_event(consumed[b])
                loss_host[b].copy_(e2e_graphs[b][1].detach(), non_blocking=True)
                loss_read[b].record(d2h_stream)
            state["next"] = i + 1
            prev, state["pending"] = state["pending"], b
            if prev is None:
                return None
            loss_read[prev].synchronize()                 # the previous step's loss has arrived
            return float(loss_host[prev])
    else:
        value_step = replica_step = step
        l0 = K.LAUNCHES
        step(0)
        per_step_launches = K.LAUNCHES - l0

        def e2e_step(i):
            for p in params:
                p.grad = None
            x = host_x[i % N_INPUT_SETS].to(dev, non_blocking=True).requires_grad_(True)
            out = m(x)
            loss = mean_loss(out) + m.aux_loss
            loss.backward()
            return loss.item()

    sampler = ClockSampler(local)     # started well ahead of the timed region it is read for
    replica_ms = comm_ms = None
    if with_comm and use_graph:
        replica_ms, _, _ = timed(replica_step, args.steps, warmup)
        # the all-reduce alone, back to back on the communication stream
        def comm_only(i):
            with torch.cuda.stream(comm_stream):
                if peer_ar is not None:
                    peer_ar()
                else:
                    dist.all_reduce(bucket)
            torch.cuda.current_stream().wait_stream(comm_stream)
        comm_ms, _, _ = timed(comm_only, args.steps, warmup)
    # the same step through the package's graph wrapper (what a trainer calls instead of the bench's
    # own capture): GraphedMoEBlock.forward + autograd backward, forward and backward each a replay
    graphed_ms = None
    if use_graph:
        from nanospeaker_b200 import GraphedMoEBlock
        gm = GraphedMoEBlock(m)

        def graphed_step(i):
            for p in params:
                p.grad = None
            x = dev_x[i % N_INPUT_SETS].detach().requires_grad_(True)
            out = gm(x)
            torch.autograd.backward([out, gm.aux_loss], [dev_dout[i % N_INPUT_SETS], one])
        graphed_ms, _, _ = timed(graphed_step, args.steps, warmup)
    ms, t0, t1 = timed(value_step, args.steps, warmup)
    launches = per_step_launches * args.steps
    # K steps last ~10 ms, less than one nvidia-smi sampling period (and eight ranks starting
    # nvidia-smi at once take a while to print their first line): the identical step keeps running,
    # untimed, until the sampler has seen the GPU under this load for about half a second
    # (the same number of extra steps on every rank: they contain collectives)
    n_extra = int(500.0 / max(ms / args.steps, 1e-3)) + 1
    for i_extra in range(n_extra):
        value_step(args.steps + i_extra)
        if i_extra % 64 == 63:
            torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop(t0, time.time())
    clocks["window"] = "the timed steps and ~0.5 s of the same step replayed after them"
    K.check_status(dev)
    e2e_ms, _, _ = timed(e2e_step, args.steps, warmup)

    value = TOKENS * world * args.steps / (ms / 1e3)
    e2e_value = TOKENS * world * args.steps / (e2e_ms / 1e3)

    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": e2e_value, "unit": "tokens/s",
                    "h2d_bytes_per_step": TOKENS * D_MODEL * 2, "d2h_bytes_per_step": 4,
                    "h2d_gbs_per_rank": TOKENS * D_MODEL * 2 / (e2e_ms / args.steps * 1e-3) / 1e9,
                    "ms_per_step": e2e_ms / args.steps,
                    "how": "MoEBlock.forward + loss.backward captured in a CUDA graph; every "
                           "step copies its x from pinned host memory (on a copy stream, "
                           "overlapping the previous step) and copies its loss to pinned host "
                           "memory, which the host reads one step later"},
            "gpu_launches": launches, "clocks": clocks,
            "pct_bf16_peak": {"measured_burst": 100 * value / world * FLOP_PER_TOKEN_FWD_BWD
                              / (pk["bf16_tflops"] * 1e12),
                              "nominal_2250": 100 * value / world * FLOP_PER_TOKEN_FWD_BWD / 2.25e15},
            "grad_allreduce": bool(with_comm),
            "cuda_graph": use_graph,
            "eager_ms_per_step": eager_ms / args.steps,
            "graphed_module_ms_per_step": None if graphed_ms is None else graphed_ms / args.steps,
        }
        if with_comm and replica_ms is not None:
            line["grad_allreduce_detail"] = {
                "what": "weight gradients of the block summed over the ranks: one flattened bf16 "
                        "bucket, " + ("reduce-scatter + all-gather by device-to-device copies "
                                      "through peer memory (copy engines) with a local fp32 sum"
                                      if peer_ar is not None else "ncclAllReduce")
                        + " on a communication stream under the next step's compute; inside the "
                          "timed region",
                "how": "peer" if peer_ar is not None else "nccl",
                "bytes": int(n_grad) * 2,
                "allreduce_alone_ms": comm_ms / args.steps,
                "allreduce_bus_gbs": 2 * (world - 1) / world * n_grad * 2 / (comm_ms / args.steps * 1e-3) / 1e9,
                "replicas_only_ms_per_step": replica_ms / args.steps,
                "replicas_only_value": TOKENS * world * args.steps / (replica_ms / 1e3)}
        if not args.no_stages:
            stages = stage_rooflines(m, dev_x[0], pk)
            top = max(stages, key=lambda s: s["us"] * s["launches_per_step"])
            line["roofline"] = {"kernel": top["kernel"], "bound": top["bound"],
                                "achieved": top["achieved"], "peak": top["peak"],
                                "unit": top["unit"], "frac": top["frac"],
                                "traffic": NCU_TRAFFIC_BYTES.get(top["kernel"]),
                                "peak_source": pk["source"] + " (burst: kernel timed alone)",
                                "algorithmic_work": "flop (or bytes) per token of the stage x "
                                                    f"{TOKENS} tokens, pad rows and recompute not counted"}
            if "hbm_frac" in top:
                # A GEMM stage is reported against the tensor roof. Next to it, as extra keys, the
                # stage's time against the HBM bytes THIS DESIGN moves for it (operands read once,
                # outputs written once, materialised intermediates included): that byte count is
                # the design's, not algorithmic work.
                work_flop = top["achieved"] * 1e12 * top["us"] * 1e-6
                line["roofline"].update({
                    "design_hbm_bytes": top["hbm_bytes"], "design_hbm_gbs": top["hbm_gbs"],
                    "design_hbm_frac": top["hbm_frac"],
                    "flop_per_design_hbm_byte": round(work_flop / top["hbm_bytes"], 1),
                    "ridge_flop_per_byte": round(pk["bf16_tflops"] * 1e12 / (pk["hbm_gbs"] * 1e9), 1)})
            line["stages"] = stages
    if world > 1:
        dist.barrier()
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            sec = cpu_steps(TOKENS, 3, 1, threads)
            line["cpu_baseline"] = {
                "value": TOKENS / sec, "unit": "tokens/s", "cores": threads, "kind": "port",
                "sample": f"full T={TOKENS} fwd+bwd, 1 warm-up + 3 timed steps, bf16, "
                          f"torch {torch.__version__} CPU"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def ep_phase_times(grp, m, x, gout, w_in, w_out, dev, world, dist, reps=5):
    """Where the peer-memory step's time goes on every rank: each phase of the step (the calls
    between two phase boundaries) is captured in a CUDA graph of its own and the graphs are replayed
    in order with a CUDA event between them, so the figures are device time, not the eager launch
    time of eight Python processes on one host. Pushes and pulls are NVLink phases, owner phases are
    GEMMs, a boundary's time is the wait for the slowest rank. Returns per-rank milliseconds per
    phase and the rows each rank owns."""
    me = grp.me
    cast = lambda t: t.detach().to(x.dtype).contiguous()
    bias = m.router.logit_bias
    bias = None if bias is None else bias.to(torch.float32).contiguous()
    w_sh_in, w_sh_out = cast(m.W_sh_in), cast(m.W_sh_out)
    wi, wo = cast(w_in), cast(w_out)
    keep = {}

    def route():
        keep["cnt"] = grp.gather_counts(me.f1_route(x.detach(), m.router.W.detach(), bias,
                                                    bool(m.router.normalize_weights), False))
        me.f3_shared(w_sh_in, w_sh_out, "silu", True)
        torch.cuda.current_stream().wait_stream(me.side)   # a graph must join what it forks

    def push_dout():
        me.b1_push(gout)
        torch.cuda.current_stream().wait_stream(me.side)

    def pull_y():      # (the pulls join the side stream: bring it into this graph first)
        me.side.wait_stream(torch.cuda.current_stream())
        keep["out"] = me.f4_pull(0.0)

    def pull_dx():
        me.side.wait_stream(torch.cuda.current_stream())
        keep["dx"] = me.b3_pull(None)

    seq = [("route + counts all-gather", route),
           ("push x", lambda: me.f2_push(keep["cnt"])),
           ("boundary 1", grp.boundary),
           ("owner fwd", lambda: me.f3_experts(wi, wo, w_sh_in, w_sh_out, "silu", True)),
           ("boundary 2", grp.boundary),
           ("pull y", pull_y),
           ("push dOut", push_dout),
           ("boundary 3", grp.boundary),
           ("owner bwd", me.b2_experts),
           ("boundary 4", grp.boundary),
           ("pull dX + router bwd", pull_dx)]
    graphs = []
    for name, fn in seq:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()                                  # warm-up outside capture
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        graphs.append(g)
    dist.barrier()
    torch.cuda.synchronize()
    total = [0.0] * len(seq)
    for it in range(reps + 1):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(seq) + 1)]
        for i, g in enumerate(graphs):
            evs[i].record()
            g.replay()
        evs[-1].record()
        torch.cuda.synchronize()
        if it > 0:
            for i in range(len(seq)):
                total[i] += evs[i].elapsed_time(evs[i + 1]) / reps
    local = torch.tensor(total + [float(me.own_npp.item())], device=dev)
    every = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(every, local)
    table = torch.stack(every).cpu()
    return {"per_rank_ms": {n: [round(float(v), 3) for v in table[:, i]]
                            for i, (n, _) in enumerate(seq)},
            "rows_owned_per_rank": [int(v) for v in table[:, -1]],
            "method": "one CUDA graph per phase, CUDA events between the replays; the shared "
                      "experts' forward / backward (side stream in the real step, under the push "
                      "and the boundary) are joined inside 'route' / 'push dOut' here"}


def ep_nvlink_roofline(phases, T, world):
    """The push / pull phases against the NVLink roof: bytes that cross the links per rank and
    direction (a row per routed pair whose owner is another rank: the (world - 1) / world share
    under uniform routing; a pushed row carries its slot id and router weight) over the slowest
    rank's phase time, against the measured peer-copy bandwidth of this pool (770 GB/s per
    direction, nominal 900)."""
    if not phases:
        return None
    remote = T * TOP_K * (world - 1) / world
    row = D_MODEL * 2
    out = {"bound": "nvlink", "peak": 770.0, "unit": "GB/s per direction per GPU",
           "peak_source": "measured peer copy on this pool (nominal 900)"}
    for key, name, extra in (("push_x", "push x", 6), ("pull_y", "pull y", 0),
                             ("push_dout", "push dOut", 0), ("pull_dx", "pull dX + router bwd", 0)):
        ms = max(phases["per_rank_ms"][name])
        out[key] = {"bytes_per_rank": int(remote * (row + extra)), "ms": ms,
                    "achieved": round(remote * (row + extra) / (ms * 1e-3) / 1e9, 1),
                    "frac": round(remote * (row + extra) / (ms * 1e-3) / 1e9 / 770.0, 3)}
    return out


def run_ep_workload(args):
    """BASELINE config 5: expert-parallel forward + backward. 76 routed experts partitioned over the
    ranks, shared experts and router replicated, T=65536 tokens per GPU, uniform or hot-spot routing (--routing). One rank
    per GPU under torchrun; eager launches (the split sizes of the all-to-all are read on the
    host); CUDA events, max over ranks."""
    import torch.distributed as dist
    from nanospeaker_b200 import MoEBlock, expert_parallel as EP, kernels as K
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--workload ep needs torchrun with at least 2 ranks")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    T = 65536
    w, _ = init_weights()
    m = MoEBlock(D_MODEL, N_EXPERTS, d_ff=D_FF, top_k=TOP_K, n_shared=N_SHARED,
                 capacity_factor=None).to(torch.bfloat16)
    with torch.no_grad():
        m.router.W.copy_(w["router_W"])
        m.W_sh_in.copy_(w["W_sh_in"])
        m.W_sh_out.copy_(w["W_sh_out"])
    m = m.to(dev).eval()           # eval: top-k softmax router, no balance loss in this workload
    if args.routing == "hotspot":
        # +1.14 on the logits of experts 0..3 gives them 0.50 of all assignments with this router
        # initialisation (1.10 -> 0.487, 1.15 -> 0.506); all four belong to rank 0
        hot = torch.zeros(N_EXPERTS, device=dev)
        hot[:4] = 1.14
        m.router.logit_bias = hot
    lo, hi = EP.expert_partition(N_EXPERTS, world)[rank]
    w_in = w["W_in"][lo:hi].bfloat16().to(dev).requires_grad_(True)
    w_out = w["W_out"][lo:hi].bfloat16().to(dev).requires_grad_(True)
    g = torch.Generator().manual_seed(100 + rank)
    xs = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev).requires_grad_(True)
          for _ in range(2)]
    gout = torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev)
    replicated = [m.router.W, m.W_sh_in, m.W_sh_out]

    push = args.ep_impl == "push"
    if push:
        from nanospeaker_b200 import ep_push
        grp = ep_push.SymmetricGroup(N_EXPERTS, TOP_K, N_SHARED, D_MODEL, T, dev)

    def step(i):
        x = xs[i % 2]
        x.grad = None
        if push:
            out, _, _ = ep_push.ep_push_block_forward(x, m.router, w_in, w_out, m.W_sh_in,
                                                      m.W_sh_out, "silu", grp)
        else:
            out, _ = EP.ep_block_forward(x, m.router, w_in, w_out, m.W_sh_in, m.W_sh_out, "silu")
        out.backward(gout)
        EP.all_reduce_replicated_grads(replicated)

    steps, warmup = args.steps, max(args.warmup, 3)
    for i in range(warmup):
        step(i)
    dist.barrier()
    torch.cuda.synchronize()
    use_graph = push and not args.no_graph
    run = step
    if use_graph:
        # The peer-memory step has no host read and no data-dependent shape: forward + backward of
        # both input sets are captured once (collectives included) and replayed, so the ~70
        # launches of a step cost one submission (eight eager ranks on one host are launch-bound).
        graphs = []
        for i in range(2):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(i)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g_i = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_i):
                step(i)
            graphs.append(g_i)
        run = lambda i: graphs[i % 2].replay()
        for i in range(3):
            run(i)
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        run(warmup + i)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t) / steps
    K.check_status(dev)
    phases = None
    if push:
        phases = ep_phase_times(grp, m, xs[0], gout, w_in, w_out, dev, world, dist)
    if rank == 0:
        print(json.dumps({
            "metric": "MoE-block tokens/s (fwd+bwd, expert parallel)",
            "value": T * world / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "BASELINE config 5: experts partitioned over the ranks, "
                                   f"T={T} tokens per GPU, {args.routing} routing, forward + backward, "
                                   + ("rows pushed into / pulled from the owners' buffers "
                                      "through peer pointers (symmetric memory)" if push else
                                      "dispatch / combine by NCCL all-to-all")},
            "cuda_graph": use_graph, "phases": phases,
            "roofline": ep_nvlink_roofline(phases, T, world)}), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    # Tear-down. With the step captured in CUDA graphs (NCCL collectives and symmetric-memory
    # buffers inside), destroy_process_group() does not return: neither with the graphs alive nor
    # after releasing the graphs and the exchange buffers first (tried; both ranks then sit in the
    # tear-down until the launcher's timeout). The results are out and every rank has passed the
    # barrier, so a graph run leaves directly.
    if use_graph:
        sys.stdout.flush()
        os._exit(0)
    dist.destroy_process_group()


def run_ep_loopback(args):
    """The peer-memory expert-parallel step with G virtual ranks on ONE GPU (`--gpus G`, default 2):
    every "peer" buffer is local, so this times the kernels and the plan without NVLink, phase by
    phase (CUDA events; ms per rank), and gives ncu something to capture on a single GPU."""
    from nanospeaker_b200 import MoEBlock, ep_push, kernels as K
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    world, T = max(args.gpus, 2), args.ep_tokens
    w, _ = init_weights()
    m = MoEBlock(D_MODEL, N_EXPERTS, d_ff=D_FF, top_k=TOP_K, n_shared=N_SHARED,
                 capacity_factor=None).to(torch.bfloat16)
    with torch.no_grad():
        for name in ("W_in", "W_out", "W_sh_in", "W_sh_out"):
            getattr(m, name).copy_(w[name])
        m.router.W.copy_(w["router_W"])
    m = m.to(dev).eval()
    grp = ep_push.LoopbackGroup(world, N_EXPERTS, TOP_K, N_SHARED, D_MODEL, T, dev)
    g = torch.Generator().manual_seed(100)
    xs = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev) for _ in range(world)]
    gs = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev) for _ in range(world)]
    R = grp.ranks
    names = ["route", "plan + push x", "owner fwd", "pull y", "push dOut", "owner bwd",
             "pull dX + router bwd"]
    total = [0.0] * len(names)
    steps, warmup = args.steps, max(args.warmup, 3)
    W_in, W_out = m.W_in.detach(), m.W_out.detach()
    local = [(W_in[r.lo:r.hi].contiguous(), W_out[r.lo:r.hi].contiguous()) for r in R]
    for it in range(warmup + steps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        e[0].record()
        cnt = torch.stack([r.f1_route(x, m.router.W.detach(), None, True, False)
                           for r, x in zip(R, xs)])
        e[1].record()
        for r in R:
            r.f2_push(cnt)
        e[2].record()
        for r, (wi, wo) in zip(R, local):
            r.f3_experts(wi, wo, m.W_sh_in.detach(), m.W_sh_out.detach(), "silu", True)
        e[3].record()
        for r in R:
            r.f4_pull(0.0)
        e[4].record()
        for r, go in zip(R, gs):
            r.b1_push(go)
        e[5].record()
        for r in R:
            r.b2_experts()
        e[6].record()
        for r in R:
            r.b3_pull()
        e[7].record()
        torch.cuda.synchronize()
        if it >= warmup:
            for i in range(len(names)):
                total[i] += e[i].elapsed_time(e[i + 1]) / world / steps
    K.check_status(dev)
    print(json.dumps({
        "metric": "expert-parallel step, virtual ranks on one GPU (ms per rank)",
        "value": sum(total), "unit": "ms", "higher_is_better": False, "n_gpus": 1,
        "steps": steps, "warmup": warmup,
        "config": {"workload": f"{world} virtual ranks x T={T} tokens, 76 experts partitioned, "
                               "forward + backward, peer buffers local (no NVLink)"},
        "phases_ms_per_rank": {n: round(v, 3) for n, v in zip(names, total)}}))


def run_side_workload(args):
    """The two forward-only workloads of the block's other callers, one JSON line each (not the
    headline): `decode` = 20 stacked blocks on T=64 tokens replayed from one CUDA graph
    (BASELINE config 3), `prefill` = one block on T=131072 tokens (BASELINE config 4, one GPU's
    view). Single GPU."""
    from nanospeaker_b200 import MoEBlock, kernels as K
    from nanospeaker_b200.decode import StackedMoEDecoder
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE block has no CPU implementation")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    steps, warmup = args.steps, max(args.warmup, 3)

    def make_block(seed):
        g = torch.Generator().manual_seed(seed)
        r = lambda *sh: torch.randn(*sh, generator=g)
        m = MoEBlock(D_MODEL, N_EXPERTS, d_ff=D_FF, top_k=TOP_K, n_shared=N_SHARED,
                     capacity_factor=None).to(torch.bfloat16)
        with torch.no_grad():
            m.router.W.copy_(r(D_MODEL, N_EXPERTS) * 0.02)
            m.W_in.copy_(r(N_EXPERTS, D_MODEL, 2 * D_HIDDEN) * D_MODEL ** -0.5)
            m.W_out.copy_(r(N_EXPERTS, D_HIDDEN, D_MODEL) * D_HIDDEN ** -0.5)
            m.W_sh_in.copy_(r(N_SHARED, D_MODEL, 2 * D_HIDDEN) * D_MODEL ** -0.5)
            m.W_sh_out.copy_(r(N_SHARED, D_HIDDEN, D_MODEL) * D_HIDDEN ** -0.5)
        return m.to(dev).eval()

    def time_loop(fn):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    g = torch.Generator().manual_seed(100)
    if args.workload == "muon":
        # Muon's Newton-Schulz on the block's stacked weight gradients (the next consumer of dW_in
        # / dW_out, src/train/optim.py:27-40): 78 x [576, 256] and 78 x [128, 576], 5 iterations
        # each, replayed from a CUDA graph; next to it the same iteration as torch batched matmuls.
        from nanospeaker_b200.muon import _ns_torch, newton_schulz5
        E = N_EXPERTS + N_SHARED
        grads = [(torch.randn(E, D_MODEL, 2 * D_HIDDEN, generator=g) * 0.02).bfloat16().to(dev),
                 (torch.randn(E, D_HIDDEN, D_MODEL, generator=g) * 0.02).bfloat16().to(dev)]

        def graphed(fn):
            for _ in range(2):
                [fn(t) for t in grads]
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                outs = [fn(t) for t in grads]
            return gr, outs
        l0 = K.LAUNCHES
        g_k, _ = graphed(lambda t: newton_schulz5(t))
        launches = (K.LAUNCHES - l0) // 3
        g_t, _ = graphed(lambda t: _ns_torch(t, 5, 1e-7))
        ms = time_loop(lambda i: g_k.replay())
        ms_torch = time_loop(lambda i: g_t.replay())
        K.check_status(dev)
        flop = 0
        for r_, c_ in ((2 * D_HIDDEN, D_MODEL), (D_HIDDEN, D_MODEL)):     # small side, large side
            flop += E * 5 * (2 * r_ * r_ * c_ * 2 + 2 * r_ ** 3)
        print(json.dumps({
            "metric": "Muon Newton-Schulz on the block's stacked expert gradients (5 iterations)",
            "value": ms, "unit": "ms", "higher_is_better": False, "n_gpus": 1, "steps": steps,
            "warmup": warmup, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{E} x [576, 256] and {E} x [128, 576] bf16 gradients, "
                                   "X <- aX + (bA + cAA)X five times each, CUDA graph replay"},
            "gpu_launches_per_step": launches, "tflops": flop / (ms * 1e-3) / 1e12,
            "torch_bmm_ms": ms_torch}), flush=True)
        return
    if args.workload == "sublayer":
        from nanospeaker_b200.sublayer import MoEFFNSublayer
        T = TOKENS
        sub = MoEFFNSublayer(make_block(7)).to(torch.bfloat16).to(dev).train()
        with torch.no_grad():
            sub.norm_gamma.copy_(1 + 0.1 * torch.randn(D_MODEL, generator=g))
        params = list(sub.parameters())
        one = torch.ones((), device=dev)

        def graph_of(fn):
            xs = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev).requires_grad_(True)
                  for _ in range(4)]
            gos = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev) for _ in range(4)]
            graphs = []
            for x, go in zip(xs, gos):
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(3):
                        for p in params:
                            p.grad = None
                        x.grad = None
                        out, aux = fn(x)
                        torch.autograd.backward([out, aux], [go, one])
                torch.cuda.current_stream().wait_stream(side)
                del out, aux
                sub.ffn.aux_loss = torch.zeros((), device=dev)
                for p in params:
                    p.grad = None
                x.grad = None
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    out, aux = fn(x)
                    torch.autograd.backward([out, aux], [go, one])
                graphs.append((gr, x, go, out))
            return graphs

        def unfused(x):
            h = torch.nn.functional.rms_norm(x, (D_MODEL,), sub.norm_gamma, sub.epsilon)
            return x + sub.ffn(h), sub.ffn.aux_loss

        fused_graphs = graph_of(lambda x: sub(x))
        ms = time_loop(lambda i: fused_graphs[i % 4][0].replay())
        unfused_graphs = graph_of(unfused)
        ms_unfused = time_loop(lambda i: unfused_graphs[i % 4][0].replay())
        line = {"metric": "FFN sublayer tokens/s (fwd+bwd)", "value": T / (ms / 1e3),
                "unit": "tokens/s", "higher_is_better": True, "ms_per_step": ms,
                "unfused_ms_per_step": ms_unfused,
                "config": {"workload": "x + ffn(rmsnorm(x)) forward + backward, T=16384, bf16: the "
                                       "fused autograd node against torch rms_norm + block + add"}}
    elif args.workload == "decode":
        layers, T = 20, 64
        stack = StackedMoEDecoder([make_block(1000 + i) for i in range(layers)])
        xs = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev) for _ in range(8)]
        stack.eager(xs[0])        # (the first step also pads every block's router weight, once)
        l0 = K.LAUNCHES
        stack.eager(xs[0])
        launches = K.LAUNCHES - l0
        eager_ms = time_loop(lambda i: stack.eager(xs[i % 8]))
        ms = time_loop(lambda i: stack.step(xs[i % 8]))
        # the same stack with the combine in the down GEMM's epilogue (one launch fewer per block;
        # bf16 atomics, so not bit-reproducible from run to run: not the decoder's default)
        stack_atomic = StackedMoEDecoder(stack.blocks, combine="atomic")
        ms_atomic = time_loop(lambda i: stack_atomic.step(xs[i % 8]))
        line = {"metric": "MoE decode stack latency (20 blocks, forward)", "value": ms,
                "unit": "ms", "higher_is_better": False, "tokens_per_s": T / (ms / 1e3),
                "eager_ms": eager_ms, "gpu_launches_per_step": launches,
                "atomic_combine_ms": ms_atomic,
                "config": {"workload": "BASELINE config 3: 20 stacked MoE blocks (independent "
                                       "weights), T=64 tokens, bf16, forward, one CUDA graph"}}
    else:
        T = 131072
        m = make_block(7)
        xs = [torch.randn(T, D_MODEL, generator=g).bfloat16().to(dev) for _ in range(4)]
        with torch.no_grad():
            l0 = K.LAUNCHES
            m(xs[0])
            launches = K.LAUNCHES - l0
            ms = time_loop(lambda i: m(xs[i % 4]))
        line = {"metric": "MoE-block tokens/s (forward, prefill)", "value": T / (ms / 1e3),
                "unit": "tokens/s", "higher_is_better": True, "ms_per_step": ms,
                "gpu_launches_per_step": launches,
                "config": {"workload": "BASELINE config 4 (one GPU's view): one MoE block forward, "
                                       "T=131072 tokens, bf16, eager launches"}}
    K.check_status(dev)
    line.update({"n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16",
                 "data": "synthetic"})
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--grad-allreduce-impl", default="auto", choices=["auto", "nccl", "peer"],
                    help="N > 1: how the weight gradients are summed over the ranks: device-to-"
                         "device copies through peer memory (parallel.PeerGradAllReduce; NCCL if "
                         "symmetric memory cannot be set up), or an NCCL all-reduce. auto: peer "
                         "up to 4 ranks, NCCL beyond (measured: at 8 ranks NCCL's in-switch "
                         "reduction takes 0.17 ms alone, the 14 copies per rank 0.44 ms)")
    ap.add_argument("--no-grad-allreduce", action="store_true",
                    help="N > 1: time the bare token-sharded replicas, without the gradient all-reduce")
    ap.add_argument("--grad-allreduce", action="store_true",
                    help="(default at N > 1; kept so that older command lines still parse)")
    ap.add_argument("--no-stages", action="store_true", help="skip the per-kernel roofline pass")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager module calls instead of a captured CUDA graph of the step")
    ap.add_argument("--profile-stage", default="",
                    help="run only the stage whose name contains this text, 3 launches (for ncu)")
    ap.add_argument("--ep-tokens", type=int, default=16384,
                    help="ep-loopback workload: tokens per virtual rank")
    ap.add_argument("--workload", default="train",
                    choices=["train", "decode", "prefill", "sublayer", "muon", "ep", "ep-loopback"],
                    help="train = the headline (forward + backward, T=16384); decode / prefill = "
                         "the forward-only workloads of the block's other callers; sublayer = "
                         "x + ffn(rmsnorm(x)) forward + backward at T=16384, fused node against "
                         "norm, block and add as separate steps")
    ap.add_argument("--skew", default="cv1", choices=sorted(SKEWS),
                    help="train workload: spread of the per-expert routing bias (see SKEWS)")
    ap.add_argument("--ep-impl", default="push", choices=["push", "nccl"],
                    help="ep workload: rows moved by the push / pull kernels over peer memory, or "
                         "by NCCL all-to-all around the single-GPU kernels")
    ap.add_argument("--routing", default="uniform", choices=["uniform", "hotspot"],
                    help="ep workload: no routing bias, or a bias on experts 0-3 that sends half "
                         "of all assignments to them (all four live on rank 0)")
    args = ap.parse_args()
    global SKEW_NAME, BIAS_STD
    SKEW_NAME, BIAS_STD = args.skew, SKEWS[args.skew]
    if args.workload == "ep-loopback":
        run_ep_loopback(args)
    elif args.workload == "ep":
        run_ep_workload(args)
    elif args.workload != "train":
        run_side_workload(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
