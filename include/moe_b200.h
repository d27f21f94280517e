/*
 * moe_b200.h -- C ABI of the B200 (sm_100a) dropless MoE block kernels.
 *
 * The library is a drop-in for the GPU half of nanoSpeaker's MoE block: each entry point below
 * replaces one stage that the reference runs as Triton kernels (src/model/moe_kernel.py) or as
 * plain PyTorch (src/model/router.py, src/model/moe.py), and is what a host binding (ctypes,
 * pybind, a torch.library op) calls.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless marked "host".
 *   - Activations, weights and per-pair rows are bf16, row-major, 16-byte aligned.
 *   - Index tensors are int32 except topk_idx, which is int64 (what torch.topk returns).
 *   - Nothing here allocates, frees or synchronises; work is queued on `stream`
 *     (a cudaStream_t passed as void*).
 *   - Return value: MOE_B200_OK or a negative MOE_B200_ERR_* (see moe_b200_error_string).
 *   - `status` is a device int32 word the kernels set non-zero when they notice a problem while
 *     running (a bounded wait that ran out = 1, an expert id out of range = 2). The host reads it
 *     whenever it wants to pay for the synchronisation.
 *   - "slot order": pairs (token, expert) sorted by expert, every expert's run padded to a
 *     multiple of 128 rows; pad slots hold the sentinel n_pairs in sorted_ids and zero rows in
 *     every slot-ordered activation buffer. l_cap = moe_b200_l_cap(n_pairs, n_experts) rows.
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_B200_OK 0
#define MOE_B200_ERR_SHAPE (-1)       /* a size is negative, zero where it may not be, or inconsistent */
#define MOE_B200_ERR_NULL (-2)        /* a required pointer is NULL */
#define MOE_B200_ERR_ALIGN (-3)       /* a pointer or row stride is not aligned (16 bytes for inputs, 32 for GEMM operands and outputs) */
#define MOE_B200_ERR_SCRATCH (-4)     /* scratch buffer missing or too small */
#define MOE_B200_ERR_UNSUPPORTED (-5) /* shape / activation the kernels do not cover */
#define MOE_B200_ERR_TMA (-6)         /* the driver refused a tensor map */
#define MOE_B200_ERR_CUDA (-7)        /* a launch failed; see cudaGetLastError */
#define MOE_B200_ERR_TOO_LARGE (-8)   /* problem exceeds the fixed scratch of a *_static entry point */

/* Activation ids; same numbering as KERNEL_ACTIVATIONS in src/model/moe_kernel.py:75. */
#define MOE_B200_ACT_SILU 0
#define MOE_B200_ACT_GELU 1
#define MOE_B200_ACT_RELU 2
#define MOE_B200_ACT_SIGMOID 3
#define MOE_B200_ACT_TANH 4

/* ABI version of this header. */
int32_t moe_b200_abi_version(void);

/* Text for a MOE_B200_ERR_* code (host pointer, static storage). */
const char* moe_b200_error_string(int32_t code);

/* Worst-case padded pair count, a multiple of 128.
 * Replaces _l_cap (src/model/moe_kernel.py:100-108). */
int64_t moe_b200_l_cap(int64_t n_pairs, int32_t n_experts);

/* Bytes of scratch moe_b200_dispatch needs (per-block expert histograms). */
size_t moe_b200_dispatch_scratch_bytes(int64_t n_pairs, int32_t n_experts);

/* Router top-k on fp32 logits [n_tokens, n_experts] (n_experts <= 256, top_k <= 16).
 * Replaces the softmax / topk / renormalise half of TopKRouter.forward
 * (src/model/router.py:79-97). Selection is by descending logit, ties to the lowest expert index,
 * output sorted the same way. full_softmax != 0 is the training spelling (weights from the softmax
 * over all experts, renormalised over the winners when normalize != 0 and top_k > 1; probs
 * [n_tokens, n_experts] written when non-NULL); full_softmax == 0 is the eval spelling (softmax
 * over the winning logits when normalize != 0, else the full-softmax probabilities).
 * topk_w [n_tokens, top_k] fp32, topk_idx [n_tokens, top_k] int64. */
int moe_b200_router_topk(const float* logits, int64_t n_tokens, int32_t n_experts, int32_t top_k,
                         int32_t normalize, int32_t full_softmax, float* topk_w, int64_t* topk_idx,
                         float* probs, void* stream);

/* d(logits) [n_tokens, n_experts] fp32 from d(topk_w) [n_tokens, top_k] fp32 and, optionally,
 * d(probs) [n_tokens, n_experts] fp32 (the balance-loss path). Replaces what autograd derives for
 * src/model/router.py:79-97. */
int moe_b200_router_topk_bwd(const float* logits, const int64_t* topk_idx, const float* d_topk_w,
                             const float* d_probs, int64_t n_tokens, int32_t n_experts,
                             int32_t top_k, int32_t normalize, int32_t full_softmax,
                             float* d_logits, void* stream);

/* Fused router step of the whole-block path: the selection / softmax arithmetic of
 * moe_b200_router_topk, reading the bf16 logits [n_tokens, ld] the router GEMM wrote (plus an
 * optional fp32 per-expert bias), writing w_all / idx_all [n_tokens, top_k + n_shared] (bf16 /
 * int64) whose last n_shared columns are the shared experts as (expert n_experts + s, weight 1)
 * pairs, and -- when full_softmax != 0 and colsum != NULL -- ADDING sum_t softmax(l_t)[e] into
 * colsum[e] (fp32 [n_experts], zero it first), the only statistic balance_loss needs
 * (src/model/router.py:100-111). No [T, E] fp32 tensor is written.
 * noise (may be NULL): fp32 [n_tokens, n_experts], added to the logits like the bias -- the
 * exploration noise of a training step (src/model/router.py:76-77), drawn by the caller so that the
 * random stream stays outside the kernels. */
int moe_b200_router_fused(const void* logits, int32_t ld, const float* bias, const float* noise,
                          int64_t n_tokens,
                          int32_t n_experts, int32_t top_k, int32_t n_shared, int32_t normalize,
                          int32_t full_softmax, void* w_all, int64_t* idx_all, float* colsum,
                          void* stream);

/* Backward of moe_b200_router_fused: d(logits) as bf16 [n_tokens, ld_out] (columns >= n_experts
 * zero) from d(w_all) (bf16; the shared columns are ignored) and, when d_aux != NULL, the
 * balance loss's gradient d_aux[0] * aux_coef * n_experts / n_tokens * counts[e] / sum(counts)
 * on every probability of expert e (counts int32 [n_experts] from the dispatch). */
int moe_b200_router_fused_bwd(const void* logits, int32_t ld, const float* bias,
                              const float* noise, const int64_t* idx_all, const void* dw_all, int64_t n_tokens,
                              int32_t n_experts, int32_t top_k, int32_t n_shared,
                              int32_t normalize, int32_t full_softmax, const float* d_aux,
                              const int32_t* counts, float aux_coef, void* d_logits,
                              int32_t ld_out, void* stream);

/* aux[0] = aux_coef * n_experts * sum_e (counts[e] / sum counts) * (colsum[e] / n_tokens):
 * TopKRouter.balance_loss (src/model/router.py:100-111) from the column sums. */
int moe_b200_balance_loss(const float* colsum, const int32_t* counts, int32_t n_experts,
                          int64_t n_tokens, float aux_coef, float* aux, void* stream);

/* Dispatch plan from topk_idx (flat [n_pairs] int64): replaces moe_dispatch and its four kernels
 * (src/model/moe_kernel.py:113-209) and MoEBlock._plan (src/model/moe.py:208-223).
 *   sorted_ids  [l_cap]      slot -> pair id, sentinel n_pairs in pad slots
 *   expert_ids  [l_cap/128]  owner of each 128-row block (0 past the live range)
 *   pad_offsets [E+1]        128-aligned run starts
 *   counts      [E]          routing histogram
 *   n_post_pad  [1]          live padded length
 *   inv_ids     [n_pairs]    pair id -> slot
 * Unlike the reference's atomic scatter the order inside a run is STABLE (ascending pair id), so
 * sorted_ids with the sentinels removed equals a stable sort of the expert ids.
 * capacity = 0: dropless. capacity > 0 is the fixed-capacity schedule of the reference's padded
 * path (MoEBlock._slots / _forward_padded, src/model/moe.py:225-283) on the same kernels: every
 * expert below n_capped (the routed ones; shared experts dispatched as extra experts behind them
 * are never limited) keeps the first `capacity` pairs of its run and drops the rest; a dropped pair gets no
 * slot (inv_ids = -1, which moe_b200_combine reads as a zero row), the runs and n_post_pad are laid
 * out by the kept counts, and counts still reports the routing decisions before the drop. A pair
 * whose expert id is out of range also gets inv_ids = -1 (and sets the status word). */
int moe_b200_dispatch(const int64_t* topk_idx, int64_t n_pairs, int32_t n_experts,
                      int32_t* sorted_ids, int32_t* expert_ids, int32_t* pad_offsets,
                      int32_t* counts, int32_t* n_post_pad, int32_t* inv_ids, void* scratch,
                      size_t scratch_bytes, int32_t capacity, int32_t n_capped, int32_t* status,
                      void* stream);

/* Router top-k and dispatch in two launches for the whole-block path: the router kernel
 * (moe_b200_router_fused's arithmetic and outputs) runs with one block per chunk of 128+ tokens and
 * leaves that chunk's histogram of expert ids, so the dispatch's histogram pass is not needed; the
 * plan + scatter kernel follows over idx_all [n_tokens, top_k + n_shared] with n_experts + n_shared
 * experts (outputs as moe_b200_dispatch; l_cap = moe_b200_l_cap(n_tokens * (top_k + n_shared),
 * n_experts + n_shared)). scratch: moe_b200_router_dispatch_scratch_bytes(n_tokens,
 * n_experts + n_shared) bytes. Replaces TopKRouter.forward's selection (src/model/router.py:79-97)
 * followed by moe_dispatch (src/model/moe_kernel.py:180-218). 
 * A batch of at most 128 tokens (one block) is routed, planned and scattered by a single launch. */
size_t moe_b200_router_dispatch_scratch_bytes(int64_t n_tokens, int32_t n_experts_total);
int moe_b200_router_dispatch(const void* logits, int32_t ld, const float* bias,
                             const float* noise, int64_t n_tokens,
                             int32_t n_experts, int32_t top_k, int32_t n_shared,
                             int32_t normalize, int32_t full_softmax, void* w_all,
                             int64_t* idx_all, float* colsum, int32_t* sorted_ids,
                             int32_t* expert_ids, int32_t* pad_offsets, int32_t* counts,
                             int32_t* n_post_pad, int32_t* inv_ids, void* scratch,
                             size_t scratch_bytes, int32_t* status, void* stream);

/* moe_b200_dispatch for callers that cannot supply scratch memory. (No counterpart in the
 * reference: its dispatch allocates through torch.) Meant for hosts that may not allocate device
 * memory at call time -- a process whose memory plan was frozen at start-up, or a foreign-function
 * caller that owns its input/output buffers but has no device allocator. The per-block histograms
 * live in a 128 KB __device__ array inside the library instead of a caller buffer, so:
 *   - the array holds 128 blocks x 256 experts, which is the most the dispatch ever uses (past
 *     128 blocks it doubles the pairs per block instead), so the limit on n_pairs is the dispatch's
 *     own 2^30 = moe_b200_dispatch_static_max_pairs(n_experts); beyond it the call returns
 *     MOE_B200_ERR_TOO_LARGE;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current); make that first call outside any stream capture;
 *   - all calls on a device share the one array: two calls that may overlap on the GPU (different
 *     streams, no dependency) race and give wrong plans. Calls ordered on one stream are safe, and
 *     nothing needs clearing between them because every entry that is read is rewritten first.
 * It allocates nothing and frees nothing. Outputs are exactly those of moe_b200_dispatch. */
int64_t moe_b200_dispatch_static_max_pairs(int32_t n_experts);
int moe_b200_dispatch_static(const int64_t* topk_idx, int64_t n_pairs, int32_t n_experts,
                             int32_t* sorted_ids, int32_t* expert_ids, int32_t* pad_offsets,
                             int32_t* counts, int32_t* n_post_pad, int32_t* inv_ids,
                             int32_t* status, void* stream);

/* Token permute: xs[slot, :] = x[sorted_ids[slot] / top_k, :], zero rows in pad slots, for slots
 * below n_post_pad. Replaces x.index_select(0, token_idx) (src/model/moe.py:397) and the gather
 * loads inside _gemm1_kernel (src/model/moe_kernel.py:295-305). x [n_tokens, d_model],
 * xs [l_cap, d_model]. n_post_pad points at any device int32 that holds the number of slot rows to
 * fill (a multiple of 8): the dispatch's n_post_pad for all of them, or pad_offsets + E to stop at
 * the first shared expert's run when the GEMMs read those runs from x in place (a_tokens of
 * moe_b200_up_gemm). */
int moe_b200_permute(const void* x, int64_t n_tokens, int32_t d_model, int32_t top_k,
                     const int32_t* sorted_ids, const int32_t* n_post_pad, int64_t l_cap, void* xs,
                     void* stream);

/* Token-major combine: out[t, :] = sum_j y[inv_ids[t*top_k + j], :] (+ extra[t, :] + extra2[t, :])
 * accumulated in fp32; a negative inv_ids entry (a pair the dispatch dropped) counts as a zero row.
 * Replaces _reduce_kernel (src/model/moe_kernel.py:415-437) and
 * out.index_add_ (src/model/moe.py:413); extra / extra2 (nullable, [n_tokens, d_model]) carry the
 * shared experts' rows (src/model/moe.py:416-417). */
int moe_b200_combine(const void* y, const int32_t* inv_ids, int64_t n_tokens, int32_t top_k,
                     int32_t d_model, const void* extra, const void* extra2, void* out,
                     void* stream);

/* Per-expert column sums of a slot-ordered buffer: out[e, :] += sum over the rows of run e of
 * row_w * buf[row, :] (fp32 [n_groups, width]; the caller zeroes it first; one atomic add per
 * 128-row tile and column). row_w = pair_w[sorted_ids[row]] when pair_w is given (pad rows weigh 0),
 * else 1. alt / first_alt_group: the runs from first_alt_group on read row `slot - pad_offsets[run]`
 * of the token-major matrix alt [alt_rows, width] instead (rows past alt_rows count as zero), as
 * the GEMMs do for the shared experts. These are the bias gradients of the block:
 * db_in = column sums of dA1, db_out = column sums of w * dOut -- the segment sums the reference
 * takes with index_add_ (src/model/moe_kernel.py:723-737). width % 8 == 0. */
int moe_b200_segment_colsum(const void* buf, int64_t rows, int32_t width,
                            const int32_t* expert_ids, const int32_t* n_post_pad,
                            const int32_t* pad_offsets, int32_t n_groups,
                            const int32_t* sorted_ids, const void* pair_w, int64_t n_pairs,
                            const void* alt, int64_t alt_rows, int32_t first_alt_group,
                            float* out, void* stream);

/* Two element-wise helpers of the batched Newton-Schulz iteration that Muon runs on the stacked
 * expert weights (zeropower_via_newtonschulz5, src/train/optim.py:27-40); its matrix products run on
 * the grouped GEMM entry points above with the fixed schedule.
 *   moe_b200_group_sumsq: sumsq[g] += sum of squares of x[g, :] (x [groups, per_group] bf16, per_group
 *     a multiple of 8; sumsq fp32 [groups], zeroed by the caller) -- the Frobenius norms of
 *     `X / (X.norm(dim=(-2, -1)) + eps)`.
 *   moe_b200_axpby: out = alpha * s_g * x + beta * y in fp32, rounded once to bf16, with
 *     s_g = 1 / (sqrt(sumsq[g]) + eps) when sumsq is given and 1 otherwise; y may be NULL. Covers the
 *     normalisation, `b * A + c * (A @ A)` and `a * X + (...) @ X`. */
int moe_b200_group_sumsq(const void* x, int32_t groups, int64_t per_group, float* sumsq,
                         void* stream);
int moe_b200_axpby(const void* x, const void* y, void* out, int32_t groups, int64_t per_group,
                   float alpha, float beta, const float* sumsq, float eps, void* stream);

/* dst[r, c] = c < cols ? src[r, c] : 0 for 0 <= c < dst_ld; 16-bit elements, row strides src_ld /
 * dst_ld elements. Pads the router weight [d_model, n_experts] (src/model/router.py:51) to the
 * 64-column multiple the GEMM kernels' tensor maps need, and strips the pad columns from its
 * gradient. No reference counterpart (the reference's router is a plain matmul). */
int moe_b200_copy_cols(const void* src, int64_t rows, int32_t cols, int32_t src_ld, void* dst,
                       int32_t dst_ld, void* stream);

/* RMSNorm in front of the block: h[t] = x[t] * rstd[t] * gamma, rstd[t] = rsqrt(mean(x[t]^2) + eps)
 * (x, gamma, h bf16; rstd fp32 [n_rows], kept for the backward). d_model % 8 == 0, <= 2048.
 * Replaces RMSNorm.forward (src/model/ln.py:31-38) as used by Block.forward's
 * `x + self.ffn(self.norm_ffn(x))` (src/model/nanospeaker.py:165-169). */
int moe_b200_rmsnorm(const void* x, const void* gamma, int64_t n_rows, int32_t d_model, float eps,
                     void* h, float* rstd, void* stream);

/* Its backward, with the residual branch's gradient folded in:
 *   dx[t] = rstd * (gamma * dh[t]) - x[t] * rstd^3 / d_model * <gamma * dh[t], x[t]>  (+ add[t])
 *   dgamma += sum_t dh[t] * x[t] * rstd[t]        (fp32 [d_model], accumulated: zero it first)
 * add may be NULL. Replaces autograd through F.rms_norm (src/model/ln.py:33) and the residual's
 * gradient add. */
int moe_b200_rmsnorm_bwd(const void* dh, const void* x, const float* rstd, const void* gamma,
                         const void* add, int64_t n_rows, int32_t d_model, void* dx,
                         float* dgamma, void* stream);

/* Schedule arguments shared by the row-grouped GEMMs below:
 *   rows            rows of the slot-ordered A buffer (l_cap), or the token count when
 *                   n_fixed_groups > 0
 *   expert_ids, n_post_pad   from moe_b200_dispatch
 *   n_fixed_groups  0: routed schedule, per-block owners from expert_ids.
 *                   S > 0: shared-expert schedule -- weight matrices 0..S-1 are each applied to all
 *                   `rows` rows in token order (`rows` need not be a multiple of 128); outputs are
 *                   stacked [S, rows, width].
 *   w_extra, n_extra  optional second weight stack (routed schedule only): expert ids in
 *                   [n_groups, n_groups + n_extra) index it. This is how the shared experts ride in
 *                   the same launches as the routed ones: the dispatch sees them as n_extra more
 *                   experts that every token is routed to, and their weights stay in their own
 *                   tensors (W_sh_in / W_sh_out, src/model/moe.py:160-168). */

/* Gathered A operand (routed schedule only): with gather_top_k > 0 the A argument is the
 * token-major matrix [n_pairs / gather_top_k, width] and the kernel itself reads row
 * sorted_ids[slot] / gather_top_k for slot `slot` (zero rows in pad slots), so no permuted copy has
 * to exist -- the gather loads of _gemm1_kernel (src/model/moe_kernel.py:295-305). With
 * gather_top_k == 0 A is a slot-ordered [rows, width] buffer (e.g. from moe_b200_permute). */

/* Up/gate GEMM with the GLU fused: [g | u] = a[row] @ w_in[e] (w_in [n_groups, d_model,
 * 2*d_hidden]); hid[row] = act(g) * u  ([rows, d_hidden]); when raw != NULL it also receives
 * [g | u] ([rows, 2*d_hidden], kept for the backward). a is [rows, d_model] (shared by all fixed
 * groups) or gathered. Replaces _gemm1_kernel (src/model/moe_kernel.py:269-323).
 * d_hidden must be 128.
 * a_tokens (may be NULL; routed schedule with a second weight stack, no gather): the token-major
 * matrix [n_tokens, d_model] the slot-ordered rows were copied from. The groups of the second stack
 * (shared experts: every token once, in token order) then read row `slot - pad_offsets[group]` of
 * a_tokens instead of row `slot` of a, so their rows of a need not have been written at all (see
 * moe_b200_permute: pass pad_offsets + n_groups as its live-row count). Rows past n_tokens read as
 * zeros.
 * bias (may be NULL; routed schedule): [n_groups + n_extra, 2*d_hidden] in the activation dtype --
 * b_in followed by the second stack's b_sh_in (src/model/moe.py:155-156, 166-167) -- added to
 * [g | u] before the GLU (src/model/moe_kernel.py:311-313); raw then holds the biased values. */
int moe_b200_up_gemm(const void* a, int64_t rows, int32_t d_model, const void* w_in,
                     int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_hidden, const int32_t* expert_ids,
                     const int32_t* n_post_pad, int32_t n_fixed_groups,
                     const int32_t* sorted_ids, int32_t gather_top_k, int64_t n_pairs,
                     int32_t activation, void* hid, void* raw, const void* a_tokens,
                     int64_t n_tokens, const int32_t* pad_offsets, const void* bias,
                     int32_t* status, void* stream);

/* Down GEMM with the router weight fused: y[row] = (hid[row] @ w_out[e]) * pair_w[sorted_ids[row]]
 * (w_out [n_groups, k_dim, d_model]; weight 1 when pair_w is NULL). With fixed groups hid is
 * [S, rows, k_dim]. Replaces the forward use of _gemm2_kernel
 * (src/model/moe_kernel.py:339-402, 603-613). 
 * bias (may be NULL; routed schedule): [n_groups + n_extra, d_model], b_out followed by the second
 * stack's b_sh_out, added before the weight scale (src/model/moe_kernel.py:395-399). */
int moe_b200_down_gemm(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                       int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model, const int32_t* expert_ids,
                       const int32_t* n_post_pad, int32_t n_fixed_groups,
                       const int32_t* sorted_ids, const void* pair_w, int64_t n_pairs, void* y,
                       const void* bias, int32_t* status, void* stream);

/* The down GEMM fused with the combine: instead of storing per-pair rows, every live row is ADDED to
 * row sorted_ids[row] / top_k of the token-major matrix acc [n_tokens, d_model] (bf16; the caller
 * fills it first: zeros, or a residual / other summand). One asynchronous bulk reduction per row
 * and 192-column tile; the adds are bf16 atomics performed in L2, so the k rows of a token are
 * summed in bf16 in whatever order they arrive (what out.index_add_ does in the reference's eager
 * path, src/model/moe.py:407-413, there in expert order) and no y [l_cap, d_model] is written or
 * read back. The store-then-reduce pair moe_b200_down_gemm + moe_b200_combine (fp32 sum in pair
 * order, bitwise reproducible) is the reference's choice (src/model/moe_kernel.py:26-30, 362-365,
 * 579-582); this is the atomic variant it weighs it against. Fixed schedule: row r of every group
 * is added to row r of acc (rows <= n_tokens). Other arguments as moe_b200_down_gemm. */
int moe_b200_down_gemm_acc(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                           int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model,
                           const int32_t* expert_ids, const int32_t* n_post_pad,
                           int32_t n_fixed_groups, const int32_t* sorted_ids, const void* pair_w,
                           int64_t n_pairs, int32_t top_k, void* acc, int64_t n_tokens,
                           const void* bias, int32_t* status, void* stream);

/* Backward through the down GEMM and the GLU in one kernel: G = douts[row] @ w_out[e]^T, then with
 * [g | u] = a1[row] and w = pair_w[pair]:  dtw[pair] = <G, act(g)*u>,
 * da1[row] = [w*G*u*act'(g) | w*G*act(g)],  hidw[row] = w * act(g) * u.
 * douts is [rows, d_model] (shared by all fixed groups) or, with gather_top_k > 0, the token-major
 * dOut gathered through sorted_ids; a1, da1, hidw are stacked per fixed group.
 * Replaces the dH use of _gemm2_kernel plus _glu_bwd_kernel
 * (src/model/moe_kernel.py:676-692, 510-553). dtw may be NULL.
 * dout_tokens / n_tokens / pad_offsets: as a_tokens of moe_b200_up_gemm, for the rows of douts. */
int moe_b200_dhidden_glu_bwd(const void* douts, int64_t rows, int32_t d_model, const void* w_out,
                             int32_t n_groups, const void* w_extra, int32_t n_extra,
                             int32_t d_hidden, const int32_t* expert_ids,
                             const int32_t* n_post_pad, int32_t n_fixed_groups,
                             const int32_t* sorted_ids, int32_t gather_top_k, const void* pair_w,
                             int64_t n_pairs, const void* a1, int32_t activation, void* da1,
                             void* hidw, void* dtw, const void* dout_tokens, int64_t n_tokens,
                             const int32_t* pad_offsets, int32_t* status, void* stream);

/* dX GEMM: ydx[row] = da1[row] @ w_in[e]^T, reading w_in [n_groups, d_model, 2*d_hidden] in place
 * (no transposed copy). With fixed groups da1 and ydx are stacked [S, rows, .]. Replaces the dX use
 * of _gemm2_kernel and the w_in.transpose copy (src/model/moe_kernel.py:696-707). */
int moe_b200_dx_gemm(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                     int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model, const int32_t* expert_ids,
                     const int32_t* n_post_pad, int32_t n_fixed_groups, void* ydx,
                     int32_t* status, void* stream);

/* The dX GEMM fused with the combine: row `row` of da1 @ w_in[e]^T is added to row
 * sorted_ids[row] / top_k of acc [n_tokens, d_model] (bf16, filled by the caller), as
 * moe_b200_down_gemm_acc does for the forward. Replaces the dX use of _gemm2_kernel together with
 * the _reduce_kernel pass behind it (src/model/moe_kernel.py:696-710). pad_offsets (may be NULL;
 * routed schedule): the dispatch's run starts [n_groups + n_extra + 1]; with them the kernel runs
 * on CTA pairs that share each weight tile (half the weight traffic per SM), without them on
 * single CTAs. */
int moe_b200_dx_gemm_acc(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                         int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model,
                         const int32_t* expert_ids, const int32_t* n_post_pad,
                         int32_t n_fixed_groups, const int32_t* sorted_ids, int64_t n_pairs,
                         int32_t top_k, void* acc, int64_t n_tokens, const int32_t* pad_offsets,
                         int32_t* status, void* stream);

/* Group-summed row GEMMs with plain stores: out[t] = sum over g < n_sum of
 *   hid[run_offsets[g] + t] @ w_out[g]            (moe_b200_down_gemm_sum, k_dim = d_hidden)
 *   da1[run_offsets[g] + t] @ w_in[g]^T           (moe_b200_dx_gemm_sum)
 * for t < n_tokens. run_offsets [n_sum] int32 on the device: where each group's token-ordered run
 * starts in the slot-ordered buffer of `rows` rows (for the shared experts: pad_offsets + n_experts).
 * They write the shared experts' share of the block's output (router weight 1) and of dX straight
 * into the token-major accumulators, which then need no zero fill, and leave only the routed
 * experts' rows to the atomic adds of moe_b200_down_gemm_acc / moe_b200_dx_gemm_acc (called with
 * n_post_pad = the start of the first shared run, n_extra = 0). The shared branch of the reference
 * is src/model/moe.py:310-329, added at :414-416. */
int moe_b200_down_gemm_sum(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                           int32_t n_sum, int32_t d_model, const int32_t* run_offsets,
                           int64_t n_tokens, void* out, int32_t* status, void* stream);
int moe_b200_dx_gemm_sum(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                         int32_t n_sum, int32_t d_model, const int32_t* run_offsets,
                         int64_t n_tokens, void* out, int32_t* status, void* stream);

/* Bytes of fp32 scratch moe_b200_wgrad needs for its partial tiles (contents arbitrary).
 * routed != 0: the pad_offsets schedule over `rows` = l_cap rows. ks_rows as for moe_b200_wgrad. */
int moe_b200_wgrad_scratch_bytes(int32_t m_dim, int32_t n_dim, int64_t rows, int32_t n_groups,
                                 int32_t routed, int32_t ks_rows, size_t* partial_bytes);

/* Per-expert weight gradient dw[e] = a_e^T @ b_e over the rows of run e
 * (a [rows, m_dim], b [rows, n_dim], dw [n_groups, m_dim, n_dim]); empty runs give zeros.
 * Routed schedule: pad_offsets [n_groups+1] from the dispatch. Fixed schedule: pad_offsets NULL,
 * every group spans rows [0, rows); a_grouped / b_grouped say whether that operand is stacked
 * [n_groups, rows, .] or shared by all groups. The contraction is split into chunks of ks_rows rows
 * (a multiple of 64; 0 = let the library choose) so long runs spread over many SMs; a run's partial
 * tiles are added in chunk order by a second small kernel, so the result is deterministic.
 * gather_which = 1 (a) or 2 (b), routed schedule only: that operand is the token-major matrix
 * [n_pairs / gather_top_k, width] and its rows are gathered through sorted_ids inside the kernel
 * (0 = both operands are slot-ordered buffers).
 * dw holds groups [0, n_first); with n_first < n_groups the remaining groups are written to
 * dw_extra [n_groups - n_first, m_dim, n_dim] (the shared experts' gradients).
 * alt (may be NULL; routed schedule, no gather, n_first < n_groups): token-major matrix
 * [alt_rows, m_dim] (alt_which = 1) or [alt_rows, n_dim] (alt_which = 2). The runs from n_first on
 * read that operand's row `slot - pad_offsets[run]` from alt instead of row `slot` of a / b.
 * Replaces _dw_kernel (src/model/moe_kernel.py:453-507, 712-721), which has no split-K. */
int moe_b200_wgrad(const void* a, int32_t a_grouped, int32_t m_dim, const void* b,
                   int32_t b_grouped, int32_t n_dim, int64_t rows, const int32_t* pad_offsets,
                   int32_t n_groups, int32_t ks_rows, const int32_t* sorted_ids,
                   int32_t gather_top_k, int64_t n_pairs, int32_t gather_which, void* dw,
                   int32_t n_first, void* dw_extra, void* partials, size_t partial_bytes,
                   const void* alt, int64_t alt_rows, int32_t alt_which, int32_t* status,
                   void* stream);

/* ---- Expert parallelism over peer memory (one node, up to 8 ranks) --------------------------------
 * The routed experts are partitioned contiguously over the ranks; rank r owns experts
 * [bounds[r], bounds[r+1]). The reference is single-GPU and has no counterpart for these entry
 * points; they are the multi-GPU form of its dispatch / gather / combine
 * (src/model/moe_kernel.py:113-218, 295-305, 415-437). No entry point waits on another GPU: the
 * caller separates the phases with a collective. Pointer tables are HOST arrays of device pointers
 * that are valid in the calling process (peer mappings of the other ranks' buffers, 16-byte
 * aligned); only plain loads and stores touch peer memory. */

/* From the all-gathered counts cnt_all [n_ranks, n_experts] (pairs per home rank and routed
 * expert): for this rank as a sender owner_of [E] and send_row0 [E] (row, in the owner's
 * slot-ordered buffer, of this rank's first pair of expert e; an owner's runs are 128-aligned and
 * hold the home ranks' pairs in rank order); as an owner own_offs [E_r+1], own_counts [E_r],
 * own_npp [1], own_eids [cap_tiles] -- the pad_offsets / counts / n_post_pad / expert_ids the
 * grouped GEMMs take. All arrays on the device; bounds [n_ranks+1] too. */
int moe_b200_ep_plan(const int32_t* cnt_all, const int32_t* bounds, int32_t n_ranks,
                     int32_t n_experts, int32_t rank, int32_t* owner_of, int32_t* send_row0,
                     int32_t* own_offs, int32_t* own_counts, int32_t* own_npp, int32_t* own_eids,
                     int64_t cap_tiles, void* stream);

/* Per pair p = t * k_all + j of the home rank: pair_rank[p], pair_row[p] = where its row lives
 * (owner and row in the owner's buffer). Pairs of the shared experts (idx_all >= n_experts) get
 * rank n_ranks (the local extra table entry) and row s * n_tokens + t. local_offs = the home
 * rank's own pad_offsets, inv_ids its inverse permutation (moe_b200_dispatch). */
int moe_b200_ep_pair_map(const int64_t* idx_all, const int32_t* inv_ids, const int32_t* local_offs,
                         const int32_t* owner_of, const int32_t* send_row0, int64_t n_tokens,
                         int32_t k_all, int32_t n_experts, int32_t n_ranks, int32_t* pair_rank,
                         int32_t* pair_row, void* stream);

/* The token permute fused with the dispatch exchange: row src[sorted_ids[s] / k_all] goes to row
 * pair_row[pair] of dst_rows[pair_rank[pair]], for the slots s < *n_live_slots of the home plan
 * (pass pad_offsets + n_experts: the shared experts' runs stay at home). With dst_sid / dst_w (may
 * be NULL) the destination row also gets its own index and the pair's weight w_all[pair].
 * first_slot (device int32, may be NULL = 0): the slot the walk starts at before it wraps around;
 * pass pad_offsets + bounds[(rank + 1) % n_ranks] so that the ranks write to different owners at
 * any one time instead of all to the same one. */
int moe_b200_ep_push_rows(const void* src, int64_t n_tokens, int32_t d_model, int32_t k_all,
                          const int32_t* sorted_ids, const int32_t* n_live_slots,
                          const int32_t* first_slot, int64_t max_slots, const int32_t* pair_rank,
                          const int32_t* pair_row, const void* const* dst_rows,
                          const void* const* dst_sid, const void* const* dst_w, int32_t n_ranks,
                          const void* w_all, void* stream);

/* Owner side: zero rows (and, with sid, the sentinel id) in the pad slots
 * [own_offs[e] + own_counts[e], own_offs[e+1]) of every local run. */
int moe_b200_ep_pad_fix(const int32_t* own_offs, const int32_t* own_counts, int32_t n_local,
                        void* rows, int32_t d_model, int32_t* sid, int32_t sentinel, void* stream);

/* The combine fused with the return exchange: out[t] = sum_j y[pair_rank[p]][pair_row[p]]
 * (+ extra[t]) in fp32, pair order as moe_b200_combine. y holds n_tables pointers (the ranks'
 * output buffers, then the local shared-expert buffer). */
int moe_b200_ep_pull_combine(const void* const* y, int32_t n_tables, const int32_t* pair_rank,
                             const int32_t* pair_row, int64_t n_tokens, int32_t k_all,
                             int32_t d_model, const void* extra, void* out, void* stream);

/* out[p] = v[pair_rank[p]][pair_row[p]] (bf16) for the routed columns j < top_k, 0 elsewhere. */
int moe_b200_ep_pull_vec(const void* const* v, int32_t n_ranks, const int32_t* pair_rank,
                         const int32_t* pair_row, int64_t n_tokens, int32_t k_all, int32_t top_k,
                         void* out, void* stream);

/* ---- The whole block in one host call per direction -------------------------------------------
 * moe_b200_block_fwd / moe_b200_block_bwd issue the complete stage sequence of a training step of
 * MoEBlock.forward (src/model/moe.py:345-418, router.py:56-111) and of its backward from C++: a
 * host that pays per call into this library (ctypes from Python: ~22 calls, ~1 ms per step at
 * T = 16384, more than the GPU needs) makes two. Training form: the permuted rows xs, the
 * pre-activations a1, the bf16 logits and the routing plan are kept for the backward; combine in
 * the GEMM epilogues (atomic); no residual, no per-expert biases (use the stage entry points for
 * those). Tensors: x [T, D], router_w [D, E], w_in [E, D, 2H], w_out [E, H, D], w_sh_* likewise
 * with n_shared groups (NULL when n_shared == 0), all bf16 and contiguous; logit_bias [E] and
 * noise [T, E] fp32 or NULL. With ld = E rounded up to 64, kS = top_k + n_shared, M = T * kS and
 * L = moe_b200_l_cap(M, E + n_shared) the caller provides out [T, D], aux (1 float), counts [E],
 * xs [L, D], a1 [L, 2H], logits [T, ld], w_all [T, kS] bf16, idx_all [T, kS] int64,
 * sorted_ids [L], expert_ids [L / 128], pad_offsets [E + n_shared + 1], counts_all [E + n_shared],
 * n_post_pad [1], inv_ids [M], router_w_padded [D, ld], and scratch of
 * moe_b200_block_fwd_scratch_bytes(...) bytes (contents arbitrary). n_launches (host, may be NULL)
 * receives the number of kernel launches made. */
size_t moe_b200_block_fwd_scratch_bytes(int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                                        int32_t n_experts, int32_t n_shared, int32_t top_k);
int moe_b200_block_fwd(const void* x, int64_t n_tokens, int32_t d_model, const void* router_w,
                       const float* logit_bias, const float* noise, const void* w_in,
                       const void* w_out, int32_t n_experts, int32_t d_hidden,
                       const void* w_sh_in, const void* w_sh_out, int32_t n_shared,
                       int32_t top_k, int32_t normalize, int32_t full_softmax, float aux_coef,
                       int32_t activation, void* out, float* aux, int32_t* counts, void* xs,
                       void* a1, void* logits, void* w_all, int64_t* idx_all,
                       int32_t* sorted_ids, int32_t* expert_ids, int32_t* pad_offsets,
                       int32_t* counts_all, int32_t* n_post_pad, int32_t* inv_ids,
                       void* router_w_padded, void* scratch, size_t scratch_bytes,
                       int32_t* n_launches, int32_t* status, void* stream);

/* The inference forward of the whole block in one call: out [T, D] = block(x) (+ residual [T, D]
 * when given), nothing kept. router_w_padded [D, ld] is the router weight zero-padded to ld = E
 * rounded up to 64 columns (moe_b200_copy_cols, built once per weight); the up/gate GEMM gathers
 * the token rows itself; atomic_combine != 0 adds the rows in the down GEMM's epilogue (bf16
 * atomics), 0 is the deterministic store-then-reduce combine. The caller of the decode loop
 * (src/model/nanospeaker.py:254-269) makes this one call per layer. */
size_t moe_b200_block_infer_scratch_bytes(int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                                          int32_t n_experts, int32_t n_shared, int32_t top_k);
int moe_b200_block_infer(const void* x, int64_t n_tokens, int32_t d_model,
                         const void* router_w_padded, const float* logit_bias, const void* w_in,
                         const void* w_out, int32_t n_experts, int32_t d_hidden,
                         const void* w_sh_in, const void* w_sh_out, int32_t n_shared,
                         int32_t top_k, int32_t normalize, int32_t activation,
                         const void* residual, int32_t atomic_combine, void* out, void* scratch,
                         size_t scratch_bytes, int32_t* n_launches, int32_t* status,
                         void* stream);

/* The backward of moe_b200_block_fwd: grad_out [T, D] bf16, grad_aux (1 float on the device, or
 * NULL), the forward's inputs and kept tensors -> dx [T, D], d_router [D, E], dw_in, dw_out,
 * dw_sh_in, dw_sh_out (shapes of the weights; the last two NULL when n_shared == 0). After the
 * dHidden kernel the work splits into three independent branches (dW_in + dX; dW_out; the
 * router's backward); side_stream_a / side_stream_b (cudaStream_t, may be NULL) take the second
 * and third, forked from and joined back into `stream` with events, so the call is capturable in
 * a CUDA graph and the caller only ever sees `stream`. scratch:
 * moe_b200_block_bwd_scratch_bytes(...) bytes. */
size_t moe_b200_block_bwd_scratch_bytes(int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                                        int32_t n_experts, int32_t n_shared, int32_t top_k);
int moe_b200_block_bwd(const void* grad_out, const float* grad_aux, const void* x,
                       int64_t n_tokens, int32_t d_model, const float* logit_bias,
                       const float* noise, const void* w_in, const void* w_out,
                       int32_t n_experts, int32_t d_hidden, const void* w_sh_in,
                       const void* w_sh_out, int32_t n_shared, int32_t top_k, int32_t normalize,
                       int32_t full_softmax, float aux_coef, int32_t activation, const void* xs,
                       const void* a1, const void* logits, const void* w_all,
                       const int64_t* idx_all, const int32_t* sorted_ids,
                       const int32_t* expert_ids, const int32_t* pad_offsets,
                       const int32_t* counts_all, const int32_t* n_post_pad,
                       const void* router_w_padded, void* dx, void* d_router, void* dw_in,
                       void* dw_out, void* dw_sh_in, void* dw_sh_out, void* scratch,
                       size_t scratch_bytes, void* side_stream_a, void* side_stream_b,
                       int32_t* n_launches, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H_ */
