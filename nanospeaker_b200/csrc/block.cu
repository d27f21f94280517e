// The whole block's forward and backward as ONE host call each: the stage sequence of
// nanospeaker_b200/moe_kernel.py (router GEMM, routing + dispatch, permute, up/gate GEMM + GLU,
// down GEMM with the atomic combine, balance loss; and the backward with its three independent
// branches on three streams) issued from C++, for hosts that pay per call into this library -- a
// Python caller's ~22 ctypes calls per step cost it more than the GPU needs for the work.
// Everything here is host code over the other entry points of include/moe_b200.h, plus four
// trivial kernels: zero / copy a few words (memset and device-to-device copy nodes go to a copy
// engine, where they queue behind a caller's large host-to-device copy in flight: the end-to-end
// step lost 13 us to that), and the forward's first and last launch, which fold what would
// otherwise be small launches of their own on the critical path (pad the router weight + clear
// the column sums; counts for the caller + balance loss). All of them wait for their
// predecessors programmatically like the library's other kernels, so none of them breaks the
// chain of early launches. Training form only: pre-activations and permuted rows are kept,
// combine mode "atomic", no residual, no per-expert biases.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"
#include "pdl.cuh"

namespace {

__global__ void zero_words_kernel(uint32_t* dst, int64_t n) {
  moe::pdl_trigger();
  moe::pdl_wait();
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n;
       i += int64_t(gridDim.x) * blockDim.x)
    dst[i] = 0u;
}
__global__ void copy_words_kernel(const uint32_t* src, uint32_t* dst, int64_t n) {
  moe::pdl_trigger();
  moe::pdl_wait();
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n;
       i += int64_t(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}
inline int zero_words(void* dst, int64_t n_words, cudaStream_t st) {
  const int64_t blocks = (n_words + 255) / 256;
  moe::launch_pdl(zero_words_kernel, dim3(unsigned(blocks < 592 ? blocks : 592)), dim3(256), 0, st,
                  static_cast<uint32_t*>(dst), n_words);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}
inline int copy_words(const void* src, void* dst, int64_t n_words, cudaStream_t st) {
  const int64_t blocks = (n_words + 255) / 256;
  moe::launch_pdl(copy_words_kernel, dim3(unsigned(blocks < 592 ? blocks : 592)), dim3(256), 0, st,
                  static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), n_words);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

// The forward's first launch: the router weight [D, E] zero-padded to [D, ld] (what
// moe_b200_copy_cols does) and, in the same launch, the column sums of the balance loss cleared.
__global__ void __launch_bounds__(256)
    pad_router_kernel(const uint16_t* __restrict__ src, int64_t rows, int32_t cols,
                      uint16_t* __restrict__ dst, int32_t dst_ld, float* __restrict__ colsum) {
  moe::pdl_trigger();
  moe::pdl_wait();
  const int64_t first = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (colsum != nullptr && first < cols) colsum[first] = 0.f;
  const int64_t total = rows * dst_ld;
  for (int64_t i = first; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = i / dst_ld;
    const int32_t c = int32_t(i - r * dst_ld);
    dst[i] = c < cols ? src[r * cols + c] : uint16_t(0);
  }
}
inline int pad_router(const void* src, int64_t rows, int32_t cols, void* dst, int32_t dst_ld,
                      float* colsum, cudaStream_t st) {
  int64_t blocks = (rows * dst_ld + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks * 256 < cols) return MOE_B200_ERR_SHAPE;   // (the clearing threads are the first `cols`)
  moe::launch_pdl(pad_router_kernel, dim3(unsigned(blocks)), dim3(256), 0, st,
                  static_cast<const uint16_t*>(src), rows, cols, static_cast<uint16_t*>(dst),
                  dst_ld, colsum);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

// The forward's last launch: the routed experts' counts for the caller and the balance loss
// aux = coef * E * sum_e (counts[e] / sum counts) * (colsum[e] / T) -- the arithmetic of
// moe_b200_balance_loss, same order -- or zero when the loss is off (colsum == nullptr). One warp.
// It does not release its dependents early: when a backward follows in the same graph, letting
// that backward's first kernel become resident under the down GEMM cost the step 2 us.
__global__ void finish_fwd_kernel(const int32_t* __restrict__ counts_all,
                                  int32_t* __restrict__ counts, const float* __restrict__ colsum,
                                  int n_experts, int64_t n_tokens, float coef,
                                  float* __restrict__ aux) {
  moe::pdl_wait();
  const int lane = threadIdx.x;
  float dot = 0.f, tot = 0.f;
  for (int e = lane; e < n_experts; e += 32) {
    const int32_t ci = counts_all[e];
    counts[e] = ci;
    if (colsum != nullptr) {
      const float c = float(ci);
      dot += c * colsum[e];
      tot += c;
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    dot += __shfl_xor_sync(0xffffffffu, dot, o);
    tot += __shfl_xor_sync(0xffffffffu, tot, o);
  }
  if (lane == 0)
    aux[0] = colsum == nullptr ? 0.f
                               : coef * float(n_experts) * dot / fmaxf(tot, 1.f) /
                                     float(n_tokens > 0 ? n_tokens : 1);
}
inline int finish_fwd(const int32_t* counts_all, int32_t* counts, const float* colsum,
                      int n_experts, int64_t n_tokens, float coef, float* aux, cudaStream_t st) {
  moe::launch_pdl(finish_fwd_kernel, dim3(1), dim3(32), 0, st, counts_all, counts, colsum,
                  n_experts, n_tokens, coef, aux);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

constexpr size_t ALIGN = 256;
inline size_t up(size_t n) { return (n + ALIGN - 1) / ALIGN * ALIGN; }
inline int32_t router_ld(int32_t n_experts) { return (n_experts + 63) / 64 * 64; }

struct Carver {   // hands out aligned pieces of one caller-provided buffer
  char* base;
  size_t used = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  void* take(size_t bytes) {
    void* r = base ? base + used : nullptr;
    used += up(bytes);
    return r;
  }
};

struct Sizes {
  int32_t ld, ks, n_all;
  int64_t m, l_cap;
};
inline Sizes sizes(int64_t n_tokens, int32_t n_experts, int32_t n_shared, int32_t top_k) {
  Sizes s;
  s.ld = router_ld(n_experts);
  s.ks = top_k + n_shared;
  s.n_all = n_experts + n_shared;
  s.m = n_tokens * s.ks;
  s.l_cap = moe_b200_l_cap(s.m, s.n_all);
  return s;
}

struct FwdScratch {
  void* hid;
  void* block_hist;
  size_t block_hist_bytes;
  float* colsum;
  size_t total;
};
FwdScratch carve_fwd(void* p, int64_t n_tokens, int32_t d_hidden, int32_t n_experts,
                     int32_t n_shared, int32_t top_k) {
  const Sizes z = sizes(n_tokens, n_experts, n_shared, top_k);
  Carver c(p);
  FwdScratch f;
  f.hid = c.take(size_t(z.l_cap) * d_hidden * 2);
  f.block_hist_bytes = moe_b200_router_dispatch_scratch_bytes(n_tokens, z.n_all);
  f.block_hist = c.take(f.block_hist_bytes);
  f.colsum = static_cast<float*>(c.take(size_t(n_experts) * 4));
  f.total = c.used;
  return f;
}

struct InferScratch {
  void *logits, *w_all, *hid, *y, *block_hist;
  int64_t* idx_all;
  int32_t *sorted_ids, *expert_ids, *pad_offsets, *counts, *n_post_pad, *inv_ids;
  size_t block_hist_bytes, total;
};
InferScratch carve_infer(void* p, int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                         int32_t n_experts, int32_t n_shared, int32_t top_k) {
  const Sizes z = sizes(n_tokens, n_experts, n_shared, top_k);
  Carver c(p);
  InferScratch f;
  f.logits = c.take(size_t(n_tokens) * z.ld * 2);
  f.w_all = c.take(size_t(z.m) * 2);
  f.idx_all = static_cast<int64_t*>(c.take(size_t(z.m) * 8));
  f.sorted_ids = static_cast<int32_t*>(c.take(size_t(z.l_cap) * 4));
  f.expert_ids = static_cast<int32_t*>(c.take(size_t(z.l_cap / 128 + 1) * 4));
  f.pad_offsets = static_cast<int32_t*>(c.take(size_t(z.n_all + 1) * 4));
  f.counts = static_cast<int32_t*>(c.take(size_t(z.n_all) * 4));
  f.n_post_pad = static_cast<int32_t*>(c.take(4));
  f.inv_ids = static_cast<int32_t*>(c.take(size_t(z.m) * 4));
  f.block_hist_bytes = moe_b200_router_dispatch_scratch_bytes(n_tokens, z.n_all);
  f.block_hist = c.take(f.block_hist_bytes);
  f.hid = c.take(size_t(z.l_cap) * d_hidden * 2);
  f.y = c.take(size_t(z.l_cap) * d_model * 2);
  f.total = c.used;
  return f;
}

struct BwdScratch {
  void *douts, *da1, *hidw, *dtw, *dl, *d_router_padded, *part_in, *part_out, *part_r;
  size_t part_in_bytes, part_out_bytes, part_r_bytes, total;
};
int carve_bwd(void* p, int64_t n_tokens, int32_t d_model, int32_t d_hidden, int32_t n_experts,
              int32_t n_shared, int32_t top_k, BwdScratch* b) {
  const Sizes z = sizes(n_tokens, n_experts, n_shared, top_k);
  Carver c(p);
  b->douts = c.take(size_t(z.l_cap) * d_model * 2);
  b->da1 = c.take(size_t(z.l_cap) * 2 * d_hidden * 2);
  b->hidw = c.take(size_t(z.l_cap) * d_hidden * 2);
  b->dtw = c.take(size_t(z.m) * 2);
  b->dl = c.take(size_t(n_tokens) * z.ld * 2);
  b->d_router_padded = c.take(size_t(d_model) * z.ld * 2);
  int rc = moe_b200_wgrad_scratch_bytes(d_model, 2 * d_hidden, z.l_cap, z.n_all, 1, 0,
                                        &b->part_in_bytes);
  if (rc != MOE_B200_OK) return rc;
  rc = moe_b200_wgrad_scratch_bytes(d_hidden, d_model, z.l_cap, z.n_all, 1, 0, &b->part_out_bytes);
  if (rc != MOE_B200_OK) return rc;
  rc = moe_b200_wgrad_scratch_bytes(d_model, z.ld, n_tokens, 1, 0, 0, &b->part_r_bytes);
  if (rc != MOE_B200_OK) return rc;
  b->part_in = c.take(b->part_in_bytes);
  b->part_out = c.take(b->part_out_bytes);
  b->part_r = c.take(b->part_r_bytes);
  b->total = c.used;
  return MOE_B200_OK;
}

inline bool bad_shape(int64_t n_tokens, int32_t d_model, int32_t d_hidden, int32_t n_experts,
                      int32_t n_shared, int32_t top_k) {
  return n_tokens < 1 || d_model < 64 || d_hidden < 1 || n_experts < 1 || n_shared < 0 ||
         top_k < 1 || top_k > n_experts;
}

#define STEP(call)                   \
  do {                               \
    const int rc_ = (call);          \
    if (rc_ != MOE_B200_OK) return rc_; \
    ++launched;                      \
  } while (0)

}  // namespace

extern "C" {

size_t moe_b200_block_fwd_scratch_bytes(int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                                        int32_t n_experts, int32_t n_shared, int32_t top_k) {
  if (bad_shape(n_tokens, d_model, d_hidden, n_experts, n_shared, top_k)) return 0;
  return carve_fwd(nullptr, n_tokens, d_hidden, n_experts, n_shared, top_k).total;
}

size_t moe_b200_block_infer_scratch_bytes(int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                                          int32_t n_experts, int32_t n_shared, int32_t top_k) {
  if (bad_shape(n_tokens, d_model, d_hidden, n_experts, n_shared, top_k)) return 0;
  return carve_infer(nullptr, n_tokens, d_model, d_hidden, n_experts, n_shared, top_k).total;
}

int moe_b200_block_infer(const void* x, int64_t n_tokens, int32_t d_model,
                         const void* router_w_padded, const float* logit_bias, const void* w_in,
                         const void* w_out, int32_t n_experts, int32_t d_hidden,
                         const void* w_sh_in, const void* w_sh_out, int32_t n_shared,
                         int32_t top_k, int32_t normalize, int32_t activation,
                         const void* residual, int32_t atomic_combine, void* out, void* scratch,
                         size_t scratch_bytes, int32_t* n_launches, int32_t* status,
                         void* stream) {
  if (bad_shape(n_tokens, d_model, d_hidden, n_experts, n_shared, top_k)) return MOE_B200_ERR_SHAPE;
  if (!x || !router_w_padded || !w_in || !w_out || !out || !scratch || !status)
    return MOE_B200_ERR_NULL;
  if (n_shared > 0 && (!w_sh_in || !w_sh_out)) return MOE_B200_ERR_NULL;
  const InferScratch f = carve_infer(scratch, n_tokens, d_model, d_hidden, n_experts, n_shared, top_k);
  if (scratch_bytes < f.total) return MOE_B200_ERR_SCRATCH;
  const Sizes z = sizes(n_tokens, n_experts, n_shared, top_k);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int launched = 0;
  STEP(moe_b200_down_gemm(x, n_tokens, d_model, router_w_padded, 1, nullptr, 0, z.ld, nullptr,
                          nullptr, 1, nullptr, nullptr, 0, f.logits, nullptr, status, stream));
  STEP(moe_b200_router_dispatch(f.logits, z.ld, logit_bias, nullptr, n_tokens, n_experts, top_k,
                                n_shared, normalize, 0, f.w_all, f.idx_all, nullptr, f.sorted_ids,
                                f.expert_ids, f.pad_offsets, f.counts, f.n_post_pad, f.inv_ids,
                                f.block_hist, f.block_hist_bytes, status, stream));
  if (n_tokens > 128) ++launched;   // the dispatch's scatter pass is a launch of its own
  // up/gate GEMM gathering the token rows itself (no permuted copy), then down GEMM + combine
  STEP(moe_b200_up_gemm(x, z.l_cap, d_model, w_in, n_experts, w_sh_in, n_shared, d_hidden,
                        f.expert_ids, f.n_post_pad, 0, f.sorted_ids, z.ks, z.m, activation, f.hid,
                        nullptr, nullptr, 0, nullptr, nullptr, status, stream));
  if (atomic_combine) {
    if (residual) STEP(copy_words(residual, out, n_tokens * d_model / 2, st));
    else STEP(zero_words(out, n_tokens * d_model / 2, st));
    STEP(moe_b200_down_gemm_acc(f.hid, z.l_cap, d_hidden, w_out, n_experts, w_sh_out, n_shared,
                                d_model, f.expert_ids, f.n_post_pad, 0, f.sorted_ids, f.w_all,
                                z.m, z.ks, out, n_tokens, nullptr, status, stream));
  } else {
    STEP(moe_b200_down_gemm(f.hid, z.l_cap, d_hidden, w_out, n_experts, w_sh_out, n_shared,
                            d_model, f.expert_ids, f.n_post_pad, 0, f.sorted_ids, f.w_all, z.m,
                            f.y, nullptr, status, stream));
    STEP(moe_b200_combine(f.y, f.inv_ids, n_tokens, z.ks, d_model, residual, nullptr, out, stream));
  }
  if (n_launches) *n_launches = launched;
  return MOE_B200_OK;
}

size_t moe_b200_block_bwd_scratch_bytes(int64_t n_tokens, int32_t d_model, int32_t d_hidden,
                                        int32_t n_experts, int32_t n_shared, int32_t top_k) {
  if (bad_shape(n_tokens, d_model, d_hidden, n_experts, n_shared, top_k)) return 0;
  BwdScratch b;
  if (carve_bwd(nullptr, n_tokens, d_model, d_hidden, n_experts, n_shared, top_k, &b) !=
      MOE_B200_OK)
    return 0;
  return b.total;
}

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
                       int32_t* n_launches, int32_t* status, void* stream) {
  if (bad_shape(n_tokens, d_model, d_hidden, n_experts, n_shared, top_k)) return MOE_B200_ERR_SHAPE;
  if (!x || !router_w || !w_in || !w_out || !out || !aux || !counts || !xs || !a1 || !logits ||
      !w_all || !idx_all || !sorted_ids || !expert_ids || !pad_offsets || !counts_all ||
      !n_post_pad || !inv_ids || !router_w_padded || !scratch || !status)
    return MOE_B200_ERR_NULL;
  if (n_shared > 0 && (!w_sh_in || !w_sh_out)) return MOE_B200_ERR_NULL;
  const FwdScratch f = carve_fwd(scratch, n_tokens, d_hidden, n_experts, n_shared, top_k);
  if (scratch_bytes < f.total) return MOE_B200_ERR_SCRATCH;
  const Sizes z = sizes(n_tokens, n_experts, n_shared, top_k);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int launched = 0;
  const int32_t* first_shared = pad_offsets + n_experts;   // start of the first shared run

  // router: zero-padded weight, logits GEMM (one fixed group, no pair weights), routing + dispatch
  float* colsum = full_softmax ? f.colsum : nullptr;
  STEP(pad_router(router_w, d_model, n_experts, router_w_padded, z.ld, colsum, st));
  STEP(moe_b200_down_gemm(x, n_tokens, d_model, router_w_padded, 1, nullptr, 0, z.ld, nullptr,
                          nullptr, 1, nullptr, nullptr, 0, logits, nullptr, status, stream));
  STEP(moe_b200_router_dispatch(logits, z.ld, logit_bias, noise, n_tokens, n_experts, top_k,
                                n_shared, normalize, full_softmax, w_all, idx_all, colsum,
                                sorted_ids, expert_ids, pad_offsets, counts_all, n_post_pad,
                                inv_ids, f.block_hist, f.block_hist_bytes, status, stream));
  ++launched;   // (two launches, one for batches of up to 128 tokens: counted as two)
  // experts: permute the routed rows, up/gate + GLU, down with the combine in its epilogue
  STEP(moe_b200_permute(x, n_tokens, d_model, z.ks, sorted_ids,
                        n_shared ? first_shared : n_post_pad, z.l_cap, xs, stream));
  STEP(moe_b200_up_gemm(xs, z.l_cap, d_model, w_in, n_experts, w_sh_in, n_shared, d_hidden,
                        expert_ids, n_post_pad, 0, nullptr, 0, 0, activation, f.hid, a1,
                        n_shared ? x : nullptr, n_shared ? n_tokens : 0, pad_offsets, nullptr,
                        status, stream));
  if (n_shared) {
    STEP(moe_b200_down_gemm_sum(f.hid, z.l_cap, d_hidden, w_sh_out, n_shared, d_model,
                                first_shared, n_tokens, out, status, stream));
    STEP(moe_b200_down_gemm_acc(f.hid, z.l_cap, d_hidden, w_out, n_experts, nullptr, 0, d_model,
                                expert_ids, first_shared, 0, sorted_ids, w_all, z.m, z.ks, out,
                                n_tokens, nullptr, status, stream));
  } else {
    STEP(zero_words(out, n_tokens * d_model / 2, st));
    STEP(moe_b200_down_gemm_acc(f.hid, z.l_cap, d_hidden, w_out, n_experts, nullptr, 0, d_model,
                                expert_ids, n_post_pad, 0, sorted_ids, w_all, z.m, z.ks, out,
                                n_tokens, nullptr, status, stream));
  }
  STEP(finish_fwd(counts_all, counts, colsum, n_experts, n_tokens, aux_coef, aux, st));
  if (n_launches) *n_launches = launched;
  return MOE_B200_OK;
}

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
                       int32_t* n_launches, int32_t* status, void* stream) {
  if (bad_shape(n_tokens, d_model, d_hidden, n_experts, n_shared, top_k)) return MOE_B200_ERR_SHAPE;
  if (!grad_out || !x || !w_in || !w_out || !xs || !a1 || !logits || !w_all || !idx_all ||
      !sorted_ids || !expert_ids || !pad_offsets || !counts_all || !n_post_pad ||
      !router_w_padded || !dx || !d_router || !dw_in || !dw_out || !scratch || !status)
    return MOE_B200_ERR_NULL;
  if (n_shared > 0 && (!w_sh_in || !w_sh_out || !dw_sh_in || !dw_sh_out)) return MOE_B200_ERR_NULL;
  BwdScratch b;
  const int rcb = carve_bwd(scratch, n_tokens, d_model, d_hidden, n_experts, n_shared, top_k, &b);
  if (rcb != MOE_B200_OK) return rcb;
  if (scratch_bytes < b.total) return MOE_B200_ERR_SCRATCH;
  const Sizes z = sizes(n_tokens, n_experts, n_shared, top_k);
  cudaStream_t main_st = static_cast<cudaStream_t>(stream);
  // the two side branches run on the caller's side streams, or in line when none are given
  cudaStream_t sa = side_stream_a ? static_cast<cudaStream_t>(side_stream_a) : main_st;
  cudaStream_t sb = side_stream_b ? static_cast<cudaStream_t>(side_stream_b) : main_st;
  int launched = 0;
  const int32_t* first_shared = pad_offsets + n_experts;
  const int32_t* live = n_shared ? first_shared : n_post_pad;

  STEP(moe_b200_permute(grad_out, n_tokens, d_model, z.ks, sorted_ids, live, z.l_cap, b.douts,
                        stream));
  STEP(moe_b200_dhidden_glu_bwd(b.douts, z.l_cap, d_model, w_out, n_experts, w_sh_out, n_shared,
                                d_hidden, expert_ids, n_post_pad, 0, sorted_ids, 0, w_all, z.m,
                                a1, activation, b.da1, b.hidw, b.dtw,
                                n_shared ? grad_out : nullptr, n_shared ? n_tokens : 0,
                                n_shared ? pad_offsets : nullptr, status, stream));
  // fork: everything below depends only on the two launches above
  cudaEvent_t ev_fork = nullptr, ev_dx = nullptr, ev_a = nullptr, ev_b = nullptr;
  auto fail = [&](int code) {
    for (cudaEvent_t e : {ev_fork, ev_dx, ev_a, ev_b})
      if (e) cudaEventDestroy(e);
    return code;
  };
  for (cudaEvent_t* e : {&ev_fork, &ev_dx, &ev_a, &ev_b})
    if (cudaEventCreateWithFlags(e, cudaEventDisableTiming) != cudaSuccess)
      return fail(MOE_B200_ERR_CUDA);
#define STEP_F(call)                          \
  do {                                        \
    const int rc_ = (call);                   \
    if (rc_ != MOE_B200_OK) return fail(rc_); \
    ++launched;                               \
  } while (0)
#define CU_F(call) \
  if ((call) != cudaSuccess) return fail(MOE_B200_ERR_CUDA)
  CU_F(cudaEventRecord(ev_fork, main_st));
  if (sa != main_st) CU_F(cudaStreamWaitEvent(sa, ev_fork, 0));
  if (sb != main_st) CU_F(cudaStreamWaitEvent(sb, ev_fork, 0));

  // main: dx's first value (the shared experts' share, stored), dW_in, the routed rows of dx
  if (n_shared) {
    STEP_F(moe_b200_dx_gemm_sum(b.da1, z.l_cap, d_hidden, w_sh_in, n_shared, d_model,
                                first_shared, n_tokens, dx, status, stream));
  } else {
    STEP_F(zero_words(dx, n_tokens * d_model / 2, main_st));
  }
  CU_F(cudaEventRecord(ev_dx, main_st));
  STEP_F(moe_b200_wgrad(xs, 0, d_model, b.da1, 0, 2 * d_hidden, z.l_cap, pad_offsets, z.n_all, 0,
                        nullptr, 0, 0, 0, dw_in, n_experts, n_shared ? dw_sh_in : nullptr,
                        b.part_in, b.part_in_bytes, n_shared ? x : nullptr,
                        n_shared ? n_tokens : 0, n_shared ? 1 : 0, status, stream));
  STEP_F(moe_b200_dx_gemm_acc(b.da1, z.l_cap, d_hidden, w_in, n_experts, nullptr, 0, d_model,
                              expert_ids, live, 0, sorted_ids, z.m, z.ks, dx, n_tokens,
                              pad_offsets, status, stream));
  // side a: dW_out
  STEP_F(moe_b200_wgrad(b.hidw, 0, d_hidden, b.douts, 0, d_model, z.l_cap, pad_offsets, z.n_all,
                        0, nullptr, 0, 0, 0, dw_out, n_experts, n_shared ? dw_sh_out : nullptr,
                        b.part_out, b.part_out_bytes, n_shared ? grad_out : nullptr,
                        n_shared ? n_tokens : 0, n_shared ? 2 : 0, status, sa));
  // side b: the router's backward, its weight gradient, its share of dx
  STEP_F(moe_b200_router_fused_bwd(logits, z.ld, logit_bias, noise, idx_all, b.dtw, n_tokens,
                                   n_experts, top_k, n_shared, normalize, full_softmax, grad_aux,
                                   counts_all, aux_coef, b.dl, z.ld, sb));
  STEP_F(moe_b200_wgrad(x, 0, d_model, b.dl, 0, z.ld, n_tokens, nullptr, 1, 0, nullptr, 0, 0, 0,
                        b.d_router_padded, 1, nullptr, b.part_r, b.part_r_bytes, nullptr, 0, 0,
                        status, sb));
  STEP_F(moe_b200_copy_cols(b.d_router_padded, d_model, n_experts, z.ld, d_router, n_experts, sb));
  if (sb != main_st) CU_F(cudaStreamWaitEvent(sb, ev_dx, 0));
  STEP_F(moe_b200_dx_gemm_acc(b.dl, n_tokens, z.ld / 2, router_w_padded, 1, nullptr, 0, d_model,
                              nullptr, nullptr, 1, nullptr, 0, 1, dx, n_tokens, nullptr, status,
                              sb));
  // join
  if (sa != main_st) {
    CU_F(cudaEventRecord(ev_a, sa));
    CU_F(cudaStreamWaitEvent(main_st, ev_a, 0));
  }
  if (sb != main_st) {
    CU_F(cudaEventRecord(ev_b, sb));
    CU_F(cudaStreamWaitEvent(main_st, ev_b, 0));
  }
#undef STEP_F
#undef CU_F
  fail(0);   // the events are released once their work has completed
  if (n_launches) *n_launches = launched + 3;   // the three weight gradients may add a reduction pass
  return MOE_B200_OK;
}

}  // extern "C"
