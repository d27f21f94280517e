// Routing for the dropless MoE block: top-k selection with softmax weights (and its backward),
// then the dispatch plan -- per-expert histogram, 128-aligned run offsets, tile->expert map and a
// STABLE counting-sort permutation (inside a run, pairs keep ascending pair id, which is the order
// a stable sort of the flat expert ids gives).
//
// All kernels are integer / fp32 SIMT work bound by HBM and latency: warp shuffles and
// __match_any_sync do the selection and ranking, global accesses are 16-byte vectors where the
// layout allows.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <mutex>

#include "../../include/moe_b200.h"
#include "pdl.cuh"
#include "gemm.cuh"  // DevStatus
#include "routing.cuh"
#include "dispatch_scatter.cuh"

namespace moe {


// One warp per token; lane l holds experts l, l+32, ... (NSLOT of them). A winner is found with two
// hardware warp reductions: the largest key, then the smallest expert index among the lanes that
// hold it -- i.e. descending value, ties to the lowest index, and the output comes out sorted.
// full_softmax != 0 : weights come from the softmax over all experts (renormalised over the k
//                     winners when normalize != 0 and k > 1), and probs [T,E] is written if given.
// full_softmax == 0 : normalize != 0 -> softmax over the k winning logits;
//                     normalize == 0 -> the full-softmax probabilities of the winners.
template <int NSLOT>
__global__ void __launch_bounds__(256)
    router_topk_kernel(const float* __restrict__ logits, int64_t n_tokens, int n_experts, int top_k,
                       int normalize, int full_softmax, float* __restrict__ topk_w,
                       int64_t* __restrict__ topk_idx, float* __restrict__ probs) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (t >= n_tokens) return;
  const float* row = logits + t * n_experts;

  float v[NSLOT];
  uint32_t key[NSLOT];  // 0 = not a candidate (out of range or already taken)
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) {
    const int e = i * 32 + lane;
    const bool in = e < n_experts;
    v[i] = in ? row[e] : -CUDART_INF_F;
    // float_key is never 0 for a real value except -NaN patterns; +1 saturating keeps 0 free
    const uint32_t fk = float_key(v[i]);
    key[i] = in ? (fk == 0u ? 1u : fk) : 0u;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  const bool need_full = full_softmax || !normalize;
  float denom = 0.f;
  if (need_full) {
#pragma unroll
    for (int i = 0; i < NSLOT; ++i)
      if (i * 32 + lane < n_experts) denom += expf(v[i] - mx);
#pragma unroll
    for (int o = 16; o; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    if (probs != nullptr) {
#pragma unroll
      for (int i = 0; i < NSLOT; ++i) {
        const int e = i * 32 + lane;
        if (e < n_experts) probs[t * n_experts + e] = expf(v[i] - mx) / denom;
      }
    }
  }

  float sel_val = 0.f;  // lane j < top_k keeps the j-th winner
  int sel_idx = 0;
  for (int j = 0; j < top_k; ++j) {
    uint32_t best = 0u;
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) best = key[i] > best ? key[i] : best;
    const uint32_t top = __reduce_max_sync(0xffffffffu, best);
    uint32_t cand = 0xFFFFFFFFu;  // lowest expert index in this lane that holds the top key
#pragma unroll
    for (int i = NSLOT - 1; i >= 0; --i)
      if (key[i] == top) cand = uint32_t(i * 32 + lane);
    const int e_win = int(__reduce_min_sync(0xffffffffu, cand));
    const int owner = e_win & 31, slot = e_win >> 5;
    float val = 0.f;
#pragma unroll
    for (int i = 0; i < NSLOT; ++i)
      if (i == slot) {
        val = v[i];
        if (lane == owner) key[i] = 0u;
      }
    val = __shfl_sync(0xffffffffu, val, owner);
    if (lane == j) {
      sel_val = val;
      sel_idx = e_win;
    }
  }

  // weights: lanes [0, top_k) hold the winners
  float wgt;
  const bool active = lane < top_k;
  if (need_full) {
    wgt = active ? expf(sel_val - mx) / denom : 0.f;
    if (normalize && top_k > 1 && full_softmax) {
      float s = wgt;
#pragma unroll
      for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      wgt = wgt / s;
    }
  } else {
    // softmax over the k winning logits; the first winner is the row maximum
    const float top = __shfl_sync(0xffffffffu, sel_val, 0);
    const float ex = active ? expf(sel_val - top) : 0.f;
    float s = ex;
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    wgt = ex / s;
  }
  if (active) {
    topk_w[t * top_k + lane] = wgt;
    topk_idx[t * top_k + lane] = sel_idx;
  }
}

// Backward of router_topk w.r.t. the logits. Recomputes the softmax from the saved logits.
//   full_softmax, normalize, k>1 : w_i = p_i / s,  s = sum_{i in S} p_i
//        dp_i = (dw_i - sum_j dw_j w_j) / s on S;  dp += d_probs;  dl = p * (dp - <p, dp>)
//   full_softmax, else           : dp_i = dw_i on S (+ d_probs), same softmax Jacobian
//   !full_softmax, normalize     : dl_i = w_i (dw_i - sum_j w_j dw_j) on S, 0 elsewhere
//   !full_softmax, !normalize    : dp_i = dw_i on S, softmax Jacobian
template <int NSLOT>
__global__ void __launch_bounds__(256)
    router_topk_bwd_kernel(const float* __restrict__ logits, const int64_t* __restrict__ topk_idx,
                           const float* __restrict__ d_topk_w, const float* __restrict__ d_probs,
                           int64_t n_tokens, int n_experts, int top_k, int normalize,
                           int full_softmax, float* __restrict__ d_logits) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (t >= n_tokens) return;
  const float* row = logits + t * n_experts;

  float v[NSLOT], pr[NSLOT], dp[NSLOT];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < n_experts ? row[e] : -CUDART_INF_F;
    mx = fmaxf(mx, v[i]);
    dp[i] = 0.f;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

  const bool active = lane < top_k;
  const int my_idx = active ? int(topk_idx[t * top_k + lane]) : -1;
  const float my_dw = active ? d_topk_w[t * top_k + lane] : 0.f;
  const bool need_full = full_softmax || !normalize;

  if (!need_full) {
    // local softmax over the winners
    float my_l = 0.f;
    {
      // fetch my winner's logit from the owning lane's registers via shared index math
      my_l = active ? row[my_idx] : -CUDART_INF_F;
    }
    float top = my_l;
#pragma unroll
    for (int o = 16; o; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
    const float ex = active ? expf(my_l - top) : 0.f;
    float s = ex;
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float w = ex / s;
    float dot = w * my_dw;
#pragma unroll
    for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    // zero the row, then scatter the k entries
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      if (e < n_experts) d_logits[t * n_experts + e] = 0.f;
    }
    __syncwarp();
    if (active) d_logits[t * n_experts + my_idx] = w * (my_dw - dot);
    return;
  }

  float denom = 0.f;
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) {
    pr[i] = (i * 32 + lane < n_experts) ? expf(v[i] - mx) : 0.f;
    denom += pr[i];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) pr[i] /= denom;

  // probability of my winner
  float my_p = active ? expf(row[my_idx] - mx) / denom : 0.f;
  float my_dp = my_dw;
  if (normalize && top_k > 1 && full_softmax) {
    float s = my_p;
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float w = my_p / s;
    float dot = my_dw * w;
#pragma unroll
    for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    my_dp = (my_dw - dot) / s;
  }
  // scatter winners' dp into the per-lane expert slots
  for (int j = 0; j < top_k; ++j) {
    const int e = __shfl_sync(0xffffffffu, my_idx, j);
    const float d = __shfl_sync(0xffffffffu, my_dp, j);
    if ((e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < NSLOT; ++i)
        if (i == (e >> 5)) dp[i] += d;
    }
  }
  if (d_probs != nullptr) {
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      if (e < n_experts) dp[i] += d_probs[t * n_experts + e];
    }
  }
  float inner = 0.f;
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) inner += pr[i] * dp[i];
#pragma unroll
  for (int o = 16; o; o >>= 1) inner += __shfl_xor_sync(0xffffffffu, inner, o);
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) {
    const int e = i * 32 + lane;
    if (e < n_experts) d_logits[t * n_experts + e] = pr[i] * (dp[i] - inner);
  }
}

// ------------------------------------------------------------------------------- dispatch
// Stable counting sort of the pairs by expert in two launches. The pairs are cut into at most
// DISPATCH_MAX_BLOCKS chunks of `chunk` pairs (a power-of-two multiple of 1024), one block each.
static int64_t dispatch_chunk(int64_t n_pairs) {
  int64_t chunk = DISPATCH_MIN_CHUNK;
  while ((n_pairs + chunk - 1) / chunk > DISPATCH_MAX_BLOCKS) chunk *= 2;
  return chunk;
}

// Pass 1: per-block histogram of expert ids -> block_hist[expert][block]; also paints this block's
// share of sorted_ids with the sentinel so pad slots need no separate fill launch.
__global__ void __launch_bounds__(DISPATCH_THREADS)
    dispatch_hist_kernel(const int64_t* __restrict__ topk_idx, int64_t n_pairs, int n_experts,
                         int chunk, int32_t* __restrict__ block_hist,
                         int32_t* __restrict__ sorted_ids, int64_t l_cap, int32_t* status) {
  pdl_trigger();
  pdl_wait();
  __shared__ int32_t hist[MAX_EXPERTS];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int64_t base = int64_t(blockIdx.x) * chunk;
  for (int i = threadIdx.x; i < chunk; i += blockDim.x) {
    const int64_t pidx = base + i;
    if (pidx < n_pairs) {
      const int64_t e = topk_idx[pidx];
      if (e >= 0 && e < n_experts)
        atomicAdd(&hist[int(e)], 1);
      else
        atomicExch(status, ST_BAD_EXPERT);
    }
  }
  // sentinel fill: each block paints an equal slice of [0, l_cap)
  const int64_t per = (l_cap + gridDim.x - 1) / gridDim.x;
  const int64_t lo = per * blockIdx.x;
  const int64_t hi = lo + per < l_cap ? lo + per : l_cap;
  for (int64_t s = lo + threadIdx.x; s < hi; s += blockDim.x) sorted_ids[s] = int32_t(n_pairs);
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
    block_hist[int64_t(e) * gridDim.x + blockIdx.x] = hist[e];
}

// Pass 2 (dispatch_scatter.cuh): plan + stable scatter, one block per chunk.
__global__ void __launch_bounds__(DISPATCH_THREADS)
    dispatch_scatter_kernel(const int64_t* __restrict__ topk_idx, int64_t n_pairs, int n_experts,
                            int chunk, int n_blocks, const int32_t* __restrict__ block_hist,
                            int32_t* __restrict__ counts, int32_t* __restrict__ pad_offsets,
                            int32_t* __restrict__ n_post_pad, int32_t* __restrict__ expert_ids,
                            int64_t n_tiles_cap, int32_t* __restrict__ sorted_ids,
                            int32_t* __restrict__ inv_ids, int32_t capacity, int32_t n_capped) {
  pdl_trigger();
  pdl_wait();
  dispatch_scatter_body<false>(topk_idx, n_pairs, n_experts, chunk, n_blocks, block_hist, counts,
                               pad_offsets, n_post_pad, expert_ids, n_tiles_cap, sorted_ids, inv_ids,
                               capacity, n_capped, int(blockIdx.x), int(gridDim.x));
}

// Both dispatch entry points: histogram pass, then plan + scatter.
static int launch_dispatch(const int64_t* topk_idx, int64_t n_pairs, int32_t n_experts,
                           int32_t* sorted_ids, int32_t* expert_ids, int32_t* pad_offsets,
                           int32_t* counts, int32_t* n_post_pad, int32_t* inv_ids,
                           int32_t* block_hist, int32_t* status, cudaStream_t st,
                           int32_t capacity = 0, int32_t n_capped = 0) {
  const int64_t l_cap = moe_b200_l_cap(n_pairs, n_experts);
  const int chunk = int(dispatch_chunk(n_pairs));
  const int blocks = int((n_pairs + chunk - 1) / chunk);
  if (blocks > 0)
    launch_pdl(dispatch_hist_kernel, dim3(blocks), dim3(DISPATCH_THREADS), 0, st, topk_idx, n_pairs,
               n_experts, chunk, block_hist, sorted_ids, l_cap, status);
  launch_pdl(dispatch_scatter_kernel, dim3(blocks > 0 ? blocks : 1), dim3(DISPATCH_THREADS), 0, st,
             topk_idx, n_pairs, n_experts, chunk, blocks, block_hist, counts, pad_offsets,
             n_post_pad, expert_ids, l_cap / ALIGN_M, sorted_ids, inv_ids, capacity, n_capped);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // namespace moe

using namespace moe;

extern "C" {

int64_t moe_b200_l_cap(int64_t n_pairs, int32_t n_experts) {
  const int64_t live = n_pairs < n_experts ? n_pairs : n_experts;
  return (n_pairs + live * (ALIGN_M - 1) + ALIGN_M - 1) / ALIGN_M * ALIGN_M;
}

size_t moe_b200_dispatch_scratch_bytes(int64_t n_pairs, int32_t n_experts) {
  if (n_pairs < 0) n_pairs = 0;
  const int64_t chunk = dispatch_chunk(n_pairs);
  const int64_t blocks = (n_pairs + chunk - 1) / chunk;
  return size_t(blocks > 0 ? blocks : 1) * size_t(n_experts) * sizeof(int32_t);
}

int moe_b200_router_topk(const float* logits, int64_t n_tokens, int32_t n_experts, int32_t top_k,
                         int32_t normalize, int32_t full_softmax, float* topk_w, int64_t* topk_idx,
                         float* probs, void* stream) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS || top_k < 1 || top_k > n_experts ||
      top_k > MAX_TOPK || n_tokens < 0)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!logits || !topk_w || !topk_idx) return MOE_B200_ERR_NULL;
  const int64_t threads = n_tokens * 32;
  const unsigned grid = unsigned((threads + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LAUNCH(NS)                                                                          \
  launch_pdl(router_topk_kernel<NS>, dim3(grid), dim3(256), 0, st, logits, n_tokens, n_experts, top_k, normalize, \
                                               full_softmax, topk_w, topk_idx, probs)
  const int nslot = (n_experts + 31) / 32;
  if (nslot <= 1) LAUNCH(1);
  else if (nslot <= 2) LAUNCH(2);
  else if (nslot <= 3) LAUNCH(3);
  else if (nslot <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_router_topk_bwd(const float* logits, const int64_t* topk_idx, const float* d_topk_w,
                             const float* d_probs, int64_t n_tokens, int32_t n_experts,
                             int32_t top_k, int32_t normalize, int32_t full_softmax,
                             float* d_logits, void* stream) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS || top_k < 1 || top_k > n_experts ||
      top_k > MAX_TOPK || n_tokens < 0)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!logits || !topk_idx || !d_topk_w || !d_logits) return MOE_B200_ERR_NULL;
  const int64_t threads = n_tokens * 32;
  const unsigned grid = unsigned((threads + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LAUNCH(NS)                                                                             \
  launch_pdl(router_topk_bwd_kernel<NS>, dim3(grid), dim3(256), 0, st, logits, topk_idx, d_topk_w, d_probs, n_tokens, \
                                                   n_experts, top_k, normalize, full_softmax,     \
                                                   d_logits)
  const int nslot = (n_experts + 31) / 32;
  if (nslot <= 1) LAUNCH(1);
  else if (nslot <= 2) LAUNCH(2);
  else if (nslot <= 3) LAUNCH(3);
  else if (nslot <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_dispatch(const int64_t* topk_idx, int64_t n_pairs, int32_t n_experts,
                      int32_t* sorted_ids, int32_t* expert_ids, int32_t* pad_offsets,
                      int32_t* counts, int32_t* n_post_pad, int32_t* inv_ids, void* scratch,
                      size_t scratch_bytes, int32_t capacity, int32_t n_capped, int32_t* status,
                      void* stream) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS || n_pairs < 0 || n_pairs > (int64_t(1) << 30) ||
      capacity < 0 || n_capped < 0 || n_capped > n_experts)
    return MOE_B200_ERR_SHAPE;
  if (n_pairs && (!sorted_ids || !topk_idx || !inv_ids)) return MOE_B200_ERR_NULL;
  if (!pad_offsets || !counts || !n_post_pad || !status) return MOE_B200_ERR_NULL;
  if (scratch_bytes < moe_b200_dispatch_scratch_bytes(n_pairs, n_experts) || !scratch)
    return MOE_B200_ERR_SCRATCH;
  return launch_dispatch(topk_idx, n_pairs, n_experts, sorted_ids, expert_ids, pad_offsets, counts,
                         n_post_pad, inv_ids, static_cast<int32_t*>(scratch), status,
                         static_cast<cudaStream_t>(stream), capacity, n_capped);
}

}  // extern "C"

namespace moe {
// Tokens per block of the fused router + dispatch: a multiple of 128, at most DISPATCH_MAX_BLOCKS
// blocks.
static int64_t router_tokens_per_block(int64_t n_tokens) {
  int64_t tpb = 128;
  while ((n_tokens + tpb - 1) / tpb > DISPATCH_MAX_BLOCKS) tpb *= 2;
  return tpb;
}
}  // namespace moe

extern "C" {

size_t moe_b200_router_dispatch_scratch_bytes(int64_t n_tokens, int32_t n_experts_total) {
  if (n_tokens < 0) n_tokens = 0;
  const int64_t tpb = router_tokens_per_block(n_tokens);
  const int64_t blocks = (n_tokens + tpb - 1) / tpb;
  return size_t(blocks > 0 ? blocks : 1) * size_t(n_experts_total) * sizeof(int32_t);
}

int moe_b200_router_dispatch(const void* logits, int32_t ld, const float* bias,
                             const float* noise, int64_t n_tokens,
                             int32_t n_experts, int32_t top_k, int32_t n_shared,
                             int32_t normalize, int32_t full_softmax, void* w_all,
                             int64_t* idx_all, float* colsum, int32_t* sorted_ids,
                             int32_t* expert_ids, int32_t* pad_offsets, int32_t* counts,
                             int32_t* n_post_pad, int32_t* inv_ids, void* scratch,
                             size_t scratch_bytes, int32_t* status, void* stream) {
  const int32_t n_all = n_experts + n_shared;
  if (n_experts < 1 || n_all > MAX_EXPERTS || top_k < 1 || top_k > n_experts || n_shared < 0 ||
      top_k + n_shared > 32 || top_k > MAX_TOPK || n_tokens < 1 || ld < n_experts ||
      n_tokens * (top_k + n_shared) > (int64_t(1) << 30))
    return MOE_B200_ERR_SHAPE;
  if (!logits || !w_all || !idx_all || !sorted_ids || !pad_offsets || !counts || !n_post_pad ||
      !inv_ids || !status)
    return MOE_B200_ERR_NULL;
  if (!scratch || scratch_bytes < moe_b200_router_dispatch_scratch_bytes(n_tokens, n_all))
    return MOE_B200_ERR_SCRATCH;
  const int kS = top_k + n_shared;
  const int64_t n_pairs = n_tokens * kS;
  const int64_t l_cap = moe_b200_l_cap(n_pairs, n_all);
  const int tpb = int(router_tokens_per_block(n_tokens));
  const int blocks = int((n_tokens + tpb - 1) / tpb);
  int32_t* block_hist = static_cast<int32_t*>(scratch);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // a batch that fits one block (128 tokens) is routed, planned and scattered by ONE launch
  const ScatterArgs sc{counts, pad_offsets, n_post_pad, expert_ids, l_cap / ALIGN_M, inv_ids};
  bool did_scatter = false;
  const int rc = launch_router_fused_chunked(
      static_cast<const __nv_bfloat16*>(logits), ld, bias, noise, n_tokens, n_experts, top_k,
      n_shared,
      normalize, full_softmax, static_cast<__nv_bfloat16*>(w_all), idx_all, colsum, tpb, blocks,
      block_hist, sorted_ids, l_cap, st, &sc, &did_scatter);
  if (rc != MOE_B200_OK) return rc;
  if (did_scatter) return MOE_B200_OK;
  launch_pdl(dispatch_scatter_kernel, dim3(blocks), dim3(DISPATCH_THREADS), 0, st,
             static_cast<const int64_t*>(idx_all), n_pairs, int(n_all), tpb * kS, blocks,
             static_cast<const int32_t*>(block_hist), counts, pad_offsets, n_post_pad, expert_ids,
             l_cap / ALIGN_M, sorted_ids, inv_ids, 0, 0);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // extern "C"

// ------------------------------------------------------- dispatch without caller scratch
// Some hosts cannot hand this library a scratch buffer: a serving process that fixed its whole
// device-memory plan at start-up and forbids any later allocation (a late cudaMalloc can
// synchronise the device and fragment the pool), or a thin foreign-function caller that owns
// pointers for its inputs and outputs but has no device allocator to ask for one more buffer.
// For them the per-block histograms of the dispatch live in this fixed array instead. Every GPU
// that loads the library carries it (128 KB) until the process exits. The dispatch never uses more
// than DISPATCH_MAX_BLOCKS blocks (the chunk a block covers doubles instead) and never more than
// MAX_EXPERTS experts, so the array covers every input the dispatch itself accepts.
constexpr int STATIC_SCRATCH_INTS = DISPATCH_MAX_BLOCKS * MAX_EXPERTS;
static_assert(STATIC_SCRATCH_INTS * sizeof(int32_t) == 128 * 1024, "128 KB of int32");
static __device__ __align__(256) int32_t g_dispatch_scratch[STATIC_SCRATCH_INTS];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_scratch_mutex;
int32_t* g_scratch_ptr[MAX_DEVICES] = {};  // device address of g_dispatch_scratch, per device
}  // namespace

// In host code `g_dispatch_scratch` is only a handle for the symbol, not a device address, so the
// address is looked up once per device (with that device current) and cached.
static int static_scratch_for_current_device(int32_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return MOE_B200_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_dispatch_scratch) != cudaSuccess || p == nullptr)
      return MOE_B200_ERR_CUDA;
    g_scratch_ptr[dev] = static_cast<int32_t*>(p);
  }
  *out = g_scratch_ptr[dev];
  return MOE_B200_OK;
}

extern "C" {

int64_t moe_b200_dispatch_static_max_pairs(int32_t n_experts) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS) return 0;
  return int64_t(1) << 30;   // the dispatch's own limit: the array is never the tighter one
}

int moe_b200_dispatch_static(const int64_t* topk_idx, int64_t n_pairs, int32_t n_experts,
                             int32_t* sorted_ids, int32_t* expert_ids, int32_t* pad_offsets,
                             int32_t* counts, int32_t* n_post_pad, int32_t* inv_ids,
                             int32_t* status, void* stream) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS || n_pairs < 0) return MOE_B200_ERR_SHAPE;
  if (n_pairs > moe_b200_dispatch_static_max_pairs(n_experts) ||
      moe_b200_dispatch_scratch_bytes(n_pairs, n_experts) > sizeof(int32_t) * STATIC_SCRATCH_INTS)
    return MOE_B200_ERR_TOO_LARGE;
  if (n_pairs && (!sorted_ids || !topk_idx || !inv_ids)) return MOE_B200_ERR_NULL;
  if (!pad_offsets || !counts || !n_post_pad || !status) return MOE_B200_ERR_NULL;
  int32_t* block_hist = nullptr;
  const int rc = static_scratch_for_current_device(&block_hist);
  if (rc != MOE_B200_OK) return rc;
  // Nothing in the array has to start at zero: pass 1 overwrites every (expert, block) entry that
  // pass 2 reads, so whatever the previous call left behind is never seen.
  return launch_dispatch(topk_idx, n_pairs, n_experts, sorted_ids, expert_ids, pad_offsets, counts,
                         n_post_pad, inv_ids, block_hist, status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
