// Router kernels of the whole-block op: the same selection and softmax arithmetic as
// router_topk_kernel (routing.cu), but reading the bf16 logits the router GEMM wrote (row stride
// `ld`, optional fp32 per-expert bias), writing weights in the activation dtype, appending the
// shared experts as extra (expert E+s, weight 1) pairs, and reducing the balance-loss statistics
// on the fly -- so that no [T, E] fp32 tensor (logits, probs, d_probs) ever goes through HBM.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/moe_b200.h"
#include "pdl.cuh"
#include "routing.cuh"
#include "dispatch_scatter.cuh"

namespace moe {

constexpr int RF_WARPS = 8;

// Warps stride over tokens. Per token: winners by (value desc, index asc); weights as in
// router_topk_kernel. colsum[e] += sum_t softmax(l_t)[e] (only when full_softmax and colsum given):
// lane-local partial sums, one shared-memory reduction per block, one atomic per block and expert.
// With tokens_per_block > 0 the kernel also does the first pass of the dispatch: block b owns tokens
// [b * tokens_per_block, ...) -- one chunk of the counting sort -- and leaves the chunk's histogram
// of expert ids (shared experts included) in block_hist[expert][block] and its share of the sentinel
// fill of sorted_ids, so that dispatch_scatter_kernel can follow directly.
template <int NSLOT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
    router_fused_kernel(const __nv_bfloat16* __restrict__ logits, int ld,
                        const float* __restrict__ bias, const float* __restrict__ noise, int64_t n_tokens, int n_experts, int top_k,
                        int n_shared, int normalize, int full_softmax,
                        __nv_bfloat16* __restrict__ w_all, int64_t* __restrict__ idx_all,
                        float* __restrict__ colsum, int tokens_per_block,
                        int32_t* __restrict__ block_hist, int32_t* __restrict__ sorted_ids,
                        int64_t l_cap) {
  pdl_trigger();
  pdl_wait();
  __shared__ float cs[WARPS][NSLOT * 32];
  __shared__ int32_t hist[MAX_EXPERTS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool chunked = tokens_per_block > 0;
  if (chunked) {
    for (int e = threadIdx.x; e < n_experts + n_shared; e += blockDim.x) hist[e] = 0;
    __syncthreads();
  }
  const int kS = top_k + n_shared;
  const bool need_full = full_softmax || !normalize;
  const bool want_colsum = full_softmax && colsum != nullptr;

  float b[NSLOT], csum[NSLOT];
#pragma unroll
  for (int i = 0; i < NSLOT; ++i) {
    const int e = i * 32 + lane;
    b[i] = (bias != nullptr && e < n_experts) ? bias[e] : 0.f;
    csum[i] = 0.f;
  }

  const int64_t t_first = chunked ? int64_t(blockIdx.x) * tokens_per_block + warp
                                  : int64_t(blockIdx.x) * WARPS + warp;
  const int64_t t_stride = chunked ? WARPS : int64_t(gridDim.x) * WARPS;
  const int64_t t_hi = chunked ? min(int64_t(blockIdx.x + 1) * tokens_per_block, n_tokens) : n_tokens;
  for (int64_t t = t_first; t < t_hi; t += t_stride) {
    const __nv_bfloat16* row = logits + t * ld;
    float v[NSLOT];
    uint32_t key[NSLOT];  // 0 = not a candidate (out of range or already taken)
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      const bool in = e < n_experts;
      v[i] = in ? __bfloat162float(row[e]) + b[i] +
                      (noise != nullptr ? __ldg(noise + t * n_experts + e) : 0.f)
                : -CUDART_INF_F;
      const uint32_t fk = float_key(v[i]);
      key[i] = in ? (fk == 0u ? 1u : fk) : 0u;
      mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

    float denom = 0.f;
    if (need_full) {
      float ex[NSLOT];
#pragma unroll
      for (int i = 0; i < NSLOT; ++i) {
        ex[i] = (i * 32 + lane < n_experts) ? expf(v[i] - mx) : 0.f;
        denom += ex[i];
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
      if (want_colsum) {
#pragma unroll
        for (int i = 0; i < NSLOT; ++i) csum[i] += ex[i] / denom;
      }
    }

    float sel_val = 0.f;
    int sel_idx = 0;
    for (int j = 0; j < top_k; ++j) {
      uint32_t best = 0u;
#pragma unroll
      for (int i = 0; i < NSLOT; ++i) best = key[i] > best ? key[i] : best;
      const uint32_t top = __reduce_max_sync(0xffffffffu, best);
      uint32_t cand = 0xFFFFFFFFu;
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
      const float top = __shfl_sync(0xffffffffu, sel_val, 0);
      const float ex = active ? expf(sel_val - top) : 0.f;
      float s = ex;
#pragma unroll
      for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      wgt = ex / s;
    }
    if (active) {
      w_all[t * kS + lane] = __float2bfloat16(wgt);
      idx_all[t * kS + lane] = sel_idx;
      if (chunked) atomicAdd(&hist[sel_idx], 1);
    } else if (lane < kS) {  // the shared experts: every token, weight 1
      w_all[t * kS + lane] = __float2bfloat16(1.f);
      idx_all[t * kS + lane] = n_experts + (lane - top_k);
    }
  }

  if (want_colsum) {
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) cs[warp][i * 32 + lane] = csum[i];
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) s += cs[w][e];
      atomicAdd(colsum + e, s);
    }
  }
  if (chunked) {
    __syncthreads();
    const int64_t t_lo = int64_t(blockIdx.x) * tokens_per_block;
    const int32_t mine = int32_t(t_hi > t_lo ? t_hi - t_lo : 0);  // every token visits every shared expert
    for (int e = threadIdx.x; e < n_experts + n_shared; e += blockDim.x)
      block_hist[int64_t(e) * gridDim.x + blockIdx.x] = e < n_experts ? hist[e] : mine;
    // sentinel fill: each block paints an equal slice of [0, l_cap)
    const int64_t n_pairs = n_tokens * kS;
    const int64_t per = (l_cap + gridDim.x - 1) / gridDim.x;
    const int64_t lo = per * blockIdx.x;
    const int64_t hi = lo + per < l_cap ? lo + per : l_cap;
    for (int64_t sl = lo + threadIdx.x; sl < hi; sl += blockDim.x) sorted_ids[sl] = int32_t(n_pairs);
  }
}

// ---------------------------------------------------------------- four lanes per token
// The same routine for the common shapes (at most 96 experts, top_k <= 8), with four lanes per
// token instead of a warp: lane q of a group holds experts [q * EPL, (q + 1) * EPL) in registers,
// so a warp routes eight tokens at once and the cross-lane steps shrink to two shuffle rounds. The
// warp-per-token kernel above spends 611 warp instructions per token on E = 76 (three values per
// lane, every reduction five shuffles deep, most lanes idle in the top-k rounds) and is bound by
// instruction issue; this one needs about a quarter of that.
// Selection rule, softmax arithmetic and outputs are those of router_fused_kernel; sums run in a
// different order, so weights may differ in the last fp32 bit before they are rounded to bf16.
constexpr int RF4_THREADS = 512;
constexpr int RF4_TOKENS = RF4_THREADS / 4;   // tokens per block and pass
constexpr int RF4_MAX_TOPK = 8;

__device__ __forceinline__ float key_float(uint32_t k) {   // inverse of float_key
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

template <int EPL, bool COLSUM>
__global__ void __launch_bounds__(RF4_THREADS)
    router_fused4_kernel(const __nv_bfloat16* __restrict__ logits, int ld,
                         const float* __restrict__ bias, const float* __restrict__ noise, int64_t n_tokens, int n_experts, int top_k,
                         int n_shared, int normalize, int full_softmax,
                         __nv_bfloat16* __restrict__ w_all, int64_t* __restrict__ idx_all,
                         float* __restrict__ colsum, int tokens_per_block,
                         int32_t* __restrict__ block_hist, int32_t* __restrict__ sorted_ids,
                         int64_t l_cap, const ScatterArgs sc) {
  // No early release of the next kernel when a scatter launch follows: with it the step measured
  // 4.5 us slower (the likely reason: the dispatch's scatter blocks, 512 threads each, become
  // resident beside this kernel's blocks, which are short of issue slots as it is). A batch that
  // one block routes, plans and scatters (decode) keeps it: there the launch chain is what counts.
  if (sc.counts != nullptr) pdl_trigger();
  pdl_wait();
  static_assert(EPL % 8 == 0, "a lane loads its experts as 16-byte pieces");
  static_assert(RF4_THREADS == DISPATCH_THREADS, "the scatter pass runs on this kernel's block");
  __shared__ float cs[RF4_THREADS / 32][4 * EPL];
  __shared__ int32_t hist[MAX_EXPERTS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q = lane & 3, sub = lane >> 2;
  const int e0 = q * EPL;
  const bool chunked = tokens_per_block > 0;
  if (chunked) {
    for (int e = threadIdx.x; e < n_experts + n_shared; e += blockDim.x) hist[e] = 0;
    __syncthreads();
  }
  const int kS = top_k + n_shared;
  const bool need_full = full_softmax || !normalize;

  float b[EPL];
  [[maybe_unused]] float csum[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = e0 + i;
    b[i] = (bias != nullptr && e < n_experts) ? bias[e] : 0.f;
    if constexpr (COLSUM) csum[i] = 0.f;
  }

  // block-uniform loop bounds: every warp makes the same number of passes
  const int64_t t_lo = chunked ? int64_t(blockIdx.x) * tokens_per_block
                               : int64_t(blockIdx.x) * RF4_TOKENS;
  const int64_t t_hi = chunked ? min(t_lo + tokens_per_block, n_tokens) : n_tokens;
  const int64_t t_step = chunked ? RF4_TOKENS : int64_t(gridDim.x) * RF4_TOKENS;
  for (int64_t base = t_lo; base < t_hi; base += t_step) {
    const int64_t t = base + warp * 8 + sub;
    const bool valid = t < t_hi;
    const int64_t tc = valid ? t : t_hi - 1;   // lanes past the end repeat the last token, write nothing
    uint32_t key[EPL];   // first the values (as float bits), then the order-preserving keys
    float mx = -CUDART_INF_F;
    {
      const uint4* rp = reinterpret_cast<const uint4*>(logits + tc * ld + e0);
#pragma unroll
      for (int c = 0; c < EPL / 8; ++c) {
        const uint4 r = __ldg(rp + c);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[h]));
          const int i = c * 8 + 2 * h;
          float v0 = (e0 + i < n_experts) ? f.x + b[i] : -CUDART_INF_F;
          float v1 = (e0 + i + 1 < n_experts) ? f.y + b[i + 1] : -CUDART_INF_F;
          if (noise != nullptr) {   // exploration noise, one value per (token, expert)
            if (e0 + i < n_experts) v0 += __ldg(noise + tc * n_experts + e0 + i);
            if (e0 + i + 1 < n_experts) v1 += __ldg(noise + tc * n_experts + e0 + i + 1);
          }
          key[i] = __float_as_uint(v0);
          key[i + 1] = __float_as_uint(v1);
          mx = fmaxf(mx, fmaxf(v0, v1));
        }
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));

    float denom = 0.f;
    if (need_full) {
      float ex[EPL];
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        ex[i] = (e0 + i < n_experts) ? expf(__uint_as_float(key[i]) - mx) : 0.f;
        denom += ex[i];
      }
      denom += __shfl_xor_sync(0xffffffffu, denom, 1);
      denom += __shfl_xor_sync(0xffffffffu, denom, 2);
      if constexpr (COLSUM) {
        const float inv = valid ? 1.f / denom : 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) csum[i] += ex[i] * inv;
      }
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const uint32_t fk = float_key(__uint_as_float(key[i]));
      key[i] = (e0 + i < n_experts) ? (fk == 0u ? 1u : fk) : 0u;
    }

    // top-k: local best (lowest index among equal keys), then two rounds across the four lanes
    float sv[RF4_MAX_TOPK];
    int si[RF4_MAX_TOPK];
#pragma unroll
    for (int j = 0; j < RF4_MAX_TOPK; ++j) {
      sv[j] = 0.f;
      si[j] = 0;
      if (j < top_k) {
        uint32_t bk = 0u;
        int be = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < EPL; ++i)
          if (key[i] > bk) {
            bk = key[i];
            be = e0 + i;
          }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
          const uint32_t ok = __shfl_xor_sync(0xffffffffu, bk, o);
          const int oe = __shfl_xor_sync(0xffffffffu, be, o);
          if (ok > bk || (ok == bk && oe < be)) {
            bk = ok;
            be = oe;
          }
        }
        const int slot = be - e0;   // only the owner's slot is in range
#pragma unroll
        for (int i = 0; i < EPL; ++i)
          if (i == slot) key[i] = 0u;
        sv[j] = key_float(bk);
        si[j] = be;
      }
    }

    // weights of the selected experts (every lane of the group computes all of them)
    float p[RF4_MAX_TOPK];
    if (need_full) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < RF4_MAX_TOPK; ++j) {
        p[j] = j < top_k ? expf(sv[j] - mx) / denom : 0.f;
        s += p[j];
      }
      if (normalize && top_k > 1 && full_softmax) {
#pragma unroll
        for (int j = 0; j < RF4_MAX_TOPK; ++j) p[j] = p[j] / s;
      }
    } else {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < RF4_MAX_TOPK; ++j) {
        p[j] = j < top_k ? expf(sv[j] - sv[0]) : 0.f;
        s += p[j];
      }
#pragma unroll
      for (int j = 0; j < RF4_MAX_TOPK; ++j) p[j] = p[j] / s;
    }
    if (valid) {
#pragma unroll
      for (int j = 0; j < RF4_MAX_TOPK; ++j)
        if (j < top_k && (j & 3) == q) {
          w_all[t * kS + j] = __float2bfloat16(p[j]);
          idx_all[t * kS + j] = si[j];
          if (chunked) atomicAdd(&hist[si[j]], 1);
        }
      for (int jj = top_k + q; jj < kS; jj += 4) {   // the shared experts: every token, weight 1
        w_all[t * kS + jj] = __float2bfloat16(1.f);
        idx_all[t * kS + jj] = n_experts + (jj - top_k);
      }
    }
  }

  if constexpr (COLSUM) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      float s = csum[i];
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      if (lane < 4) cs[warp][e0 + i] = s;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < RF4_THREADS / 32; ++w) s += cs[w][e];
      atomicAdd(colsum + e, s);
    }
  }
  if (chunked) {
    __syncthreads();
    const int32_t mine = int32_t(t_hi > t_lo ? t_hi - t_lo : 0);  // every token visits every shared expert
    for (int e = threadIdx.x; e < n_experts + n_shared; e += blockDim.x)
      block_hist[int64_t(e) * gridDim.x + blockIdx.x] = e < n_experts ? hist[e] : mine;
    // sentinel fill: each block paints an equal slice of [0, l_cap)
    const int64_t n_pairs = n_tokens * kS;
    const int64_t per = (l_cap + gridDim.x - 1) / gridDim.x;
    const int64_t lo = per * blockIdx.x;
    const int64_t hi = lo + per < l_cap ? lo + per : l_cap;
    for (int64_t sl = lo + threadIdx.x; sl < hi; sl += blockDim.x) sorted_ids[sl] = int32_t(n_pairs);
    if (sc.counts != nullptr) {
      // one block holds the whole input: plan and scatter here instead of in a second launch (what
      // this block wrote above is read back through L2 after the barrier)
      __syncthreads();
      dispatch_scatter_body<true>(idx_all, n_pairs, n_experts + n_shared, tokens_per_block * kS, 1,
                                  block_hist, sc.counts, sc.pad_offsets, sc.n_post_pad,
                                  sc.expert_ids, sc.n_tiles_cap, sorted_ids, sc.inv_ids, 0, 0, 0, 1);
    }
  }
}

// Whether the four-lane kernel covers a call, and with how many experts per lane (0 = no).
static int rf4_experts_per_lane(const void* logits, int ld, int n_experts, int top_k) {
  if (top_k > RF4_MAX_TOPK || ld % 8 != 0 || (reinterpret_cast<uintptr_t>(logits) & 15u) != 0) return 0;
  if (n_experts <= 64 && ld >= 64) return 16;
  if (n_experts <= 96 && ld >= 96) return 24;
  return 0;
}

template <typename... Args>
static void launch_rf4(int epl, bool want_colsum, unsigned grid, cudaStream_t st, Args... args) {
  if (epl == 16) {
    if (want_colsum) launch_pdl(router_fused4_kernel<16, true>, dim3(grid), dim3(RF4_THREADS), 0, st, args...);
    else launch_pdl(router_fused4_kernel<16, false>, dim3(grid), dim3(RF4_THREADS), 0, st, args...);
  } else {
    if (want_colsum) launch_pdl(router_fused4_kernel<24, true>, dim3(grid), dim3(RF4_THREADS), 0, st, args...);
    else launch_pdl(router_fused4_kernel<24, false>, dim3(grid), dim3(RF4_THREADS), 0, st, args...);
  }
}

// d(logits) as bf16 [T, ld_out] (columns >= n_experts zero) from d(w_all) (first top_k columns of
// [T, top_k + n_shared], activation dtype) and the balance loss's gradient:
//   aux = aux_scale_T * sum_e counts[e] / sum(counts) * colsum[e]
//   => d colsum[e] = d_aux * aux_scale_T * counts[e] / (T * top_k), added to every d p[t, e].
template <int NSLOT>
__global__ void __launch_bounds__(RF_WARPS * 32)
    router_fused_bwd_kernel(const __nv_bfloat16* __restrict__ logits, int ld,
                            const float* __restrict__ bias, const float* __restrict__ noise, const int64_t* __restrict__ idx_all,
                            const __nv_bfloat16* __restrict__ dw_all, int64_t n_tokens,
                            int n_experts, int top_k, int n_shared, int normalize,
                            int full_softmax, const float* __restrict__ d_aux,
                            const int32_t* __restrict__ counts, float aux_scale_T,
                            __nv_bfloat16* __restrict__ dl, int ld_out) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kS = top_k + n_shared;
  const bool need_full = full_softmax || !normalize;

  float b[NSLOT], dcs[NSLOT];
  {
    const float g = (d_aux != nullptr && full_softmax) ? *d_aux : 0.f;
    // the loss weighs expert e by counts[e] / sum(counts): the sum is taken here rather than
    // assumed to be n_tokens * top_k, so that counts summed over several ranks (a global balance
    // loss) give the exact gradient too
    float c[NSLOT], tot = 0.f;
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      c[i] = (g != 0.f && e < n_experts) ? float(counts[e]) : 0.f;
      tot += c[i];
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const float denom_c = fmaxf(tot, 1.f);
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      b[i] = (bias != nullptr && e < n_experts) ? bias[e] : 0.f;
      dcs[i] = (e < n_experts && g != 0.f) ? g * aux_scale_T * c[i] / denom_c : 0.f;
    }
  }

  for (int64_t t = int64_t(blockIdx.x) * RF_WARPS + warp; t < n_tokens;
       t += int64_t(gridDim.x) * RF_WARPS) {
    const __nv_bfloat16* row = logits + t * ld;
    __nv_bfloat16* out = dl + t * ld_out;
    float v[NSLOT], dp[NSLOT];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      v[i] = e < n_experts ? __bfloat162float(row[e]) + b[i] +
                                 (noise != nullptr ? __ldg(noise + t * n_experts + e) : 0.f)
                           : -CUDART_INF_F;
      mx = fmaxf(mx, v[i]);
      dp[i] = dcs[i];
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));

    const bool active = lane < top_k;
    const int my_idx = active ? int(idx_all[t * kS + lane]) : -1;
    const float my_dw = active ? __bfloat162float(dw_all[t * kS + lane]) : 0.f;
    // my winner's logit, taken from the lane that holds it
    float my_l = -CUDART_INF_F;
    for (int j = 0; j < top_k; ++j) {
      const int e = __shfl_sync(0xffffffffu, my_idx, j);
      float val = 0.f;
#pragma unroll
      for (int i = 0; i < NSLOT; ++i)
        if (i == (e >> 5)) val = v[i];
      val = __shfl_sync(0xffffffffu, val, e & 31);
      if (lane == j) my_l = val;
    }

    float res[NSLOT];
    if (!need_full) {
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
      const float mine = w * (my_dw - dot);
#pragma unroll
      for (int i = 0; i < NSLOT; ++i) res[i] = 0.f;
      for (int j = 0; j < top_k; ++j) {
        const int e = __shfl_sync(0xffffffffu, my_idx, j);
        const float d = __shfl_sync(0xffffffffu, mine, j);
        if ((e & 31) == lane) {
#pragma unroll
          for (int i = 0; i < NSLOT; ++i)
            if (i == (e >> 5)) res[i] = d;
        }
      }
    } else {
      float pr[NSLOT];
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
      const float my_p = active ? expf(my_l - mx) / denom : 0.f;
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
      for (int j = 0; j < top_k; ++j) {
        const int e = __shfl_sync(0xffffffffu, my_idx, j);
        const float d = __shfl_sync(0xffffffffu, my_dp, j);
        if ((e & 31) == lane) {
#pragma unroll
          for (int i = 0; i < NSLOT; ++i)
            if (i == (e >> 5)) dp[i] += d;
        }
      }
      float inner = 0.f;
#pragma unroll
      for (int i = 0; i < NSLOT; ++i) inner += pr[i] * dp[i];
#pragma unroll
      for (int o = 16; o; o >>= 1) inner += __shfl_xor_sync(0xffffffffu, inner, o);
#pragma unroll
      for (int i = 0; i < NSLOT; ++i) res[i] = pr[i] * (dp[i] - inner);
    }
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      if (e < n_experts) out[e] = __float2bfloat16(res[i]);
    }
    for (int e = NSLOT * 32 + lane; e < ld_out; e += 32) out[e] = __float2bfloat16(0.f);
    // pad columns inside the NSLOT range
#pragma unroll
    for (int i = 0; i < NSLOT; ++i) {
      const int e = i * 32 + lane;
      if (e >= n_experts && e < ld_out) out[e] = __float2bfloat16(0.f);
    }
  }
}

// aux[0] = coef * E * sum_e (counts[e] / sum counts) * (colsum[e] / T)   (one warp)
__global__ void balance_loss_kernel(const float* __restrict__ colsum,
                                    const int32_t* __restrict__ counts, int n_experts,
                                    int64_t n_tokens, float coef, float* __restrict__ aux) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x;
  float dot = 0.f, tot = 0.f;
  for (int e = lane; e < n_experts; e += 32) {
    const float c = float(counts[e]);
    dot += c * colsum[e];
    tot += c;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    dot += __shfl_xor_sync(0xffffffffu, dot, o);
    tot += __shfl_xor_sync(0xffffffffu, tot, o);
  }
  if (lane == 0)
    aux[0] = coef * float(n_experts) * dot / fmaxf(tot, 1.f) / float(n_tokens > 0 ? n_tokens : 1);
}

static unsigned rf_grid(int64_t n_tokens, int blocks_per_sm = 16) {
  const int64_t want = (n_tokens + RF_WARPS - 1) / RF_WARPS;
  const int64_t cap = 148 * blocks_per_sm;  // resident blocks; warps stride over the tokens
  return unsigned(want < cap ? (want > 0 ? want : 1) : cap);
}

// 32 warps per block in chunked mode: a block owns 128+ consecutive tokens, a warp takes every 32nd.
constexpr int RF_CHUNK_WARPS = 32;

int launch_router_fused_chunked(const __nv_bfloat16* logits, int ld, const float* bias,
                                const float* noise, int64_t n_tokens, int n_experts, int top_k, int n_shared,
                                int normalize, int full_softmax, __nv_bfloat16* w_all,
                                int64_t* idx_all, float* colsum, int tokens_per_block, int n_blocks,
                                int32_t* block_hist, int32_t* sorted_ids, int64_t l_cap,
                                cudaStream_t st, const ScatterArgs* sc, bool* did_scatter) {
  if (did_scatter) *did_scatter = false;
  if (const int epl = rf4_experts_per_lane(logits, ld, n_experts, top_k)) {
    ScatterArgs fuse{};
    if (sc != nullptr && n_blocks == 1) {
      fuse = *sc;
      if (did_scatter) *did_scatter = true;
    }
    launch_rf4(epl, full_softmax && colsum != nullptr, unsigned(n_blocks), st, logits, ld, bias,
               noise, n_tokens, n_experts, top_k, n_shared, normalize, full_softmax, w_all, idx_all, colsum,
               tokens_per_block, block_hist, sorted_ids, l_cap, fuse);
    return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
  }
#define LAUNCH(NS)                                                                              \
  launch_pdl(router_fused_kernel<NS, RF_CHUNK_WARPS>, dim3(n_blocks), dim3(RF_CHUNK_WARPS * 32), 0, \
             st, logits, ld, bias, noise, n_tokens, n_experts, top_k, n_shared, normalize,          \
             full_softmax,                                                                          \
             w_all, idx_all, colsum, tokens_per_block, block_hist, sorted_ids, l_cap)
  const int nslot = (n_experts + 31) / 32;
  if (nslot <= 1) LAUNCH(1);
  else if (nslot <= 2) LAUNCH(2);
  else if (nslot <= 3) LAUNCH(3);
  else if (nslot <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // namespace moe

using namespace moe;

extern "C" {

int moe_b200_router_fused(const void* logits, int32_t ld, const float* bias, const float* noise,
                          int64_t n_tokens,
                          int32_t n_experts, int32_t top_k, int32_t n_shared, int32_t normalize,
                          int32_t full_softmax, void* w_all, int64_t* idx_all, float* colsum,
                          void* stream) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS || top_k < 1 || top_k > n_experts ||
      n_shared < 0 || top_k + n_shared > 32 || top_k > MAX_TOPK || n_tokens < 0 || ld < n_experts)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!logits || !w_all || !idx_all) return MOE_B200_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // every block ends with one atomic per expert on the same few addresses: with the balance-loss
  // statistics on, fewer blocks (each warp then takes a few tokens) keep that queue short
  const unsigned grid = rf_grid(n_tokens, (full_softmax && colsum) ? 4 : 16);
  const __nv_bfloat16* lg = static_cast<const __nv_bfloat16*>(logits);
  __nv_bfloat16* w = static_cast<__nv_bfloat16*>(w_all);
  if (const int epl = rf4_experts_per_lane(logits, ld, n_experts, top_k)) {
    int64_t blocks = (n_tokens + RF4_TOKENS - 1) / RF4_TOKENS;
    if (blocks > 148 * 2) blocks = 148 * 2;
    launch_rf4(epl, full_softmax && colsum != nullptr, unsigned(blocks), st, lg, ld, bias, noise,
               n_tokens,
               n_experts, top_k, n_shared, normalize, full_softmax, w, idx_all, colsum, 0,
               static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr), int64_t(0),
               ScatterArgs{});
    return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
  }
#define LAUNCH(NS)                                                                          \
  launch_pdl(router_fused_kernel<NS, RF_WARPS>, dim3(grid), dim3(RF_WARPS * 32), 0, st, lg, ld,    \
             bias, noise, n_tokens, n_experts, top_k, n_shared, normalize, full_softmax, w,        \
             idx_all,                                                                               \
             colsum, 0, static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr), int64_t(0))
  const int nslot = (n_experts + 31) / 32;
  if (nslot <= 1) LAUNCH(1);
  else if (nslot <= 2) LAUNCH(2);
  else if (nslot <= 3) LAUNCH(3);
  else if (nslot <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_router_fused_bwd(const void* logits, int32_t ld, const float* bias,
                              const float* noise, const int64_t* idx_all, const void* dw_all, int64_t n_tokens,
                              int32_t n_experts, int32_t top_k, int32_t n_shared,
                              int32_t normalize, int32_t full_softmax, const float* d_aux,
                              const int32_t* counts, float aux_coef, void* d_logits,
                              int32_t ld_out, void* stream) {
  if (n_experts < 1 || n_experts > MAX_EXPERTS || top_k < 1 || top_k > n_experts ||
      n_shared < 0 || top_k + n_shared > 32 || top_k > MAX_TOPK || n_tokens < 0 ||
      ld < n_experts || ld_out < n_experts)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!logits || !idx_all || !dw_all || !d_logits || (d_aux && !counts)) return MOE_B200_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = rf_grid(n_tokens);
  const float scale = aux_coef * float(n_experts) / float(n_tokens);
  const __nv_bfloat16* lg = static_cast<const __nv_bfloat16*>(logits);
  const __nv_bfloat16* dw = static_cast<const __nv_bfloat16*>(dw_all);
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(d_logits);
#define LAUNCH(NS)                                                                               \
  launch_pdl(router_fused_bwd_kernel<NS>, dim3(grid), dim3(RF_WARPS * 32), 0, st,                                     \
      lg, ld, bias, noise, idx_all, dw, n_tokens, n_experts, top_k, n_shared, normalize,          \
      full_softmax,                                                                                \
      d_aux, counts, scale, out, ld_out)
  const int nslot = (n_experts + 31) / 32;
  if (nslot <= 1) LAUNCH(1);
  else if (nslot <= 2) LAUNCH(2);
  else if (nslot <= 3) LAUNCH(3);
  else if (nslot <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_balance_loss(const float* colsum, const int32_t* counts, int32_t n_experts,
                          int64_t n_tokens, float aux_coef, float* aux, void* stream) {
  if (n_experts < 1 || n_tokens < 0) return MOE_B200_ERR_SHAPE;
  if (!colsum || !counts || !aux) return MOE_B200_ERR_NULL;
  launch_pdl(balance_loss_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), colsum,
             counts, n_experts, n_tokens, aux_coef, aux);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // extern "C"
