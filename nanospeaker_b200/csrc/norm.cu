// RMSNorm in front of the MoE block and its backward fused with the residual branch's gradient:
// the sublayer is  out = x + ffn(rmsnorm(x) * gamma)  (src/model/nanospeaker.py:165-169 with
// src/model/ln.py:31-38). One warp per token row, 16-byte chunks, fp32 arithmetic; both kernels
// are plain HBM streams (read x once / read dh, x and the residual gradient once).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"
#include "pdl.cuh"

namespace moe {

constexpr int NORM_WARPS = 8;
constexpr int NORM_MAX_CHUNKS = 8;  // 16-byte chunks per lane: rows up to 32 * 8 * 8 = 2048 columns
// The kernels are instantiated for 1, 2, 3, 4 or 8 chunks per lane: the per-lane row state lives in
// registers, and sizing it for the widest row would leave one resident block per SM.

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// h[t, :] = x[t, :] * rstd[t] * gamma,  rstd[t] = rsqrt(mean(x[t, :]^2) + eps)  (kept for the backward)
template <int NCH>
__global__ void __launch_bounds__(NORM_WARPS * 32)
    rmsnorm_fwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gamma,
                       int64_t n_rows, int32_t chunks_per_row, float eps, float inv_d,
                       uint4* __restrict__ h, float* __restrict__ rstd) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t warps = int64_t(gridDim.x) * NORM_WARPS;
  for (int64_t t = int64_t(blockIdx.x) * NORM_WARPS + (threadIdx.x >> 5); t < n_rows; t += warps) {
    uint4 v[NCH];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = i * 32 + lane;
      if (c < chunks_per_row) {
        v[i] = x[t * chunks_per_row + c];
        float f[8];
        unpack8(v[i], f);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += f[k] * f[k];
      }
    }
    const float r = rsqrtf(warp_sum(ss) * inv_d + eps);
    if (lane == 0) rstd[t] = r;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = i * 32 + lane;
      if (c < chunks_per_row) {
        float f[8], g[8];
        unpack8(v[i], f);
        unpack8(gamma[c], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = f[k] * r * g[k];
        h[t * chunks_per_row + c] = pack8(f);
      }
    }
  }
}

// dx[t] = rstd * (gamma * dh) - x * rstd^3 / D * <gamma * dh, x>  (+ add[t], the residual branch)
// dgamma += sum_t dh[t] * x[t] * rstd[t]   (fp32; per-block partial sums in shared memory, then
// one atomic per block and column)
template <int NCH>
__global__ void __launch_bounds__(NORM_WARPS * 32)
    rmsnorm_bwd_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ x,
                       const float* __restrict__ rstd, const uint4* __restrict__ gamma,
                       const uint4* __restrict__ add, int64_t n_rows, int32_t chunks_per_row,
                       float inv_d, uint4* __restrict__ dx, float* __restrict__ dgamma) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float dg_s[];  // [chunks_per_row * 8]
  const int lane = threadIdx.x & 31;
  const int n_cols = chunks_per_row * 8;
  for (int i = threadIdx.x; i < n_cols; i += blockDim.x) dg_s[i] = 0.f;
  __syncthreads();
  float dg[NCH][8];
#pragma unroll
  for (int i = 0; i < NCH; ++i)
#pragma unroll
    for (int k = 0; k < 8; ++k) dg[i][k] = 0.f;

  const int64_t warps = int64_t(gridDim.x) * NORM_WARPS;
  for (int64_t t = int64_t(blockIdx.x) * NORM_WARPS + (threadIdx.x >> 5); t < n_rows; t += warps) {
    uint4 vd[NCH], vx[NCH];
    const float r = rstd[t];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = i * 32 + lane;
      if (c < chunks_per_row) {
        vd[i] = dh[t * chunks_per_row + c];
        vx[i] = x[t * chunks_per_row + c];
        float d[8], xx[8], g[8];
        unpack8(vd[i], d);
        unpack8(vx[i], xx);
        unpack8(gamma[c], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          dot += g[k] * d[k] * xx[k];
          dg[i][k] += d[k] * xx[k] * r;
        }
      }
    }
    const float coef = warp_sum(dot) * r * r * r * inv_d;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
      const int c = i * 32 + lane;
      if (c < chunks_per_row) {
        float d[8], xx[8], g[8], o[8];
        unpack8(vd[i], d);
        unpack8(vx[i], xx);
        unpack8(gamma[c], g);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = r * g[k] * d[k] - xx[k] * coef;
        if (add != nullptr) {
          float a[8];
          unpack8(add[t * chunks_per_row + c], a);
#pragma unroll
          for (int k = 0; k < 8; ++k) o[k] += a[k];
        }
        dx[t * chunks_per_row + c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NCH; ++i) {
    const int c = i * 32 + lane;
    if (c < chunks_per_row) {
#pragma unroll
      for (int k = 0; k < 8; ++k) atomicAdd(&dg_s[c * 8 + k], dg[i][k]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_cols; i += blockDim.x) atomicAdd(dgamma + i, dg_s[i]);
}

static unsigned norm_grid(int64_t n_rows, int blocks_per_sm) {
  const int64_t want = (n_rows + NORM_WARPS - 1) / NORM_WARPS;
  const int64_t cap = int64_t(148) * blocks_per_sm;
  return unsigned(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace moe

using namespace moe;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" {

int moe_b200_rmsnorm(const void* x, const void* gamma, int64_t n_rows, int32_t d_model, float eps,
                     void* h, float* rstd, void* stream) {
  if (n_rows < 0 || d_model < 8 || d_model % 8 != 0 || d_model > 32 * NORM_MAX_CHUNKS * 8)
    return MOE_B200_ERR_SHAPE;
  if (n_rows == 0) return MOE_B200_OK;
  if (!x || !gamma || !h || !rstd) return MOE_B200_ERR_NULL;
  if (!aligned16(x) || !aligned16(gamma) || !aligned16(h)) return MOE_B200_ERR_ALIGN;
  const int nch = (d_model / 8 + 31) / 32;
#define LAUNCH(N)                                                                              \
  launch_pdl(rmsnorm_fwd_kernel<N>, dim3(norm_grid(n_rows, 8)), dim3(NORM_WARPS * 32), 0,         \
             static_cast<cudaStream_t>(stream), static_cast<const uint4*>(x),                     \
             static_cast<const uint4*>(gamma), n_rows, d_model / 8, eps, 1.f / float(d_model),    \
             static_cast<uint4*>(h), rstd)
  if (nch <= 1) LAUNCH(1);
  else if (nch <= 2) LAUNCH(2);
  else if (nch <= 3) LAUNCH(3);
  else if (nch <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_rmsnorm_bwd(const void* dh, const void* x, const float* rstd, const void* gamma,
                         const void* add, int64_t n_rows, int32_t d_model, void* dx,
                         float* dgamma, void* stream) {
  if (n_rows < 0 || d_model < 8 || d_model % 8 != 0 || d_model > 32 * NORM_MAX_CHUNKS * 8)
    return MOE_B200_ERR_SHAPE;
  if (n_rows == 0) return MOE_B200_OK;
  if (!dh || !x || !rstd || !gamma || !dx || !dgamma) return MOE_B200_ERR_NULL;
  if (!aligned16(dh) || !aligned16(x) || !aligned16(gamma) || !aligned16(add) || !aligned16(dx))
    return MOE_B200_ERR_ALIGN;
  // few blocks: every block ends with one atomic per column on dgamma
  const int nch = (d_model / 8 + 31) / 32;
#define LAUNCH(N)                                                                              \
  launch_pdl(rmsnorm_bwd_kernel<N>, dim3(norm_grid(n_rows, 3)), dim3(NORM_WARPS * 32),            \
             size_t(d_model) * sizeof(float), static_cast<cudaStream_t>(stream),                  \
             static_cast<const uint4*>(dh), static_cast<const uint4*>(x), rstd,                   \
             static_cast<const uint4*>(gamma), static_cast<const uint4*>(add), n_rows,            \
             d_model / 8, 1.f / float(d_model), static_cast<uint4*>(dx), dgamma)
  if (nch <= 1) LAUNCH(1);
  else if (nch <= 2) LAUNCH(2);
  else if (nch <= 3) LAUNCH(3);
  else if (nch <= 4) LAUNCH(4);
  else LAUNCH(8);
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // extern "C"
