// HBM-bound data movement of the MoE block: the token permute (gather rows into expert-sorted,
// 128-aligned slot order) and the token-major combine (sum each token's top_k per-pair rows in
// fp32). Both move 16 bytes per thread with fully coalesced rows; the roofline for them is the
// HBM copy bandwidth.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"
#include "pdl.cuh"

namespace moe {

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// xs[slot, :] = x[sorted_ids[slot] / top_k, :] for live slots, zero rows for pad slots.
// row_bytes is a multiple of 16. One thread moves one 16-byte chunk.
__global__ void __launch_bounds__(256)
    permute_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                        const int32_t* __restrict__ n_post_pad, int32_t n_pairs, int32_t top_k,
                        int32_t chunks_per_row, uint4* __restrict__ xs) {
  pdl_trigger();
  pdl_wait();
  const int32_t live = __ldg(n_post_pad);
  const int64_t total = int64_t(live) * chunks_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int32_t slot = int32_t(i / chunks_per_row);
    const int32_t c = int32_t(i - int64_t(slot) * chunks_per_row);
    const int32_t pair = __ldg(sorted_ids + slot);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (pair < n_pairs) v = ld_stream(x + int64_t(pair / top_k) * chunks_per_row + c);
    xs[i] = v;
  }
}

struct alignas(32) Chunk32 {
  uint32_t w[8];
};
// 32-byte load that asks L2 to keep the line: every token row is read top_k times, far apart, while
// the rows being written stream through L2 in between.
__device__ __forceinline__ Chunk32 ld_keep32(const Chunk32* p) {
  Chunk32 r;
  asm volatile(
      "ld.global.nc.L1::no_allocate.L2::evict_last.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]),
        "=r"(r.w[6]), "=r"(r.w[7])
      : "l"(p));
  return r;
}
__device__ __forceinline__ void st32(Chunk32* p, const Chunk32& r) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.w[0]),
               "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3]), "r"(r.w[4]), "r"(r.w[5]), "r"(r.w[6]),
               "r"(r.w[7])
               : "memory");
}

// Same copy in 32-byte chunks (row_bytes a multiple of 32). A warp moves 8 consecutive slot rows as
// one flat run of 8 * chunks_per_row chunks, PERMUTE_UNROLL independent loads per lane in flight.
constexpr int PERMUTE_UNROLL = 3;
__global__ void __launch_bounds__(256)
    permute_rows32_kernel(const Chunk32* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                          const int32_t* __restrict__ n_post_pad, int32_t n_pairs, int32_t top_k,
                          int32_t chunks_per_row, Chunk32* __restrict__ xs) {
  pdl_trigger();
  pdl_wait();
  const int32_t live = __ldg(n_post_pad);  // a multiple of 128
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int per_group = 8 * chunks_per_row;
  for (int32_t row0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 8; row0 < live;
       row0 += warps * 8) {
    const int32_t pair = __ldg(sorted_ids + row0 + (lane & 7));
    const int32_t my_tok = pair < n_pairs ? pair / top_k : -1;  // token of row row0 + lane % 8
    Chunk32* dst = xs + int64_t(row0) * chunks_per_row;
    for (int base = 0; base < per_group; base += 32 * PERMUTE_UNROLL) {
      Chunk32 v[PERMUTE_UNROLL];
#pragma unroll
      for (int u = 0; u < PERMUTE_UNROLL; ++u) {
        const int f = base + u * 32 + lane;
        const int r = f / chunks_per_row;
        const int tok = __shfl_sync(0xffffffffu, my_tok, r & 7);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[u].w[q] = 0u;
        if (f < per_group && tok >= 0)
          v[u] = ld_keep32(x + int64_t(tok) * chunks_per_row + (f - r * chunks_per_row));
      }
#pragma unroll
      for (int u = 0; u < PERMUTE_UNROLL; ++u) {
        const int f = base + u * 32 + lane;
        if (f < per_group) st32(dst + f, v[u]);
      }
    }
  }
}

__device__ __forceinline__ void acc_bf16x8(float* acc, uint4 r) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    const float2 f = __bfloat1622float2(h);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// out[t, :] = sum_j y[inv_ids[t*top_k + j], :]  (+ extra[t, :])  in fp32, stored as bf16.
template <int TOPK>
__global__ void __launch_bounds__(256)
    combine_rows_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ inv_ids,
                        int64_t n_tokens, int32_t top_k_rt, int32_t chunks_per_row,
                        const uint4* __restrict__ extra, const uint4* __restrict__ extra2,
                        uint4* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int top_k = TOPK > 0 ? TOPK : top_k_rt;
  const int64_t total = n_tokens * chunks_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = i / chunks_per_row;
    const int32_t c = int32_t(i - t * chunks_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (TOPK > 0) {
      uint4 rows[TOPK > 0 ? TOPK : 1];
#pragma unroll
      for (int j = 0; j < TOPK; ++j) {
        const int32_t slot = __ldg(inv_ids + t * TOPK + j);   // < 0: the pair has no row (dropped)
        rows[j] = slot >= 0 ? ld_stream(y + int64_t(slot) * chunks_per_row + c)
                            : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < TOPK; ++j) acc_bf16x8(acc, rows[j]);
    } else {
      for (int j = 0; j < top_k; ++j) {
        const int32_t slot = __ldg(inv_ids + t * top_k + j);
        if (slot >= 0) acc_bf16x8(acc, ld_stream(y + int64_t(slot) * chunks_per_row + c));
      }
    }
    if (extra != nullptr) acc_bf16x8(acc, ld_stream(extra + i));
    if (extra2 != nullptr) acc_bf16x8(acc, ld_stream(extra2 + i));
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      w[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    out[i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// out[group of tile, c] += sum over the tile's 128 rows of w(row) * buf[row, c]. One block per
// (tile, 256-column chunk); thread = one 8-column piece of one of 8 row phases; the phases are
// folded through shared memory, then one fp32 atomic per column.
__global__ void __launch_bounds__(256)
    segment_colsum_kernel(const uint4* __restrict__ buf, int32_t pieces_per_row,
                          const int32_t* __restrict__ expert_ids,
                          const int32_t* __restrict__ n_post_pad,
                          const int32_t* __restrict__ pad_offsets,
                          const int32_t* __restrict__ sorted_ids,
                          const __nv_bfloat16* __restrict__ pair_w, int32_t n_pairs,
                          const uint4* __restrict__ alt, int64_t alt_rows, int32_t first_alt_group,
                          float* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x;
  if (int64_t(tile) * 128 >= __ldg(n_post_pad)) return;
  const int group = __ldg(expert_ids + tile);
  const int piece = blockIdx.y * 32 + (threadIdx.x & 31);   // 16-byte piece (8 columns) of the row
  const int phase = threadIdx.x >> 5;                        // rows phase, phase + 8, ...
  __shared__ float part[8][32][8];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const bool from_alt = alt != nullptr && group >= first_alt_group;
  const int64_t run0 = from_alt ? __ldg(pad_offsets + group) : 0;
  if (piece < pieces_per_row) {
    for (int r = phase; r < 128; r += 8) {
      const int64_t slot = int64_t(tile) * 128 + r;
      float w = 1.f;
      if (pair_w != nullptr) {
        const int32_t pr = __ldg(sorted_ids + slot);
        w = pr < n_pairs ? __bfloat162float(__ldg(pair_w + pr)) : 0.f;
      }
      uint4 v;
      if (from_alt) {
        const int64_t tr = slot - run0;
        if (tr >= alt_rows) continue;
        v = ld_stream(alt + tr * pieces_per_row + piece);
      } else {
        v = ld_stream(buf + slot * pieces_per_row + piece);
      }
      const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wd[i]));
        acc[2 * i] += w * f.x;
        acc[2 * i + 1] += w * f.y;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) part[phase][threadIdx.x & 31][i] = acc[i];
  __syncthreads();
  // thread t: column t of the block's 256
  const int c = threadIdx.x;
  const int col = blockIdx.y * 256 + c;
  if (col < pieces_per_row * 8) {
    float sum = 0.f;
#pragma unroll
    for (int ph = 0; ph < 8; ++ph) sum += part[ph][c >> 3][c & 7];
    atomicAdd(out + int64_t(group) * pieces_per_row * 8 + col, sum);
  }
}

// sumsq[g] += sum of squares of group g's elements (fp32; the caller zeroes it). x [groups, per_group]
// bf16, per_group a multiple of 8. One block-level reduction and one atomic per block.
__global__ void __launch_bounds__(256)
    group_sumsq_kernel(const uint4* __restrict__ x, int64_t pieces_per_group,
                       float* __restrict__ sumsq) {
  pdl_trigger();
  pdl_wait();
  const int g = blockIdx.y;
  const uint4* base = x + int64_t(g) * pieces_per_group;
  float acc = 0.f;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < pieces_per_group;
       i += int64_t(gridDim.x) * blockDim.x) {
    const uint4 v = ld_stream(base + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
      acc += f.x * f.x + f.y * f.y;
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += part[i];
    atomicAdd(sumsq + g, t);
  }
}

// out = alpha * s_g * x + beta * y, element-wise in fp32, one rounding to bf16. s_g = 1 / (sqrt(
// sumsq[g]) + eps) when sumsq is given (the Frobenius normalisation of group g), else 1; y may be null.
__global__ void __launch_bounds__(256)
    axpby_kernel(const uint4* __restrict__ x, const uint4* __restrict__ y, uint4* __restrict__ out,
                 int64_t pieces_per_group, int64_t total, float alpha, float beta,
                 const float* __restrict__ sumsq, float eps) {
  pdl_trigger();
  pdl_wait();
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    float a = alpha;
    if (sumsq != nullptr) a *= 1.f / (sqrtf(__ldg(sumsq + i / pieces_per_group)) + eps);
    const uint4 vx = ld_stream(x + i);
    uint4 vy = make_uint4(0u, 0u, 0u, 0u);
    if (y != nullptr) vy = ld_stream(y + i);
    const uint32_t wx[4] = {vx.x, vx.y, vx.z, vx.w}, wy[4] = {vy.x, vy.y, vy.z, vy.w};
    uint32_t wo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 fx = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wx[k]));
      const float2 fy = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wy[k]));
      const __nv_bfloat162 h = __floats2bfloat162_rn(a * fx.x + beta * fy.x, a * fx.y + beta * fy.y);
      wo[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    out[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
  }
}

// dst[r, c] = c < cols ? src[r, c] : 0 for c < dst_ld: pads a matrix's rows to a TMA-friendly
// stride (the router weight [D, E] -> [D, ld]) or drops the pad columns again.
__global__ void __launch_bounds__(256)
    copy_cols_kernel(const uint16_t* __restrict__ src, int64_t rows, int32_t cols, int32_t src_ld,
                     uint16_t* __restrict__ dst, int32_t dst_ld) {
  pdl_trigger();
  pdl_wait();
  const int64_t total = rows * dst_ld;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = i / dst_ld;
    const int32_t c = int32_t(i - r * dst_ld);
    dst[i] = c < cols ? src[r * src_ld + c] : uint16_t(0);
  }
}

}  // namespace moe

using namespace moe;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

extern "C" {

int moe_b200_permute(const void* x, int64_t n_tokens, int32_t d_model, int32_t top_k,
                     const int32_t* sorted_ids, const int32_t* n_post_pad, int64_t l_cap, void* xs,
                     void* stream) {
  if (d_model < 8 || d_model % 8 != 0 || top_k < 1 || n_tokens < 0 || l_cap < 0)
    return MOE_B200_ERR_SHAPE;
  if (l_cap == 0 || n_tokens == 0) return MOE_B200_OK;
  if (!x || !sorted_ids || !n_post_pad || !xs) return MOE_B200_ERR_NULL;
  if (!aligned16(x) || !aligned16(xs)) return MOE_B200_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (d_model % 16 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xs)) & 31u) == 0 &&
      l_cap % 8 == 0) {
    int64_t blocks = (l_cap / 8 + 7) / 8;  // 8 warps per block, 8 rows per warp and pass
    if (blocks > 148 * 8) blocks = 148 * 8;
    launch_pdl(permute_rows32_kernel, dim3(unsigned(blocks)), dim3(256), 0, st, 
        static_cast<const Chunk32*>(x), sorted_ids, n_post_pad, int32_t(n_tokens * top_k), top_k,
        d_model / 16, static_cast<Chunk32*>(xs));
    return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
  }
  const int32_t cpr = d_model / 8;
  const int64_t total = l_cap * cpr;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;  // grid-stride; a multiple of the SM count
  launch_pdl(permute_rows_kernel, dim3(unsigned(blocks)), dim3(256), 0, st, 
      static_cast<const uint4*>(x), sorted_ids, n_post_pad, int32_t(n_tokens * top_k), top_k, cpr,
      static_cast<uint4*>(xs));
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_combine(const void* y, const int32_t* inv_ids, int64_t n_tokens, int32_t top_k,
                     int32_t d_model, const void* extra, const void* extra2, void* out,
                     void* stream) {
  if (d_model < 8 || d_model % 8 != 0 || top_k < 1 || n_tokens < 0) return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!y || !inv_ids || !out) return MOE_B200_ERR_NULL;
  if (!aligned16(y) || !aligned16(out) || !aligned16(extra) || !aligned16(extra2))
    return MOE_B200_ERR_ALIGN;
  const int32_t cpr = d_model / 8;
  const int64_t total = n_tokens * cpr;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint4* yy = static_cast<const uint4*>(y);
  const uint4* ex = static_cast<const uint4*>(extra);
  const uint4* ex2 = static_cast<const uint4*>(extra2);
  uint4* oo = static_cast<uint4*>(out);
#define LAUNCH(K) \
  launch_pdl(combine_rows_kernel<K>, dim3(unsigned(blocks)), dim3(256), 0, st, yy, inv_ids, n_tokens, top_k, cpr, ex, ex2, oo)
  switch (top_k) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    case 6: LAUNCH(6); break;
    case 8: LAUNCH(8); break;
    default: LAUNCH(0); break;
  }
#undef LAUNCH
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_segment_colsum(const void* buf, int64_t rows, int32_t width,
                            const int32_t* expert_ids, const int32_t* n_post_pad,
                            const int32_t* pad_offsets, int32_t n_groups,
                            const int32_t* sorted_ids, const void* pair_w, int64_t n_pairs,
                            const void* alt, int64_t alt_rows, int32_t first_alt_group,
                            float* out, void* stream) {
  if (rows < 0 || rows % 128 != 0 || width < 8 || width % 8 != 0 || n_groups < 1 || n_pairs < 0 ||
      n_pairs > (int64_t(1) << 30))
    return MOE_B200_ERR_SHAPE;
  if (rows == 0) return MOE_B200_OK;
  if (!buf || !expert_ids || !n_post_pad || !out) return MOE_B200_ERR_NULL;
  if (pair_w && !sorted_ids) return MOE_B200_ERR_NULL;
  if (alt && (!pad_offsets || alt_rows < 1 || first_alt_group < 0)) return MOE_B200_ERR_SHAPE;
  if (!aligned16(buf) || !aligned16(alt)) return MOE_B200_ERR_ALIGN;
  const int32_t ppr = width / 8;
  launch_pdl(segment_colsum_kernel, dim3(unsigned(rows / 128), unsigned((ppr + 31) / 32)),
             dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(buf), ppr,
             expert_ids, n_post_pad, pad_offsets, sorted_ids,
             static_cast<const __nv_bfloat16*>(pair_w), int32_t(n_pairs),
             static_cast<const uint4*>(alt), alt_rows, first_alt_group, out);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_group_sumsq(const void* x, int32_t groups, int64_t per_group, float* sumsq,
                         void* stream) {
  if (groups < 1 || groups > 65535 || per_group < 8 || per_group % 8 != 0) return MOE_B200_ERR_SHAPE;
  if (!x || !sumsq) return MOE_B200_ERR_NULL;
  if (!aligned16(x)) return MOE_B200_ERR_ALIGN;
  const int64_t ppg = per_group / 8;
  int64_t bx = (ppg + 255) / 256;
  const int64_t cap = (148 * 8 + groups - 1) / groups;
  if (bx > cap) bx = cap;
  launch_pdl(group_sumsq_kernel, dim3(unsigned(bx), unsigned(groups)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const uint4*>(x), ppg, sumsq);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_axpby(const void* x, const void* y, void* out, int32_t groups, int64_t per_group,
                   float alpha, float beta, const float* sumsq, float eps, void* stream) {
  if (groups < 1 || per_group < 8 || per_group % 8 != 0) return MOE_B200_ERR_SHAPE;
  if (!x || !out) return MOE_B200_ERR_NULL;
  if (!aligned16(x) || !aligned16(y) || !aligned16(out)) return MOE_B200_ERR_ALIGN;
  const int64_t ppg = per_group / 8, total = ppg * groups;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  launch_pdl(axpby_kernel, dim3(unsigned(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const uint4*>(x), static_cast<const uint4*>(y), static_cast<uint4*>(out),
             ppg, total, alpha, beta, sumsq, eps);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_copy_cols(const void* src, int64_t rows, int32_t cols, int32_t src_ld, void* dst,
                       int32_t dst_ld, void* stream) {
  if (rows < 0 || cols < 0 || src_ld < cols || dst_ld < 1) return MOE_B200_ERR_SHAPE;
  if (rows == 0) return MOE_B200_OK;
  if (!src || !dst) return MOE_B200_ERR_NULL;
  const int64_t total = rows * dst_ld;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  launch_pdl(copy_cols_kernel, dim3(unsigned(blocks)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(src), rows, cols,
             src_ld, static_cast<uint16_t*>(dst), dst_ld);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // extern "C"
