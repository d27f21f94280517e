// Expert parallelism over peer memory: the routed experts are partitioned over the GPUs of one node
// and the token rows travel by plain loads and stores through peer pointers (NVLink), fused with
// the movement kernels the single-GPU block already runs:
//
//   home rank     ep_plan + ep_pair_map : where every (token, expert) pair lives in its owner's
//                                         slot-ordered buffer, from the all-gathered count matrix
//                 ep_push_rows          : the token permute, writing each row straight into the
//                                         owner's buffer (no send buffer, no receive-side permute)
//   owner rank    ep_pad_fix            : zero rows / sentinel ids in the pad slots of its runs
//                 (grouped GEMMs of the block on its own slot-ordered buffer)
//   home rank     ep_pull_combine       : the token-major combine, reading each pair's row from
//                                         its owner's output buffer
//                 ep_pull_vec           : the same gather for one bf16 value per pair (d topk_w)
//
// Nothing here waits on another GPU: the caller orders the phases (a collective between them).
// Every pointer in a PeerTable is a device pointer valid in this process (a peer mapping of the
// other rank's buffer, or the rank's own buffer). Only plain ld / st touch peer memory: no TMA,
// no multicast.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"
#include "pdl.cuh"
#include "routing.cuh"

namespace moe {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_ALIGN = 128;   // rows per tile of the grouped GEMMs

struct PeerTable {
  void* p[EP_MAX_RANKS + 1];    // [rank] = that rank's buffer; [n_ranks] = a local extra buffer
};

// One block. cnt_all [n_ranks, n_experts]: pairs of every home rank per routed expert.
// bounds [n_ranks + 1]: rank r owns experts [bounds[r], bounds[r + 1]).
// Out, for the calling rank as a sender: owner_of [E], send_row0 [E] (first row, in the owner's
// buffer, of this rank's pairs of expert e: the owner's runs are 128-aligned and hold the home
// ranks' pairs in rank order). As an owner: own_offs [E_r + 1], own_counts [E_r], own_npp [1],
// own_eids [cap_tiles] (tile -> local expert, 0 past the live length).
__global__ void __launch_bounds__(256)
    ep_plan_kernel(const int32_t* __restrict__ cnt_all, const int32_t* __restrict__ bounds,
                   int n_ranks, int n_experts, int rank, int32_t* __restrict__ owner_of,
                   int32_t* __restrict__ send_row0, int32_t* __restrict__ own_offs,
                   int32_t* __restrict__ own_counts, int32_t* __restrict__ own_npp,
                   int32_t* __restrict__ own_eids, int64_t cap_tiles) {
  pdl_trigger();
  pdl_wait();
  __shared__ int32_t tot[MAX_EXPERTS], before[MAX_EXPERTS], owner[MAX_EXPERTS];
  __shared__ int32_t start[MAX_EXPERTS + 1];   // padded run start inside the owner's buffer
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int32_t t = 0, b = 0;
    for (int r = 0; r < n_ranks; ++r) {
      const int32_t c = cnt_all[r * n_experts + e];
      t += c;
      if (r < rank) b += c;
    }
    int o = 0;
    while (o + 1 < n_ranks && e >= bounds[o + 1]) ++o;
    tot[e] = t;
    before[e] = b;
    owner[e] = o;
  }
  __syncthreads();
  if (threadIdx.x == 0) {   // E <= 256: a serial scan, restarted at every owner's first expert
    int32_t run = 0;
    for (int e = 0; e < n_experts; ++e) {
      if (e == bounds[owner[e]]) run = 0;
      start[e] = run;
      run += (tot[e] + EP_ALIGN - 1) / EP_ALIGN * EP_ALIGN;
      if (e + 1 == bounds[owner[e] + 1] && owner[e] == rank) start[MAX_EXPERTS] = run;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    owner_of[e] = owner[e];
    send_row0[e] = start[e] + before[e];
  }
  const int lo = bounds[rank], hi = bounds[rank + 1];
  const int32_t live = hi > lo ? start[MAX_EXPERTS] : 0;
  for (int e = lo + threadIdx.x; e < hi; e += blockDim.x) {
    own_offs[e - lo] = start[e];
    own_counts[e - lo] = tot[e];
  }
  if (threadIdx.x == 0) {
    own_offs[hi - lo] = live;
    *own_npp = live;
  }
  for (int64_t tile = threadIdx.x; tile < cap_tiles; tile += blockDim.x) {
    int32_t who = 0;
    const int64_t row = tile * EP_ALIGN;
    if (row < live) {
      int a = lo, b = hi;   // start[a] <= row < end of b - 1
      while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (start[mid] <= row) a = mid; else b = mid;
      }
      who = a - lo;
    }
    own_eids[tile] = who;
  }
}

// pair p = t * k_all + j of the home rank -> (rank, row) of its row in an owner's buffer; the
// shared experts' pairs (expert id >= n_experts) point at the local extra buffer, laid out
// [n_shared, n_tokens, .]: rank n_ranks, row s * n_tokens + t.
__global__ void __launch_bounds__(256)
    ep_pair_map_kernel(const int64_t* __restrict__ idx_all, const int32_t* __restrict__ inv_ids,
                       const int32_t* __restrict__ local_offs, const int32_t* __restrict__ owner_of,
                       const int32_t* __restrict__ send_row0, int64_t n_pairs, int k_all,
                       int n_experts, int n_ranks, int64_t n_tokens, int32_t* __restrict__ pair_rank,
                       int32_t* __restrict__ pair_row) {
  pdl_trigger();
  pdl_wait();
  for (int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < n_pairs;
       p += int64_t(gridDim.x) * blockDim.x) {
    const int e = int(idx_all[p]);
    if (e < n_experts) {
      pair_rank[p] = owner_of[e];
      pair_row[p] = send_row0[e] + (inv_ids[p] - local_offs[e]);
    } else {
      pair_rank[p] = n_ranks;
      pair_row[p] = int32_t((e - n_experts) * n_tokens + p / k_all);
    }
  }
}

struct alignas(16) Chunk16 {
  uint32_t w[4];
};

// The permute with remote destinations: slot s of the home rank's plan (pair sorted_ids[s]) ->
// row pair_row[pair] of rows.p[pair_rank[pair]]. One warp per slot row, 16-byte chunks. With sid /
// pw tables it also leaves, per destination row, the row's own index (the owner's sorted_ids:
// identity) and the pair's router weight. Pad slots and the shared experts' slots are skipped
// (n_live_slots points at the start of the first shared run). The walk over the slots starts at
// *first_slot and wraps around: slots are in expert order, i.e. grouped by owner, so ranks that all
// started at slot 0 would all write to rank 0 at the same time, then all to rank 1, ... and share
// one GPU's NVLink ingress; rank r starts at its first pair for rank r + 1 instead (measured on 8
// GPUs: 1.2-1.9 ms per push without the rotation).
__global__ void __launch_bounds__(256)
    ep_push_rows_kernel(const Chunk16* __restrict__ src, const int32_t* __restrict__ sorted_ids,
                        const int32_t* __restrict__ n_live_slots,
                        const int32_t* __restrict__ first_slot, int64_t n_pairs, int k_all,
                        const int32_t* __restrict__ pair_rank, const int32_t* __restrict__ pair_row,
                        PeerTable rows, PeerTable sid, PeerTable pw,
                        const __nv_bfloat16* __restrict__ w_all, int chunks_per_row) {
  pdl_trigger();
  pdl_wait();
  const int live = __ldg(n_live_slots);
  int rot = first_slot != nullptr ? __ldg(first_slot) : 0;
  if (rot < 0 || rot >= live) rot = 0;
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  for (int s0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s0 < live; s0 += warps) {
    const int s = s0 + rot < live ? s0 + rot : s0 + rot - live;
    const int pair = __ldg(sorted_ids + s);
    if (pair >= n_pairs) continue;
    const int r = __ldg(pair_rank + pair);
    const int64_t row = __ldg(pair_row + pair);
    const Chunk16* from = src + int64_t(pair / k_all) * chunks_per_row;
    Chunk16* to = static_cast<Chunk16*>(rows.p[r]) + row * chunks_per_row;
    // a lane's loads of the row are all issued before its first (remote) store: written as one
    // load-store pair per iteration they ran one after the other, each behind the store before it
    // (push x 0.47 -> 0.45 ms on two GPUs; 32-byte pieces on top of that changed nothing)
    constexpr int INFLIGHT = 4;
    for (int c0 = lane; c0 < chunks_per_row; c0 += 32 * INFLIGHT) {
      Chunk16 v[INFLIGHT];
#pragma unroll
      for (int u = 0; u < INFLIGHT; ++u)
        if (c0 + 32 * u < chunks_per_row) v[u] = from[c0 + 32 * u];
#pragma unroll
      for (int u = 0; u < INFLIGHT; ++u)
        if (c0 + 32 * u < chunks_per_row) to[c0 + 32 * u] = v[u];
    }
    if (lane == 0 && sid.p[r] != nullptr) static_cast<int32_t*>(sid.p[r])[row] = int32_t(row);
    if (lane == 1 && pw.p[r] != nullptr) static_cast<__nv_bfloat16*>(pw.p[r])[row] = w_all[pair];
  }
  // no fence here: the rows are read by other GPUs only after this kernel has completed and a
  // stream-ordered collective has passed, which makes its stores visible system-wide
}

// Owner side: the pad slots of every local run -- rows [offs[e] + counts[e], offs[e + 1]) -- get
// zero rows (the GEMMs rely on them) and, when sid is given, the sentinel id.
__global__ void __launch_bounds__(256)
    ep_pad_fix_kernel(const int32_t* __restrict__ own_offs, const int32_t* __restrict__ own_counts,
                      int n_local, Chunk16* __restrict__ rows, int chunks_per_row,
                      int32_t* __restrict__ sid, int32_t sentinel) {
  pdl_trigger();
  pdl_wait();
  for (int e = blockIdx.x; e < n_local; e += gridDim.x) {
    const int64_t lo = int64_t(own_offs[e]) + own_counts[e], hi = own_offs[e + 1];
    const int64_t n = (hi - lo) * chunks_per_row;
    Chunk16 z;
    z.w[0] = z.w[1] = z.w[2] = z.w[3] = 0u;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) rows[lo * chunks_per_row + i] = z;
    if (sid != nullptr)
      for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) sid[i] = sentinel;
  }
}

__device__ __forceinline__ void ep_acc8(float* acc, const Chunk16& r) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.w[i]));
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// out[t, :] = sum_j y.p[pair_rank[p]][pair_row[p], :]  (+ extra[t, :])  in fp32 (pair order j, as the
// single-GPU combine), stored as bf16. One thread per 16-byte chunk of a token row.
__global__ void __launch_bounds__(256)
    ep_pull_combine_kernel(PeerTable y, const int32_t* __restrict__ pair_rank,
                           const int32_t* __restrict__ pair_row, int64_t n_tokens, int k_all,
                           int chunks_per_row, const Chunk16* __restrict__ extra,
                           Chunk16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int64_t total = n_tokens * chunks_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = i / chunks_per_row;
    const int c = int(i - t * chunks_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    constexpr int INFLIGHT = 8;   // rows in flight per thread (a remote load takes microseconds)
    for (int j0 = 0; j0 < k_all; j0 += INFLIGHT) {
      Chunk16 v[INFLIGHT];
#pragma unroll
      for (int u = 0; u < INFLIGHT; ++u) {
        v[u].w[0] = v[u].w[1] = v[u].w[2] = v[u].w[3] = 0u;
        if (j0 + u < k_all) {
          const int64_t p = t * k_all + j0 + u;
          v[u] = static_cast<const Chunk16*>(y.p[pair_rank[p]])[int64_t(pair_row[p]) * chunks_per_row + c];
        }
      }
#pragma unroll
      for (int u = 0; u < INFLIGHT; ++u)
        if (j0 + u < k_all) ep_acc8(acc, v[u]);
    }
    if (extra != nullptr) ep_acc8(acc, extra[i]);
    Chunk16 o;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o.w[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    out[i] = o;
  }
}

// out[p] = v.p[pair_rank[p]][pair_row[p]] for the routed pairs (columns j < top_k), 0 for the rest.
__global__ void __launch_bounds__(256)
    ep_pull_vec_kernel(PeerTable v, const int32_t* __restrict__ pair_rank,
                       const int32_t* __restrict__ pair_row, int64_t n_pairs, int k_all, int top_k,
                       __nv_bfloat16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  for (int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < n_pairs;
       p += int64_t(gridDim.x) * blockDim.x) {
    const bool routed = int(p % k_all) < top_k;
    out[p] = routed ? static_cast<const __nv_bfloat16*>(v.p[pair_rank[p]])[pair_row[p]]
                    : __float2bfloat16(0.f);
  }
}

}  // namespace moe

using namespace moe;

static bool peer_table(PeerTable* t, const void* const* ptrs, int n) {
  for (int i = 0; i <= EP_MAX_RANKS; ++i) t->p[i] = nullptr;
  if (!ptrs) return true;
  if (n < 0 || n > EP_MAX_RANKS + 1) return false;
  for (int i = 0; i < n; ++i) {
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15u) return false;
    t->p[i] = const_cast<void*>(ptrs[i]);
  }
  return true;
}
static unsigned ep_grid(int64_t work_items, int per_block) {
  int64_t b = (work_items + per_block - 1) / per_block;
  const int64_t cap = 148 * 8;
  return unsigned(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" {

int moe_b200_ep_plan(const int32_t* cnt_all, const int32_t* bounds, int32_t n_ranks,
                     int32_t n_experts, int32_t rank, int32_t* owner_of, int32_t* send_row0,
                     int32_t* own_offs, int32_t* own_counts, int32_t* own_npp, int32_t* own_eids,
                     int64_t cap_tiles, void* stream) {
  if (n_ranks < 1 || n_ranks > EP_MAX_RANKS || n_experts < n_ranks || n_experts > MAX_EXPERTS ||
      rank < 0 || rank >= n_ranks || cap_tiles < 0)
    return MOE_B200_ERR_SHAPE;
  if (!cnt_all || !bounds || !owner_of || !send_row0 || !own_offs || !own_counts || !own_npp ||
      !own_eids)
    return MOE_B200_ERR_NULL;
  launch_pdl(ep_plan_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), cnt_all,
             bounds, int(n_ranks), int(n_experts), int(rank), owner_of, send_row0, own_offs,
             own_counts, own_npp, own_eids, cap_tiles);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_ep_pair_map(const int64_t* idx_all, const int32_t* inv_ids, const int32_t* local_offs,
                         const int32_t* owner_of, const int32_t* send_row0, int64_t n_tokens,
                         int32_t k_all, int32_t n_experts, int32_t n_ranks, int32_t* pair_rank,
                         int32_t* pair_row, void* stream) {
  if (n_tokens < 0 || k_all < 1 || n_experts < 1 || n_ranks < 1 || n_ranks > EP_MAX_RANKS ||
      n_tokens * k_all > (int64_t(1) << 30))
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!idx_all || !inv_ids || !local_offs || !owner_of || !send_row0 || !pair_rank || !pair_row)
    return MOE_B200_ERR_NULL;
  const int64_t n_pairs = n_tokens * k_all;
  launch_pdl(ep_pair_map_kernel, dim3(ep_grid(n_pairs, 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), idx_all, inv_ids, local_offs, owner_of, send_row0,
             n_pairs, int(k_all), int(n_experts), int(n_ranks), n_tokens, pair_rank, pair_row);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_ep_push_rows(const void* src, int64_t n_tokens, int32_t d_model, int32_t k_all,
                          const int32_t* sorted_ids, const int32_t* n_live_slots,
                          const int32_t* first_slot, int64_t max_slots, const int32_t* pair_rank,
                          const int32_t* pair_row, const void* const* dst_rows,
                          const void* const* dst_sid, const void* const* dst_w, int32_t n_ranks,
                          const void* w_all, void* stream) {
  if (n_tokens < 0 || d_model < 8 || d_model % 8 != 0 || k_all < 1 || n_ranks < 1 ||
      n_ranks > EP_MAX_RANKS || max_slots < 0)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0 || max_slots == 0) return MOE_B200_OK;
  if (!src || !sorted_ids || !n_live_slots || !pair_rank || !pair_row || !dst_rows ||
      (dst_w && !w_all))
    return MOE_B200_ERR_NULL;
  PeerTable rows, sid, pw;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) || !peer_table(&rows, dst_rows, n_ranks) ||
      !peer_table(&sid, dst_sid, n_ranks) || !peer_table(&pw, dst_w, n_ranks))
    return MOE_B200_ERR_ALIGN;
  launch_pdl(ep_push_rows_kernel, dim3(ep_grid(max_slots, 8)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), static_cast<const Chunk16*>(src), sorted_ids,
             n_live_slots, first_slot, n_tokens * k_all, int(k_all), pair_rank, pair_row, rows, sid,
             pw,
             static_cast<const __nv_bfloat16*>(w_all), int(d_model / 8));
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_ep_pad_fix(const int32_t* own_offs, const int32_t* own_counts, int32_t n_local,
                        void* rows, int32_t d_model, int32_t* sid, int32_t sentinel, void* stream) {
  if (n_local < 0 || d_model < 8 || d_model % 8 != 0) return MOE_B200_ERR_SHAPE;
  if (n_local == 0) return MOE_B200_OK;
  if (!own_offs || !own_counts || !rows) return MOE_B200_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(rows) & 15u) return MOE_B200_ERR_ALIGN;
  launch_pdl(ep_pad_fix_kernel, dim3(unsigned(n_local)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), own_offs, own_counts, int(n_local),
             static_cast<Chunk16*>(rows), int(d_model / 8), sid, sentinel);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_ep_pull_combine(const void* const* y, int32_t n_tables, const int32_t* pair_rank,
                             const int32_t* pair_row, int64_t n_tokens, int32_t k_all,
                             int32_t d_model, const void* extra, void* out, void* stream) {
  if (n_tokens < 0 || d_model < 8 || d_model % 8 != 0 || k_all < 1 || n_tables < 1 ||
      n_tables > EP_MAX_RANKS + 1)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!y || !pair_rank || !pair_row || !out) return MOE_B200_ERR_NULL;
  PeerTable t;
  if (!peer_table(&t, y, n_tables) || (reinterpret_cast<uintptr_t>(out) & 15u) ||
      (reinterpret_cast<uintptr_t>(extra) & 15u))
    return MOE_B200_ERR_ALIGN;
  launch_pdl(ep_pull_combine_kernel, dim3(ep_grid(n_tokens * (d_model / 8), 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), t, pair_rank, pair_row, n_tokens, int(k_all),
             int(d_model / 8), static_cast<const Chunk16*>(extra), static_cast<Chunk16*>(out));
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

int moe_b200_ep_pull_vec(const void* const* v, int32_t n_ranks, const int32_t* pair_rank,
                         const int32_t* pair_row, int64_t n_tokens, int32_t k_all, int32_t top_k,
                         void* out, void* stream) {
  if (n_tokens < 0 || k_all < 1 || top_k < 1 || top_k > k_all || n_ranks < 1 ||
      n_ranks > EP_MAX_RANKS)
    return MOE_B200_ERR_SHAPE;
  if (n_tokens == 0) return MOE_B200_OK;
  if (!v || !pair_rank || !pair_row || !out) return MOE_B200_ERR_NULL;
  PeerTable t;
  if (!peer_table(&t, v, n_ranks)) return MOE_B200_ERR_ALIGN;
  launch_pdl(ep_pull_vec_kernel, dim3(ep_grid(n_tokens * k_all, 256)), dim3(256), 0,
             static_cast<cudaStream_t>(stream), t, pair_rank, pair_row, n_tokens * k_all,
             int(k_all), int(top_k), static_cast<__nv_bfloat16*>(out));
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // extern "C"
