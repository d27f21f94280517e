// Second pass of the dispatch (plan + stable scatter) as a device function, so that the stand-alone
// kernel (routing.cu) and a router kernel that owns the whole input as ONE block (router_fused.cu:
// small batches, where a second launch costs more than the work) run the same code.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "routing.cuh"

namespace moe {

constexpr int DISPATCH_THREADS = 512;
constexpr int DISPATCH_WARPS = DISPATCH_THREADS / 32;
constexpr int DISPATCH_MIN_CHUNK = 1024;
constexpr int DISPATCH_MAX_BLOCKS = 128;


// Data written earlier in the SAME kernel (by this block, before a __syncthreads) is read through
// L2, never through the read-only path.
template <bool SAME_KERNEL>
__device__ __forceinline__ int32_t ld_i32(const int32_t* p) {
  return SAME_KERNEL ? __ldcg(p) : __ldg(p);
}
template <bool SAME_KERNEL>
__device__ __forceinline__ int64_t ld_i64(const int64_t* p) {
  return SAME_KERNEL ? int64_t(__ldcg(reinterpret_cast<const long long*>(p))) : *p;
}

// Pass 2: plan + stable scatter. Every block first sums the histograms itself (n_blocks is at most
// 128, the table sits in L2): per expert the total over all blocks and the share of the blocks
// before this one; from the totals the 128-aligned run offsets. Each block writes its slice of the
// tile -> expert map, block 0 the counts, offsets and the live padded length. Then pair i of
// expert e lands at
//   pad_offsets[e] + (#pairs of e in earlier blocks) + (#pairs of e earlier in this block):
// inside the block each warp owns a contiguous slice; warps first count their slice, the counts are
// prefix-summed over warps, then every warp walks its slice 32 pairs at a time and ranks equal
// experts with __match_any_sync (lower lane = lower pair id = earlier slot).
// Launched with one block and n_blocks = 0 for an empty input (the plan is still written).
template <bool SAME_KERNEL>
__device__ __forceinline__ void dispatch_scatter_body(
    const int64_t* topk_idx, int64_t n_pairs, int n_experts, int chunk, int n_blocks,
    const int32_t* block_hist, int32_t* counts, int32_t* pad_offsets, int32_t* n_post_pad,
    int32_t* expert_ids, int64_t n_tiles_cap, int32_t* sorted_ids, int32_t* inv_ids,
    int32_t capacity, int32_t n_capped, int blk, int nblk) {
  // capacity > 0: an expert keeps the first `capacity` pairs of its run (lowest pair ids) and drops
  // the rest: a dropped pair gets no slot (inv_ids = -1) and the runs are laid out by the kept
  // counts, while counts[] still reports the routing decisions. Only experts below n_capped are
  // limited (the always-on shared experts dispatched as extra experts behind them are not).
  const int32_t cap_all = capacity > 0 ? capacity : INT32_MAX;
  auto cap_of = [&](int e) { return e < n_capped ? cap_all : INT32_MAX; };
  __shared__ int32_t total[MAX_EXPERTS];
  __shared__ int32_t before[MAX_EXPERTS];
  __shared__ int32_t off[MAX_EXPERTS + 1];
  __shared__ int32_t cursor[DISPATCH_WARPS][MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // totals and earlier-block shares: warp w takes experts w, w + WARPS, ...; lanes stride over the
  // blocks. Four experts per round with every load issued before the first sum (the table is small
  // and the kernel latency-bound: one expert at a time left ten dependent round trips per warp).
  static_assert(DISPATCH_MAX_BLOCKS <= 128, "a lane reads at most four blocks per expert");
  for (int e0 = warp; e0 < n_experts; e0 += 4 * DISPATCH_WARPS) {
    int32_t v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = e0 + u * DISPATCH_WARPS;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int b = lane + 32 * j;
        v[u][j] = (e < n_experts && b < n_blocks) ? ld_i32<SAME_KERNEL>(block_hist + int64_t(e) * n_blocks + b) : 0;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = e0 + u * DISPATCH_WARPS;
      int32_t tot = 0, bef = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        tot += v[u][j];
        if (lane + 32 * j < blk) bef += v[u][j];
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        tot += __shfl_xor_sync(0xffffffffu, tot, o);
        bef += __shfl_xor_sync(0xffffffffu, bef, o);
      }
      if (lane == 0 && e < n_experts) {
        total[e] = tot;
        before[e] = bef;
      }
    }
  }
  for (int i = threadIdx.x; i < DISPATCH_WARPS * MAX_EXPERTS; i += blockDim.x)
    (&cursor[0][0])[i] = 0;
  __syncthreads();
  // exclusive scan of the padded run lengths (one warp, 8 consecutive experts per lane)
  if (warp == 0) {
    constexpr int PER = MAX_EXPERTS / 32;
    int32_t pad[PER];
    int32_t mine = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane * PER + i;
      pad[i] = e < n_experts ? (min(total[e], cap_of(e)) + ALIGN_M - 1) / ALIGN_M * ALIGN_M : 0;
      mine += pad[i];
    }
    int32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int32_t run = incl - mine;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane * PER + i;
      if (e <= n_experts) off[e] = run;
      run += pad[i];
    }
    if (lane == 31) off[MAX_EXPERTS] = run;  // n_experts == MAX_EXPERTS: no lane holds that index
  }
  __syncthreads();
  const int32_t live = off[n_experts];
  if (blk == 0) {
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = total[e];
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) pad_offsets[e] = off[e];
    if (threadIdx.x == 0) *n_post_pad = live;
  }
  if (expert_ids != nullptr) {
    const int64_t per = (n_tiles_cap + nblk - 1) / nblk;
    const int64_t t_hi = per * (blk + 1) < n_tiles_cap ? per * (blk + 1) : n_tiles_cap;
    for (int64_t tile = per * blk + threadIdx.x; tile < t_hi; tile += blockDim.x) {
      int32_t owner = 0;
      const int64_t row = tile * ALIGN_M;
      if (row < live) {
        // last expert whose run starts at or before this row and is non-empty there
        int lo = 0, hi = n_experts;  // invariant: off[lo] <= row < off[hi]
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (off[mid] <= row) lo = mid; else hi = mid;
        }
        owner = lo;
      }
      expert_ids[tile] = owner;
    }
  }
  if (n_blocks == 0) return;

  const int slice = chunk / DISPATCH_WARPS;  // chunk is a multiple of the warp count
  const int64_t wbase = int64_t(blk) * chunk + int64_t(warp) * slice;
  const int64_t wend = wbase + slice;          // a slice need not be a multiple of 32
  auto expert_of = [&](int64_t pidx) {
    int32_t e = -1;
    if (pidx < n_pairs && pidx < wend) {
      const int64_t ee = ld_i64<SAME_KERNEL>(topk_idx + pidx);
      e = (ee >= 0 && ee < n_experts) ? int32_t(ee) : -1;
    }
    return e;
  };
  // the pairs' expert ids are fetched four rounds at a time, ahead of the counting / ranking
  constexpr int UB = 4;
  for (int r = 0; r < slice; r += 32 * UB) {
    int32_t ev[UB];
#pragma unroll
    for (int u = 0; u < UB; ++u) ev[u] = expert_of(wbase + r + 32 * u + lane);
#pragma unroll
    for (int u = 0; u < UB; ++u)
      if (ev[u] >= 0) atomicAdd(&cursor[warp][ev[u]], 1);
  }
  __syncthreads();
  // exclusive prefix over warps (ranks inside the expert's run), seeded with the earlier blocks' share
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int32_t run = before[e];
    for (int w = 0; w < DISPATCH_WARPS; ++w) {
      const int32_t c = cursor[w][e];
      cursor[w][e] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int r = 0; r < slice; r += 32 * UB) {
    int32_t ev[UB];
#pragma unroll
    for (int u = 0; u < UB; ++u) ev[u] = expert_of(wbase + r + 32 * u + lane);
#pragma unroll
    for (int u = 0; u < UB; ++u) {
      const int64_t pidx = wbase + r + 32 * u + lane;
      const int32_t e = ev[u];
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (e >= 0) {
        const int32_t rank = cursor[warp][e] + __popc(peers & ((1u << lane) - 1u));
        if (rank < cap_of(e)) {
          const int32_t dst = off[e] + rank;
          sorted_ids[dst] = int32_t(pidx);
          inv_ids[pidx] = dst;
        } else {
          inv_ids[pidx] = -1;   // over capacity: dropped
        }
      } else if (pidx < n_pairs && pidx < wend) {
        inv_ids[pidx] = -1;     // expert id out of range (status word already set): no slot
      }
      __syncwarp();
      if (e >= 0 && lane == 31 - __clz(peers)) cursor[warp][e] += __popc(peers);
      __syncwarp();
    }
  }
}


}  // namespace moe
