// Per-expert weight gradient C[e] = A_e^T @ B_e with split-K over the run's rows (see gemm.cuh).
// Both operands are read MN-major straight out of [rows, width] activation buffers (64 x 64 TMA
// boxes), the contraction index is the row. 192 threads: warp 0 TMA, warp 1 MMA, warps 2..5 epilogue.
//
// Work item = (m tile, n chunk, split-K chunk). A run longer than ks_rows is cut into chunks; each
// chunk's CTA writes an fp32 partial tile and wgrad_reduce_kernel then adds a tile's partials in
// chunk order and writes bf16 (deterministic, and the reduction is spread over many CTAs). Runs
// that fit one chunk (the common case for routed experts) store bf16 directly and skip the second
// pass. An empty run still owns one work item, which writes zeros.
#pragma once

namespace moe {

constexpr int WGRAD_THREADS = 192;

template <int BN, int STAGES>
struct WgradSmem {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int MISC_OFFSET = BAR_OFFSET + 8 * (2 * STAGES + 1);
  static constexpr int TOTAL = MISC_OFFSET + 32;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

// Number of split-K work items of a run of `rows` rows.
__host__ __device__ __forceinline__ int wgrad_chunks(int rows, int ks_rows) {
  const int c = (rows + ks_rows - 1) / ks_rows;
  return c > 0 ? c : 1;
}


// Warp-cooperative lookup of work item j: which run, which chunk of it. Writes
// sched = {group (-1 if j is past the last item), chunk, chunks of the group, first row, rows}.
__device__ __forceinline__ void wgrad_find_item(const WgradArgs& p, int j, int lane, int* sched) {
  int group = -1, chunk = 0, n_c = 0, row0 = 0, rows = 0;
  if (p.pad_offsets == nullptr) {
    n_c = wgrad_chunks(p.rows_host, p.ks_rows);
    if (j < n_c * p.n_groups) {
      group = j / n_c;
      chunk = j - group * n_c;
      row0 = chunk * p.ks_rows;
      rows = min(p.ks_rows, p.rows_host - row0);
    }
  } else {
    int running = 0;
    for (int base = 0; base < p.n_groups && group < 0; base += 32) {
      const int g = base + lane;
      int lo = 0, hi = 0;
      if (g < p.n_groups) {
        lo = __ldg(p.pad_offsets + g);
        hi = __ldg(p.pad_offsets + g + 1);
      }
      const int mine = g < p.n_groups ? wgrad_chunks(hi - lo, p.ks_rows) : 0;
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int excl = incl - mine;
      const bool owner = mine > 0 && j >= running + excl && j < running + incl;
      const unsigned who = __ballot_sync(0xffffffffu, owner);
      if (who) {
        const int src = __ffs(who) - 1;
        const int c = j - running - excl;
        group = __shfl_sync(0xffffffffu, g, src);
        chunk = __shfl_sync(0xffffffffu, c, src);
        n_c = __shfl_sync(0xffffffffu, mine, src);
        const int r0 = lo + c * p.ks_rows;
        row0 = __shfl_sync(0xffffffffu, r0, src);
        rows = __shfl_sync(0xffffffffu, max(0, min(p.ks_rows, hi - r0)), src);
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (lane == 0) {
    sched[0] = group; sched[1] = chunk; sched[2] = n_c; sched[3] = row0; sched[4] = rows;
  }
}

// First work-item index and chunk count of run `g` (warp-cooperative; result in out[0..1]).
__device__ __forceinline__ void wgrad_find_group(const WgradArgs& p, int g, int lane, int* out) {
  int first = 0, n_c = 0;
  if (p.pad_offsets == nullptr) {
    n_c = wgrad_chunks(p.rows_host, p.ks_rows);
    first = g * n_c;
  } else {
    int running = 0;
    for (int base = 0; base <= g; base += 32) {
      const int gg = base + lane;
      int mine = 0;
      if (gg < p.n_groups)
        mine = wgrad_chunks(__ldg(p.pad_offsets + gg + 1) - __ldg(p.pad_offsets + gg), p.ks_rows);
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (g >= base && g < base + 32) {
        first = running + __shfl_sync(0xffffffffu, incl - mine, g - base);
        n_c = __shfl_sync(0xffffffffu, mine, g - base);
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (lane == 0) {
    out[0] = first;
    out[1] = n_c;
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(WGRAD_THREADS)
    wgrad_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const WgradArgs p) {
  using L = WgradSmem<BN, STAGES>;
  constexpr uint32_t TMEM_COLS = BN <= 128 ? 128 : 256;
  static_assert(BN % 64 == 0 && BN <= 256, "BN must be a multiple of 64 up to 256");

  __shared__ int sched[5];  // group, chunk, chunks of the group, first row, rows in this chunk
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.z;  // global work-item index along split-K
  if (warp == 0) wgrad_find_item(p, j, lane, sched);
  __syncthreads();
  const int group = sched[0], chunk = sched[1], n_c = sched[2], row0 = sched[3];
  if (group < 0) return;  // past the last work item (uniform over the CTA, nothing set up yet)
  (void)chunk;
  const int num_k = (sched[4] + BK - 1) / BK;

  const int tile_m = blockIdx.x;
  const int n0 = blockIdx.y * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    mbar_init(accum_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      const int ga = p.a_grouped ? group : 0, gb = p.b_grouped ? group : 0;
      for (int kt = 0; kt < num_k; ++kt) {
        const int s = kt % STAGES;
        if (kt >= STAGES && !mbar_wait(empty_bar + s, ((kt / STAGES) - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        uint8_t* sA = smem + s * L::STAGE_BYTES;
        uint8_t* sB = sA + A_STAGE_BYTES;
        mbar_expect_tx(full_bar + s, L::STAGE_BYTES);
        const int r = row0 + kt * BK;
#pragma unroll
        for (int i = 0; i < BM / 64; ++i)
          tma_load_3d(sA + i * 8192, &tmA, full_bar + s, tile_m * BM + 64 * i, r, ga);
#pragma unroll
        for (int jj = 0; jj < BN / 64; ++jj)
          tma_load_3d(sB + jj * 8192, &tmB, full_bar + s, n0 + 64 * jj, r, gb);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      for (int kt = 0; kt < num_k; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(full_bar + s, (kt / STAGES) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t sA = smem_u32(smem + s * L::STAGE_BYTES);
        issue_stage_mmas<BN, true, true>(sA, sA + A_STAGE_BYTES, tmem_base, kt == 0);
        umma_commit(empty_bar + s);
      }
      umma_commit(accum_bar);
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
    const bool have_acc = num_k > 0;
    if (have_acc) {
      if (!mbar_wait(accum_bar, 0, p.status)) atomicExch(p.status, ST_WAIT_TIMEOUT);
      tc_fence_after();
    }
    const int m = tile_m * BM + row;
    const bool m_ok = m < p.m_dim;
    __nv_bfloat16* dst = p.out + (int64_t(group) * p.m_dim + m) * int64_t(p.n_dim) + n0;
    constexpr int NCH = BN / 32;

    if (n_c == 1) {
#pragma unroll 1
      for (int c = 0; c < NCH; ++c) {
        float v[32];
        if (have_acc) {
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (m_ok && n0 + c * 32 < p.n_dim) store_bf16x32(dst + c * 32, v);
      }
    } else {
      // fp32 partial of this chunk; slot layout [column chunk][row][32]
      const int64_t slot_elems = int64_t(BM) * BN;
      const int64_t tiles_xy = int64_t(gridDim.x) * gridDim.y;
      const int64_t tile_xy = int64_t(tile_m) * gridDim.y + blockIdx.y;
      float* mine = p.partials + (int64_t(j) * tiles_xy + tile_xy) * slot_elems;
#pragma unroll 1
      for (int c = 0; c < NCH; ++c) {
        float v[32];
        if (have_acc) {
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        store_f32x32(mine + (int64_t(c) * BM + row) * 32, v);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}


constexpr int WGRAD_REDUCE_SPLIT = 16;  // CTAs sharing the reduction of one output tile

// Second pass of the split-K weight gradient: for every (run, tile) that was split, add the fp32
// partial tiles in chunk order and write bf16. grid = (tiles_x * tiles_y * WGRAD_REDUCE_SPLIT,
// n_groups); tiles_x / tiles_y / BN must be those of the first pass.
template <int BN>
__global__ void __launch_bounds__(256)
    wgrad_reduce_kernel(const WgradArgs p, int tiles_x, int tiles_y) {
  __shared__ int info[2];
  const int g = blockIdx.y;
  if (threadIdx.x < 32) wgrad_find_group(p, g, threadIdx.x, info);
  __syncthreads();
  const int first = info[0], n_c = info[1];
  if (n_c <= 1) return;
  const int tile_xy = blockIdx.x / WGRAD_REDUCE_SPLIT;
  const int slice = blockIdx.x % WGRAD_REDUCE_SPLIT;
  const int tile_m = tile_xy / tiles_y, n0 = (tile_xy % tiles_y) * BN;
  const int64_t tiles_xy = int64_t(tiles_x) * tiles_y;
  constexpr int64_t slot_elems = int64_t(BM) * BN;
  constexpr int vecs = BM * BN / 4;                  // float4 per tile
  constexpr int per_slice = vecs / WGRAD_REDUCE_SPLIT;
  for (int f = slice * per_slice + threadIdx.x; f < (slice + 1) * per_slice; f += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c2 = 0; c2 < n_c; ++c2) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(
                                  p.partials + ((int64_t(first) + c2) * tiles_xy + tile_xy) * slot_elems) + f);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    // partial layout [column chunk][row][32 floats]
    const int cc = f / (BM * 8), row = (f / 8) % BM, i4 = f % 8;
    const int m = tile_m * BM + row, n = n0 + cc * 32 + i4 * 4;
    if (m < p.m_dim && n < p.n_dim) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 w;
      w.x = *reinterpret_cast<const uint32_t*>(&lo);
      w.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(p.out + (int64_t(g) * p.m_dim + m) * int64_t(p.n_dim) + n) = w;
    }
  }
}

}  // namespace moe
