// Per-expert weight gradient C[e] = A_e^T @ B_e on CTA PAIRS (tcgen05.mma.cta_group::2): the same
// work items, split-K chunks, walk order and partial-tile layout as wgrad_gemm_kernel
// (gemm_wgrad.cuh), but a cluster of two CTAs computes a 256 x BN tile of C: CTA r loads the 128
// A columns of ITS half of the tile's rows of C and only HALF of the B columns, the leader issues
// one M = 256 MMA per K step, each CTA's accumulator rows land in its own TMEM and each CTA stores
// its own 128 x BN tile. The weight-gradient GEMMs wait for operands (a 128 x 256 tile needs 48 KB
// per 64-row K block for 0.26 us of MMA); a pair needs 32 KB per CTA for the same MMA time.
// When m_dim is not a multiple of 256 the last pair's second CTA has no rows of C: its A loads are
// out of range (zero fill, no traffic) and it stores nothing.
// Barrier protocol as in gemm_rows2.cuh. Plain (non-gathered) operands only.
#pragma once

namespace moe {

template <int BN, int STAGES>
struct Wgrad2Smem {
  static constexpr int B_STAGE_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int N_BARS = 2 * STAGES + 4;
  static constexpr int MISC_OFFSET = BAR_OFFSET + 8 * N_BARS;
  static constexpr int TABLE_OFFSET = MISC_OFFSET + 16;
  static constexpr int ORDER_OFFSET = TABLE_OFFSET + 2 * (WGRAD_MAX_GROUPS + 1) * 4;
  static constexpr int TOTAL = ORDER_OFFSET + 2 * WGRAD_SORT_MAX * 4;
  static constexpr int DYNAMIC = TOTAL + 1024;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
  static_assert(BN % 128 == 0, "a B half must be whole 64-column boxes");
};

// tiles_x = number of 128-row tiles of C (the partial-tile layout and the reduction pass count in
// those); pairs_x = ceil(tiles_x / 2).
template <int BN, int STAGES>
__global__ void __launch_bounds__(WGRAD_THREADS, 1)
    wgrad_gemm2_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmAlt, const WgradArgs p, int tiles_x,
                       int tiles_y) {
  pdl_trigger();
  pdl_wait();
  using L = Wgrad2Smem<BN, STAGES>;
  constexpr uint32_t TMEM_BUF = BN <= 128 ? 128 : 256;
  constexpr uint32_t TMEM_COLS = 2 * TMEM_BUF;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* first_item = reinterpret_cast<int*>(smem + L::TABLE_OFFSET);
  int* run_start = first_item + WGRAD_MAX_GROUPS + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int n_clusters = int(gridDim.x) >> 1;
  const int cluster = int(blockIdx.x) >> 1;

  if (warp == 2) {
    wgrad_build_table(p, lane, first_item, run_start);
    if (blockIdx.x == 0) {
      __syncwarp();
      for (int g = lane; g <= p.n_groups; g += 32) p.item_table[g] = first_item[g];
    }
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmAlt);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + b, 1);
      mbar_init(tempty_bar + b, 2 * EPI_WARPS);   // leader only: epilogue warps of both CTAs
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int pairs_x = (tiles_x + 1) >> 1;
  const int units_xy = pairs_x * tiles_y;      // pair tiles per work item
  const int tiles_xy = tiles_x * tiles_y;      // single tiles per work item (partial layout)
  const int n_items = first_item[p.n_groups];
  const int total = n_items * units_xy;
  int* order = reinterpret_cast<int*>(smem + L::ORDER_OFFSET);
  int* isize = order + WGRAD_SORT_MAX;
  const bool sorted = n_items <= WGRAD_SORT_MAX;
  if (sorted) {
    for (int i = threadIdx.x; i < n_items; i += blockDim.x)
      isize[i] = wgrad_item(p, first_item, run_start, i).num_k;
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
      const int mine = isize[i];
      int rk = 0;
      for (int k = 0; k < n_items; ++k) {
        const int other = isize[k];
        rk += (other > mine || (other == mine && k < i)) ? 1 : 0;
      }
      order[rk] = i;
    }
    __syncthreads();
  }
  auto item_at = [&](int pos) { return sorted ? order[pos] : pos; };
  auto unit_of_round = [&](int rnd) {   // serpentine over the clusters
    return rnd * n_clusters + ((rnd & 1) ? n_clusters - 1 - cluster : cluster);
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int rnd = 0; rnd * n_clusters < total && !*abort_flag; ++rnd) {
        const int t = unit_of_round(rnd);
        if (t >= total) continue;
        const WgradItem w = wgrad_item(p, first_item, run_start, item_at(t / units_xy));
        const int uxy = t % units_xy;
        const int m0 = ((uxy / tiles_y) * 2 + int(rank)) * BM;       // this CTA's rows of C
        const int n0 = (uxy % tiles_y) * BN + int(rank) * (BN / 2);  // this CTA's half of B
        const int ga = p.a_grouped ? w.group : 0, gb = p.b_grouped ? w.group : 0;
        const bool alt = p.alt_which != 0 && w.group >= p.alt_first_group;
        const bool a_alt = alt && p.alt_which == 1, b_alt = alt && p.alt_which == 2;
        const CUtensorMap* ma = a_alt ? &tmAlt : &tmA;
        const CUtensorMap* mb = b_alt ? &tmAlt : &tmB;
        for (int kt = 0; kt < w.num_k; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t use = it / STAGES;
          if (use > 0 && !mbar_wait(empty_bar + s, (use - 1) & 1, p.status)) {
            *abort_flag = 1;
            atomicExch(p.status, ST_WAIT_TIMEOUT);
            break;
          }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full_bar + s, 2 * L::STAGE_BYTES);
          const int r = w.row0 + kt * BK;
          const int r_alt = r - run_start[w.group];
          // 4-D maps (64 cols, row, col / 64, group); a box group past the last column is zero fill
          tma_load_4d_2cta(sA, ma, full_bar + s, 0, a_alt ? r_alt : r, m0 / 64, a_alt ? 0 : ga);
          tma_load_4d_2cta(sB, mb, full_bar + s, 0, b_alt ? r_alt : r, n0 / 64, b_alt ? 0 : gb);
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc(2 * BM, BN, true, true);
      uint32_t it = 0;
      int ju = 0;
      for (int rnd = 0; rnd * n_clusters < total && !*abort_flag; ++rnd) {
        const int t = unit_of_round(rnd);
        if (t >= total) continue;
        const WgradItem w = wgrad_item(p, first_item, run_start, item_at(t / units_xy));
        if (w.num_k == 0) continue;
        const int b = ju & 1;
        const uint32_t use = uint32_t(ju) >> 1;
        ++ju;
        if (use > 0 && !mbar_wait(tempty_bar + b, (use - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * TMEM_BUF;
        for (int kt = 0; kt < w.num_k; ++kt, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar + s, (it / STAGES) & 1, p.status)) {
            *abort_flag = 1;
            atomicExch(p.status, ST_WAIT_TIMEOUT);
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sB = sA + A_STAGE_BYTES;
#pragma unroll
          for (int k16 = 0; k16 < BK / 16; ++k16)
            umma_f16_2cta(d_tmem, umma_desc(sA + k16 * MN_KADV, MN_LBO, MN_SBO),
                          umma_desc(sB + k16 * MN_KADV, MN_LBO, MN_SBO), idesc,
                          (kt == 0 && k16 == 0) ? 0u : 1u);
          umma_commit_2cta(empty_bar + s, 3);
        }
        umma_commit_2cta(tfull_bar + b, 3);
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    const int ew = warp - 2;
    const int q = warp & 3;
    const int half = ew >> 2;
    const int row = q * 32 + lane;
    constexpr int NCH = BN / 32;
    const int c_lo = half * (NCH / 2), c_hi = c_lo + NCH / 2;
    const uint32_t tempty_leader = mapa_u32(smem_u32(tempty_bar), 0);

    int ju = 0;
    for (int rnd = 0; rnd * n_clusters < total; ++rnd) {
      const int t = unit_of_round(rnd);
      if (t >= total) continue;
      const int j = item_at(t / units_xy), uxy = t % units_xy;
      const WgradItem w = wgrad_item(p, first_item, run_start, j);
      const int tile_m = (uxy / tiles_y) * 2 + int(rank);     // this CTA's 128-row tile of C
      const int m0 = tile_m * BM, n0 = (uxy % tiles_y) * BN;
      const bool tile_ok = tile_m < tiles_x;
      const bool have_acc = w.num_k > 0;
      const int b = ju & 1;
      if (have_acc) {
        if (!mbar_wait(tfull_bar + b, (uint32_t(ju) >> 1) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        tc_fence_after();
        ++ju;
      }
      const uint32_t taddr = tmem_base + b * TMEM_BUF + (uint32_t(q * 32) << 16);
      const int m = m0 + row;
      const bool m_ok = tile_ok && m < p.m_dim;
      __nv_bfloat16* dst = (w.group < p.n_out1 ? p.out + int64_t(w.group) * p.m_dim * p.n_dim
                                               : p.out_extra + int64_t(w.group - p.n_out1) *
                                                                   p.m_dim * p.n_dim) +
                           int64_t(m) * p.n_dim + n0;
      const int txy = tile_m * tiles_y + (uxy % tiles_y);
      float* mine = p.partials + (int64_t(j) * tiles_xy + txy) * (int64_t(BM) * BN);
      if (tile_ok) {
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
          float v[32];
          if (have_acc) {
            tmem_ld32(taddr + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
          }
          if (w.n_c == 1) {
            if (m_ok && n0 + c * 32 < p.n_dim) store_bf16x32(dst + c * 32, v);
          } else {
            store_f32x32(mine + (int64_t(c) * BM + row) * 32, v);
          }
        }
      }
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_leader + b * 8);
      }
    }
  }

  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc2(tmem_base, TMEM_COLS);
}

}  // namespace moe
