// Row-grouped GEMM on CTA PAIRS (tcgen05.mma.cta_group::2), routed schedule. Same math, operands and
// epilogues as rows_gemm_kernel (gemm_rows.cuh); what changes is who loads what:
//
//   A cluster of two CTAs takes two consecutive 128-row blocks of ONE expert's run and one N chunk.
//   Each CTA loads its own block's A rows and only HALF of the expert's weight tile; the leader
//   CTA's MMA warp issues one M = 256 instruction per K step that reads A from both CTAs and the
//   two B halves where they lie, and writes each CTA's 128 accumulator rows into that CTA's own
//   TMEM. The row GEMMs of this block are bound by what the SMs can pull out of L2 (a 128-row tile
//   re-reads its expert's whole weight tile: 295 KB for the up GEMM against 147 KB of rows), so
//   halving the weight traffic per SM is what the pairing is for. No multicast load is involved.
//
//   A run with an odd number of blocks leaves its last pair half empty: the second CTA then works
//   on rows of the following run (any finite or non-finite values: accumulator rows are
//   independent) and its epilogue stores nothing.
//
// Barriers. The smem ring's "full" barriers live in the leader only: both CTAs' TMA loads signal
// them (.cta_group::2 form of the load, barrier address with the peer bit cleared) and the leader's
// producer posts the byte count of both CTAs' loads. The MMA warp's commits are multicast to both
// CTAs ("empty" barriers of the ring, "accumulator full" barriers). Epilogue warps of both CTAs
// arrive on the leader's "accumulator empty" barriers (the peer through mapa). All waits are
// bounded; the two CTAs meet in a cluster barrier before they free TMEM and leave.
#pragma once

namespace moe {

constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;  // clears the bit that tells the pair's CTAs apart

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// (Default semantics, release at CTA scope: what the barrier orders is this warp's TMEM reads, which
// tcgen05.fence::before_thread_sync covers. A cluster-scope release would also wait until the
// epilogue's global stores are visible to the other SM -- microseconds per tile.)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_f16_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `mask` once all MMAs issued so
// far by this thread have finished.
__device__ __forceinline__ void umma_commit_2cta(uint64_t* bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], "
      "%1;" ::"r"(smem_u32(bar)),
      "h"(mask)
      : "memory");
}
// Tiled loads of a CTA pair: the completion bytes go to the LEADER's barrier at this offset.
__device__ __forceinline__ void tma_load_3d_2cta(void* dst, const CUtensorMap* m, uint64_t* bar,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_2cta(void* dst, const CUtensorMap* m, uint64_t* bar,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(c0), "r"(c1),
      "r"(c2), "r"(c3)
      : "memory");
}

constexpr int ROWS2_MAX_GROUPS = 256;

template <int BN, int STAGES, int EPI>
struct Rows2Smem {
  static constexpr int B_STAGE_BYTES = (BN / 2) * BK * 2;   // this CTA's half of the weight tile
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;  // 1024-byte aligned
  static constexpr int RED_TILE_BYTES = (BM * red_row_bytes(BN) + 1023) / 1024 * 1024;
  static constexpr int STAGING_BYTES = epi_reduces(EPI) ? 2 * RED_TILE_BYTES : 0;
  static constexpr int AUX_OFFSET = STAGING_OFFSET + STAGING_BYTES;
  static constexpr int AUX_TILE_BYTES = BM * 2 * BN * 2;
  static constexpr int BAR_OFFSET = AUX_OFFSET + (epi_loads_aux(EPI) ? 2 * AUX_TILE_BYTES : 0);
  static constexpr int N_BARS = 2 * STAGES + 8;
  static constexpr int MISC_OFFSET = BAR_OFFSET + 8 * N_BARS;
  static constexpr int PART_OFFSET = MISC_OFFSET + 16;
  static constexpr int RED_TOK_OFFSET = PART_OFFSET + 128 * 4;
  static constexpr int TABLE_OFFSET = RED_TOK_OFFSET + 2 * 128 * 4;   // pair_first, run_start
  static constexpr int TOTAL = TABLE_OFFSET + 2 * (ROWS2_MAX_GROUPS + 1) * 4;
  static constexpr int DYNAMIC = TOTAL + 1024;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
};

struct Unit2 {
  int group, m_tile, n0;
  bool valid;   // false: this CTA's half of the pair is past the end of the run
};

template <int BN, int STAGES, bool B_MN, int EPI>
__global__ void __launch_bounds__(rows_threads(EPI, false), 1)
    rows_gemm2_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmA2,
                      const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmB2,
                      const __grid_constant__ CUtensorMap tmOut, const RowsArgs p) {
  pdl_trigger();
  pdl_wait();
  using L = Rows2Smem<BN, STAGES, EPI>;
  static_assert(BN % 32 == 0 && BN <= 256, "BN must be a multiple of 32 up to 256");
  static_assert(!B_MN || BN % 128 == 0, "an MN-major weight half must be whole 64-column boxes");
  constexpr uint32_t TMEM_BUF = BN <= 128 ? 128 : 256;
  constexpr uint32_t TMEM_COLS = 2 * TMEM_BUF;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  [[maybe_unused]] uint64_t* afull_bar = tempty_bar + 2;
  [[maybe_unused]] uint64_t* aempty_bar = afull_bar + 2;
  constexpr bool AUX_IN = epi_loads_aux(EPI);
  constexpr int AUX_WARP = 2 + EPI_WARPS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  [[maybe_unused]] float* dtw_part = reinterpret_cast<float*>(smem + L::PART_OFFSET);
  int* pair_first = reinterpret_cast<int*>(smem + L::TABLE_OFFSET);
  int* run_start = pair_first + ROWS2_MAX_GROUPS + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader of the pair
  const int n_clusters = int(gridDim.x) >> 1;
  const int cluster = int(blockIdx.x) >> 1;
  const int n_groups = p.n_groups_total;

  // ------------------------------------------------------------------------- pair table
  // pair_first[g] = number of block pairs of the runs before g (a run of t blocks has ceil(t / 2))
  if (warp == 2) {
    int running = 0;
    for (int base = 0; base < n_groups; base += 32) {
      const int g = base + lane;
      int lo = 0, hi = 0;
      if (g < n_groups) {
        lo = __ldg(p.a2_offsets + g);
        hi = __ldg(p.a2_offsets + g + 1);
      }
      const int mine = (((hi - lo) >> 7) + 1) >> 1;
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (g < n_groups) {
        pair_first[g] = running + incl - mine;
        run_start[g] = lo;
      }
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      pair_first[n_groups] = running;
      run_start[n_groups] = __ldg(p.a2_offsets + n_groups);
    }
  }
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmA2);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmB2);
    if constexpr (AUX_IN) tma_prefetch_desc(&tmOut);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + s, 1);    // used in the leader only: its producer's arrive + both CTAs' bytes
      mbar_init(empty_bar + s, 1);   // one multicast commit per use
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + b, 1);
      mbar_init(tempty_bar + b, 2 * EPI_WARPS);   // leader only: the epilogue warps of both CTAs
      mbar_init(afull_bar + b, epi_reduces(EPI) ? EPI_WARPS : 1);
      mbar_init(aempty_bar + b, epi_reduces(EPI) ? RED_WARPS : EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const int total_units = pair_first[n_groups] * p.n_chunks;
  if (cluster >= total_units) return;            // the same decision in both CTAs of the pair

  if (warp == 1) {
    tmem_alloc2(tmem_slot, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();     // both CTAs' barriers are initialised and both have their TMEM
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto decode = [&](int u) {
    Unit2 c;
    const int nc = u % p.n_chunks;
    const int pr = u / p.n_chunks;
    int lo = 0, hi = n_groups;      // pair_first[lo] <= pr < pair_first[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (pair_first[mid] <= pr) lo = mid; else hi = mid;
    }
    const int blk = 2 * (pr - pair_first[lo]) + int(rank);
    c.group = lo;
    c.m_tile = (run_start[lo] >> 7) + blk;
    c.valid = blk < ((run_start[lo + 1] - run_start[lo]) >> 7);
    c.n0 = nc * BN;
    return c;
  };

  if (AUX_IN && warp == AUX_WARP) {
    // ------------------------------------------------ pre-activation tiles for the epilogue
    if (elect_one()) {
      int j = 0;
      for (int u = cluster; u < total_units && !*abort_flag; u += n_clusters, ++j) {
        const Unit2 tc = decode(u);
        const int b = j & 1;
        const uint32_t use = uint32_t(j) >> 1;
        if (use > 0 && !mbar_wait(aempty_bar + b, (use - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        uint8_t* dst = smem + L::AUX_OFFSET + b * L::AUX_TILE_BYTES;
        mbar_expect_tx(afull_bar + b, L::AUX_TILE_BYTES);
#pragma unroll
        for (int i = 0; i < 2 * BN / 64; ++i)
          tma_load_3d(dst + i * OUT_BOX_BYTES, &tmOut, afull_bar + b, 64 * i, tc.m_tile * BM, 0);
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      uint32_t it = 0;
      for (int u = cluster; u < total_units && !*abort_flag; u += n_clusters) {
        const Unit2 tc = decode(u);
        const bool a_alt = tc.group >= p.a2_first_group;
        const int a_start = a_alt ? run_start[tc.group] : 0;
        const bool first = tc.group < p.n_groups_b1;
        const CUtensorMap* mb = first ? &tmB : &tmB2;
        const int gb = first ? tc.group : tc.group - p.n_groups_b1;
        for (int kt = 0; kt < p.num_k; ++kt, ++it) {
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
          const int k0 = kt * BK;
          if (a_alt)
            tma_load_3d_2cta(sA, &tmA2, full_bar + s, k0, tc.m_tile * BM - a_start, 0);
          else
            tma_load_3d_2cta(sA, &tmA, full_bar + s, k0, tc.m_tile * BM, 0);
          if constexpr (B_MN) {   // 4-D map: (64 n, k, n / 64, group), BN / 128 boxes per copy
            tma_load_4d_2cta(sB, mb, full_bar + s, 0, k0, tc.n0 / 64 + int(rank) * (BN / 128), gb);
          } else {                // 3-D map: (k, n, group), BN / 2 weight rows per copy
            tma_load_3d_2cta(sB, mb, full_bar + s, k0, tc.n0 + int(rank) * (BN / 2), gb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc(2 * BM, BN, false, B_MN);
      uint32_t it = 0;
      int j = 0;
      for (int u = cluster; u < total_units && !*abort_flag; u += n_clusters, ++j) {
        const int b = j & 1;
        const uint32_t use = uint32_t(j) >> 1;
        if (use > 0 && !mbar_wait(tempty_bar + b, (use - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * TMEM_BUF;
        for (int kt = 0; kt < p.num_k; ++kt, ++it) {
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
          for (int k16 = 0; k16 < BK / 16; ++k16) {
            const uint64_t da = umma_desc(sA + k16 * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_desc(sB + k16 * MN_KADV, MN_LBO, MN_SBO)
                                     : umma_desc(sB + k16 * 32, 16, 1024);
            umma_f16_2cta(d_tmem, da, db, idesc, (kt == 0 && k16 == 0) ? 0u : 1u);
          }
          umma_commit_2cta(empty_bar + s, 3);   // the stage is free in both CTAs
        }
        umma_commit_2cta(tfull_bar + b, 3);     // the accumulators are ready in both CTAs
      }
    }
  } else if (epi_reduces(EPI) && warp >= 2 + EPI_WARPS) {
    // ------------------------------------------------------------------------ reducers
    if constexpr (epi_reduces(EPI)) {
      constexpr int ROWB = red_row_bytes(BN);
      int* tok_all = reinterpret_cast<int*>(smem + L::RED_TOK_OFFSET);
      const uint64_t keep = l2_policy_evict_last();
      int j = 0;
      for (int u = cluster; u < total_units; u += n_clusters, ++j) {
        const Unit2 tc = decode(u);
        const int b = j & 1;
        if (!mbar_wait(afull_bar + b, (uint32_t(j) >> 1) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        const int ncols = min(BN, p.n_dim - tc.n0);
        const int ppr = ncols >> 3;
        const uint32_t stg = smem_u32(smem + L::STAGING_OFFSET + b * L::RED_TILE_BYTES);
        const int* toks = tok_all + b * BM;
        __nv_bfloat16* dst0 = p.out + tc.n0 + lane * 8;
        constexpr int RED_UNROLL = 8;
        constexpr int STEP = 2 * RED_WARPS;
        const int rw = warp - (2 + EPI_WARPS);
        if (lane < BM / STEP) {
          const int r = rw + RED_WARPS + lane * STEP;
          const int tok = toks[r];
          if (tok >= 0)
            bulk_reduce_add_bf16(p.out + tc.n0 + int64_t(tok) * p.ld_out,
                                 smem + L::STAGING_OFFSET + b * L::RED_TILE_BYTES + r * ROWB,
                                 uint32_t(ncols) * 2u);
        }
        bulk_commit();
#pragma unroll 1
        for (int r0 = rw; r0 < BM; r0 += STEP * RED_UNROLL) {
          uint32_t w[RED_UNROLL][4];
          int tk[RED_UNROLL];
#pragma unroll
          for (int q = 0; q < RED_UNROLL; ++q) {
            const int r = r0 + q * STEP;
            tk[q] = lane < ppr ? toks[r] : -1;
            ld_shared_v4(stg + r * ROWB + (lane < ppr ? lane : 0) * 16, w[q][0], w[q][1], w[q][2],
                         w[q][3]);
          }
#pragma unroll
          for (int q = 0; q < RED_UNROLL; ++q)
            if (tk[q] >= 0)
              red_add_bf16x8(dst0 + int64_t(tk[q]) * p.ld_out, w[q][0], w[q][1], w[q][2], w[q][3],
                             keep);
        }
        bulk_wait_read<0>();
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty_bar + b);
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ---------------------------------------------------------------------- epilogue (both CTAs)
    const int ew = warp - 2;
    const int q = warp & 3;
    const int half = ew >> 2;
    const int row = q * 32 + lane;
    constexpr int NCH = (EPI == EPI_GLU ? BN / 2 : BN) / 32;
    const int c_lo = half * (NCH / 2), c_hi = c_lo + NCH / 2;
    // the leader's "accumulator empty" barriers, as cluster addresses
    const uint32_t tempty_leader = mapa_u32(smem_u32(tempty_bar), 0);

    auto load_pair = [&](int u) {
      if (u >= total_units || p.sorted_ids == nullptr) return p.n_pairs;
      const Unit2 c = decode(u);
      return c.valid ? __ldg(p.sorted_ids + int64_t(c.m_tile) * BM + row) : p.n_pairs;
    };
    auto load_w = [&](int pr) {
      if (p.pair_w == nullptr) return 1.f;
      return pr < p.n_pairs ? __bfloat162float(__ldg(p.pair_w + pr)) : 0.f;
    };
    int pair = load_pair(cluster);
    int pair_n = load_pair(cluster + n_clusters);
    float w = load_w(pair);

    int j = 0;
    for (int u = cluster; u < total_units; u += n_clusters, ++j) {
      const Unit2 tc = decode(u);
      const int b = j & 1;
      const float w_n = load_w(pair_n);
      const int pair_nn = load_pair(u + 2 * n_clusters);
      if (!mbar_wait(tfull_bar + b, (uint32_t(j) >> 1) & 1, p.status))
        atomicExch(p.status, ST_WAIT_TIMEOUT);
      tc_fence_after();
      const uint32_t taddr = tmem_base + b * TMEM_BUF + (uint32_t(q * 32) << 16);
      const int64_t grow = int64_t(tc.m_tile) * BM + row;
      const bool row_ok = tc.valid;
      __nv_bfloat16* out_row = p.out + grow * p.ld_out;

      [[maybe_unused]] const __nv_bfloat16* bias_row = nullptr;
      if constexpr (EPI == EPI_GLU || EPI == EPI_SCALE_RED) {
        if (p.bias != nullptr) bias_row = p.bias + int64_t(tc.group) * p.n_dim;
      }
      if constexpr (EPI == EPI_GLU) {
        __nv_bfloat16* raw_row = p.out2 ? p.out2 + grow * BN : nullptr;
        switch (p.act) {
          case ACT_SILU: epilogue_glu<ACT_SILU, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          case ACT_GELU: epilogue_glu<ACT_GELU, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          case ACT_RELU: epilogue_glu<ACT_RELU, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          case ACT_SIGMOID: epilogue_glu<ACT_SIGMOID, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          default: epilogue_glu<ACT_TANH, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
        }
      } else if constexpr (EPI == EPI_RAW_RED || EPI == EPI_SCALE_RED) {
        constexpr int NB = BN / 64;
        constexpr int ROWB = red_row_bytes(BN);
        const int tok = (row_ok && pair < p.n_pairs) ? pair / p.top_k : -1;
        if (j >= 2 && !mbar_wait(aempty_bar + b, ((uint32_t(j) >> 1) - 1) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        uint8_t* stg = smem + L::STAGING_OFFSET + b * L::RED_TILE_BYTES;
        if (half == 0) reinterpret_cast<int*>(smem + L::RED_TOK_OFFSET)[b * BM + row] = tok;
        const uint32_t my_row = smem_u32(stg) + row * ROWB + half * 64;
        float v[2][32];
        tmem_ld32(taddr + half * 32, v[0]);
#pragma unroll
        for (int jb = 0; jb < NB; ++jb) {
          tmem_ld_wait();
          if (jb + 1 < NB) tmem_ld32(taddr + (jb + 1) * 64 + half * 32, v[(jb + 1) & 1]);
          float* cur = v[jb & 1];
          if constexpr (EPI == EPI_SCALE_RED) {
            if (bias_row != nullptr && tc.n0 + jb * 64 + half * 32 < p.n_dim)
              add_bias32(cur, bias_row + tc.n0 + jb * 64 + half * 32);
#pragma unroll
            for (int i = 0; i < 32; ++i) cur[i] *= w;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t wd[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(cur[8 * i + 2 * k], cur[8 * i + 2 * k + 1]);
              wd[k] = *reinterpret_cast<uint32_t*>(&h2);
            }
            st_shared_v4(my_row + jb * 128 + i * 16, wd[0], wd[1], wd[2], wd[3]);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(afull_bar + b);
      } else {  // EPI_GLUBWD
        __nv_bfloat16* da1 = out_row;  // ld_out == 2 * BN
        __nv_bfloat16* hw = p.out2 + grow * BN;
        if (!mbar_wait(afull_bar + b, (uint32_t(j) >> 1) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        const uint32_t a1_tile = smem_u32(smem + L::AUX_OFFSET + b * L::AUX_TILE_BYTES);
        float part;
        switch (p.act) {
          case ACT_SILU: part = epilogue_glubwd<ACT_SILU, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          case ACT_GELU: part = epilogue_glubwd<ACT_GELU, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          case ACT_RELU: part = epilogue_glubwd<ACT_RELU, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          case ACT_SIGMOID: part = epilogue_glubwd<ACT_SIGMOID, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          default: part = epilogue_glubwd<ACT_TANH, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty_bar + b);
        if (p.dtw != nullptr) {
          if (half == 1) {
            if (j > 0) named_bar_sync(2, EPI_WARPS * 32);
            dtw_part[row] = part;
            named_bar_arrive(1, EPI_WARPS * 32);
          } else {
            named_bar_sync(1, EPI_WARPS * 32);
            if (row_ok && pair < p.n_pairs) p.dtw[pair] = __float2bfloat16(part + dtw_part[row]);
            if (u + n_clusters < total_units) named_bar_arrive(2, EPI_WARPS * 32);
          }
        }
      }
      // this warp has drained its share of accumulator buffer b: tell the leader's MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + b * 8);
      pair = pair_n;
      pair_n = pair_nn;
      w = w_n;
    }
  }

  // Nobody leaves while the other CTA may still signal its barriers or read its shared memory.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc2(tmem_base, TMEM_COLS);
}

}  // namespace moe
