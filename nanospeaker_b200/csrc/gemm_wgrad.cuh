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

constexpr int WGRAD_THREADS = 320;   // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
constexpr int WGRAD_THREADS_GATHER = 320 + (GATHER_WARPS - 1) * 32;  // + producer warps 10..12
constexpr int WGRAD_MAX_GROUPS = 256;
// Work items are walked longest first (up to this many; beyond it, in list order): CTAs take items
// round-robin, and with runs of very different lengths the list order left some CTAs with 1.6x the
// mean work at the bench's skew, the sorted order with 1.2x.
constexpr int WGRAD_SORT_MAX = 1024;

template <int BN, int STAGES>
struct WgradSmem {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int N_BARS = 2 * STAGES + 4;  // full, empty, tmem_full[2], tmem_empty[2]
  static constexpr int MISC_OFFSET = BAR_OFFSET + 8 * N_BARS;
  static constexpr int TABLE_OFFSET = MISC_OFFSET + 16;  // int first_item[G+1], int run_start[G+1]
  static constexpr int TOK_OFFSET = TABLE_OFFSET + 2 * (WGRAD_MAX_GROUPS + 1) * 4;  // int[64]
  static constexpr int ORDER_OFFSET = TOK_OFFSET + 64 * 4;  // int order[SORT_MAX], int size[SORT_MAX]
  static constexpr int TOTAL = ORDER_OFFSET + 2 * WGRAD_SORT_MAX * 4;
  static constexpr int DYNAMIC = TOTAL + 1024;
};

// Number of split-K work items of a run of `rows` rows.
__host__ __device__ __forceinline__ int wgrad_chunks(int rows, int ks_rows) {
  const int c = (rows + ks_rows - 1) / ks_rows;
  return c > 0 ? c : 1;
}

// Exclusive prefix of the per-run work-item counts into first_item[0..G] and the run starts into
// run_start[0..G]; executed by one full warp.
__device__ __forceinline__ void wgrad_build_table(const WgradArgs& p, int lane, int* first_item,
                                                  int* run_start) {
  int running = 0;
  for (int base = 0; base < p.n_groups; base += 32) {
    const int g = base + lane;
    int lo = 0, hi = 0;
    if (g < p.n_groups) {
      if (p.pad_offsets != nullptr) {
        lo = __ldg(p.pad_offsets + g);
        hi = __ldg(p.pad_offsets + g + 1);
      } else {
        hi = p.rows_host;
      }
    }
    const int mine = g < p.n_groups ? wgrad_chunks(hi - lo, p.ks_rows) : 0;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (g < p.n_groups) {
      first_item[g] = running + incl - mine;
      run_start[g] = lo;
    }
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) {
    first_item[p.n_groups] = running;
    run_start[p.n_groups] = p.pad_offsets != nullptr ? __ldg(p.pad_offsets + p.n_groups)
                                                     : p.rows_host;
  }
}

struct WgradItem {
  int group, first, n_c, row0, num_k;
};

// Work item j -> its run, its chunk and the rows it contracts over (binary search in the table).
__device__ __forceinline__ WgradItem wgrad_item(const WgradArgs& p, const int* first_item,
                                                const int* run_start, int j) {
  int lo = 0, hi = p.n_groups;  // first_item[lo] <= j < first_item[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (first_item[mid] <= j) lo = mid; else hi = mid;
  }
  WgradItem it;
  it.group = lo;
  it.first = first_item[lo];
  it.n_c = first_item[lo + 1] - it.first;
  const int start = run_start[lo];
  const int end = p.pad_offsets != nullptr ? run_start[lo + 1] : p.rows_host;
  it.row0 = start + (j - it.first) * p.ks_rows;
  int rows = end - it.row0;
  rows = rows < 0 ? 0 : (rows > p.ks_rows ? p.ks_rows : rows);
  it.num_k = (rows + BK - 1) / BK;
  return it;
}

// Persistent: one CTA per SM walks the list of (work item, m tile, n chunk); the accumulator is
// double-buffered in TMEM so a tile's store overlaps the next tile's loads and MMAs.
template <int BN, int STAGES, int GATHER>  // GATHER: 0 none, 1 = A gathered, 2 = B gathered
__global__ void __launch_bounds__(GATHER ? WGRAD_THREADS_GATHER : WGRAD_THREADS, 1)
    wgrad_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmAlt, const WgradArgs p, int tiles_x,
                      int tiles_y) {
  pdl_trigger();   // (the wait for the preceding kernels comes after the part of the prologue
                   // that reads nothing of theirs: barriers and TMEM)
  using L = WgradSmem<BN, STAGES>;
  constexpr uint32_t TMEM_BUF = BN <= 128 ? 128 : 256;
  constexpr uint32_t TMEM_COLS = 2 * TMEM_BUF;
  static_assert(BN % 64 == 0 && BN <= 256, "BN must be a multiple of 64 up to 256");

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
  constexpr bool gather = GATHER != 0;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (warp == 2) {
    pdl_wait();   // the run table is the dispatch's
    wgrad_build_table(p, lane, first_item, run_start);
    // the reduction pass reads the item counts from global memory instead of rebuilding them
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
      // a gathered operand: every lane of warp 0 arrives (through its cp.async) next to the TMA
      mbar_init(full_bar + s, gather ? GATHER_WARPS * 32 + 1 : 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + b, 1);
      mbar_init(tempty_bar + b, EPI_WARPS);
    }
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
  pdl_wait();      // every thread, before its first read of an earlier kernel's data
  const uint32_t tmem_base = *tmem_slot;
  const int tiles_xy = tiles_x * tiles_y;
  const int n_items = first_item[p.n_groups];
  const int total = n_items * tiles_xy;  // t = position in the walk order * tiles_xy + tile
  // walk order: items by decreasing length, ties by index (the same permutation in every CTA)
  int* order = reinterpret_cast<int*>(smem + L::ORDER_OFFSET);
  int* isize = order + WGRAD_SORT_MAX;
  const bool sorted = n_items <= WGRAD_SORT_MAX;
  if (sorted) {
    for (int i = threadIdx.x; i < n_items; i += blockDim.x)
      isize[i] = wgrad_item(p, first_item, run_start, i).num_k;
    __syncthreads();
    for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
      const int mine = isize[i];
      int rank = 0;
      for (int k = 0; k < n_items; ++k) {
        const int other = isize[k];
        rank += (other > mine || (other == mine && k < i)) ? 1 : 0;
      }
      order[rank] = i;
    }
    __syncthreads();
  }
  auto item_at = [&](int pos) { return sorted ? order[pos] : pos; };
  // A CTA's unit of round r: rounds run alternately up and down the CTAs (0..G-1, then G-1..0).
  // The units are in decreasing length, so plain round-robin gave CTA 0 the longest unit of every
  // round (busiest CTA 1.28 x the mean at the bench's skew); the serpentine order gives 1.09 x.
  auto unit_of_round = [&](int rnd) {
    const int g = int(gridDim.x), b = int(blockIdx.x);
    return rnd * g + ((rnd & 1) ? g - 1 - b : b);
  };

  if (warp == 0 || warp >= 2 + EPI_WARPS) {
    // Producers. Plain operands arrive by TMA (warp 0, lane 0). A gathered operand is copied with
    // 16-byte cp.async by four warps (0 and 10..12; a warp only keeps a few loads in flight), 16 of
    // the stage's 64 rows each: row `slot` is row sorted_ids[slot] / top_k of the token-major
    // source, and 64-column groups land as the same swizzled 64 x 64 boxes TMA makes.
    const int gw = warp == 0 ? 0 : warp - (1 + EPI_WARPS);
    if (gather || (warp == 0 && lane == 0)) {
      uint32_t it = 0;
      int pending = -1;  // stage whose cp.async copies are issued but not yet handed over
      for (int rnd = 0; rnd * int(gridDim.x) < total && !*abort_flag; ++rnd) {
        const int t = unit_of_round(rnd);
        if (t >= total) continue;
        const WgradItem w = wgrad_item(p, first_item, run_start, item_at(t / tiles_xy));
        const int txy = t % tiles_xy;
        const int m0 = (txy / tiles_y) * BM, n0 = (txy % tiles_y) * BN;
        const int ga = p.a_grouped ? w.group : 0, gb = p.b_grouped ? w.group : 0;
        constexpr int ROWS_PER_WARP = BK / GATHER_WARPS;  // 16 rows of a stage per producer warp
        // token of row gw*16 + lane of the NEXT stage, fetched one stage ahead of its use
        int next_tok = -1;
        auto fetch_tok = [&](int kt) {
          int tok = -1;
          if (gather && lane < ROWS_PER_WARP && kt < w.num_k) {
            const int pair = __ldg(p.sorted_ids + w.row0 + kt * BK + gw * ROWS_PER_WARP + lane);
            tok = pair < p.n_pairs ? pair / p.top_k : -1;
          }
          return tok;
        };
        next_tok = fetch_tok(0);
        for (int kt = 0; kt < w.num_k; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t use = it / STAGES;
          const int my_tok = next_tok;
          next_tok = fetch_tok(kt + 1);
          if (use > 0 && !mbar_wait(empty_bar + s, (use - 1) & 1, p.status)) {
            *abort_flag = 1;
            atomicExch(p.status, ST_WAIT_TIMEOUT);
          }
          if (gather ? __any_sync(0xffffffffu, *abort_flag) : *abort_flag) break;
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          const int r = w.row0 + kt * BK;
          if (warp == 0 && lane == 0) {
            mbar_expect_tx(full_bar + s, (GATHER == 1 ? 0 : A_STAGE_BYTES) +
                                             (GATHER == 2 ? 0 : L::B_STAGE_BYTES));
            // runs from alt_first_group on (the shared experts) take one operand from the
            // token-major matrix: its row is the slot row minus the start of the run
            const bool alt = p.alt_which != 0 && w.group >= p.alt_first_group;
            const int r_alt = r - run_start[w.group];
            const bool a_alt = alt && p.alt_which == 1, b_alt = alt && p.alt_which == 2;
            const CUtensorMap* ma = a_alt ? &tmAlt : &tmA;
            const CUtensorMap* mb = b_alt ? &tmAlt : &tmB;
            const int ra = a_alt ? r_alt : r, rb = b_alt ? r_alt : r;
            if (GATHER != 1) {
              if (p.a_fused) {
                tma_load_4d(sA, ma, full_bar + s, 0, ra, m0 / 64, a_alt ? 0 : ga);
              } else {
#pragma unroll
                for (int i = 0; i < BM / 64; ++i)
                  tma_load_3d(sA + i * 8192, ma, full_bar + s, m0 + 64 * i, ra, a_alt ? 0 : ga);
              }
            }
            if (GATHER != 2) {
              if (p.b_fused) {
                tma_load_4d(sB, mb, full_bar + s, 0, rb, n0 / 64, b_alt ? 0 : gb);
              } else {
#pragma unroll
                for (int jj = 0; jj < BN / 64; ++jj)
                  tma_load_3d(sB + jj * 8192, mb, full_bar + s, n0 + 64 * jj, rb, b_alt ? 0 : gb);
              }
            }
          }
          if (gather) {
            constexpr int cpr = GATHER == 1 ? BM / 8 : BN / 8;  // 16-byte chunks per row
            const int col0 = GATHER == 1 ? m0 : n0;
            const int width = GATHER == 1 ? p.m_dim : p.n_dim;
            const uint32_t dst0 = smem_u32(GATHER == 1 ? sA : sB);
#pragma unroll
            for (int idx = lane; idx < ROWS_PER_WARP * cpr; idx += 32) {
              const int lr = idx / cpr, c = idx - lr * cpr;
              const int tok = __shfl_sync(0xffffffffu, my_tok, lr);
              const int kr = gw * ROWS_PER_WARP + lr;
              const int col = col0 + c * 8;
              const bool ok = tok >= 0 && col < width;
              const __nv_bfloat16* src = ok ? p.gather_src + int64_t(tok) * width + col
                                            : p.gather_src;
              cp_async_16(dst0 + (c >> 3) * 8192 + kr * 128 + (((c & 7) ^ (kr & 7)) << 4), src,
                          ok ? 16u : 0u);
            }
            // hand over the PREVIOUS stage: its copies have landed after wait_group, the proxy
            // fence makes them visible to the tensor core's async-proxy reads, then arrive
            cp_async_commit();
            if (pending >= 0) {
              cp_async_wait<1>();
              fence_proxy_async();
              mbar_arrive(full_bar + pending);
            }
            pending = s;
          }
        }
      }
      if (gather && pending >= 0) {
        cp_async_wait<0>();
        fence_proxy_async();
        mbar_arrive(full_bar + pending);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      uint32_t it = 0;
      int ju = 0;  // tiles that really used an accumulator buffer so far
      for (int rnd = 0; rnd * int(gridDim.x) < total && !*abort_flag; ++rnd) {
        const int t = unit_of_round(rnd);
        if (t >= total) continue;
        const WgradItem w = wgrad_item(p, first_item, run_start, item_at(t / tiles_xy));
        if (w.num_k == 0) continue;  // empty run: the epilogue writes zeros, no accumulator used
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
          issue_stage_mmas<BN, true, true>(sA, sA + A_STAGE_BYTES, d_tmem, kt == 0);
          umma_commit(empty_bar + s);
        }
        umma_commit(tfull_bar + b);
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    const int ew = warp - 2;
    const int q = warp & 3;
    const int half = ew >> 2;
    const int row = q * 32 + lane;
    constexpr int NCH = BN / 32;
    static_assert(NCH % 2 == 0, "column chunks must split evenly over the two epilogue halves");
    const int c_lo = half * (NCH / 2), c_hi = c_lo + NCH / 2;

    int ju = 0;  // tiles that really used an accumulator buffer so far (same count as the MMA warp)
    for (int rnd = 0; rnd * int(gridDim.x) < total; ++rnd) {
      const int t = unit_of_round(rnd);
      if (t >= total) continue;
      const int j = item_at(t / tiles_xy), txy = t % tiles_xy;
      const WgradItem w = wgrad_item(p, first_item, run_start, j);
      const int m0 = (txy / tiles_y) * BM, n0 = (txy % tiles_y) * BN;
      const bool have_acc = w.num_k > 0;
      // The MMA warp skips empty runs without touching a buffer, so the epilogue neither waits
      // nor arrives for them: buffer choice and barrier phases count real uses only.
      const int b = ju & 1;
      if (have_acc) {
        if (!mbar_wait(tfull_bar + b, (uint32_t(ju) >> 1) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        tc_fence_after();
        ++ju;
      }
      const uint32_t taddr = tmem_base + b * TMEM_BUF + (uint32_t(q * 32) << 16);
      const int m = m0 + row;
      const bool m_ok = m < p.m_dim;
      __nv_bfloat16* dst = (w.group < p.n_out1 ? p.out + int64_t(w.group) * p.m_dim * p.n_dim
                                               : p.out_extra + int64_t(w.group - p.n_out1) *
                                                                   p.m_dim * p.n_dim) +
                           int64_t(m) * p.n_dim + n0;
      float* mine = p.partials + (int64_t(j) * tiles_xy + txy) * (int64_t(BM) * BN);
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
          store_f32x32(mine + (int64_t(c) * BM + row) * 32, v);  // [column chunk][row][32]
        }
      }
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar + b);
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
// n_groups); tiles_x / tiles_y / BN must be those of the first pass, which also left the item
// table in p.item_table.
template <int BN>
__global__ void __launch_bounds__(256)
    wgrad_reduce_kernel(const WgradArgs p, int tiles_x, int tiles_y) {
  pdl_trigger();
  pdl_wait();
  const int tile_xy = blockIdx.x / WGRAD_REDUCE_SPLIT;
  const int slice = blockIdx.x % WGRAD_REDUCE_SPLIT;
  const int tile_m = tile_xy / tiles_y, n0 = (tile_xy % tiles_y) * BN;
  const int64_t tiles_xy = int64_t(tiles_x) * tiles_y;
  constexpr int64_t slot_elems = int64_t(BM) * BN;
  constexpr int vecs = BM * BN / 4;                  // float4 per tile
  constexpr int per_slice = vecs / WGRAD_REDUCE_SPLIT;
  // The runs that were split, in run order (one warp compacts the item table by ballot). A CTA takes
  // every gridDim.y-th of them: the grid is sized for the few runs that can be split, not for one
  // CTA per run (launching thousands of CTAs that leave at once cost more than the sums).
  __shared__ int split_runs[WGRAD_MAX_GROUPS];
  __shared__ int n_split_s;
  if (threadIdx.x < 32) {
    int n = 0;
    for (int base = 0; base < p.n_groups; base += 32) {
      const int g = base + int(threadIdx.x);
      const bool split = g < p.n_groups && __ldg(p.item_table + g + 1) - __ldg(p.item_table + g) > 1;
      const unsigned m = __ballot_sync(0xffffffffu, split);
      if (split) split_runs[n + __popc(m & ((1u << threadIdx.x) - 1u))] = g;
      n += __popc(m);
    }
    if (threadIdx.x == 0) n_split_s = n;
  }
  __syncthreads();
  const int n_split = n_split_s;
  for (int i = blockIdx.y; i < n_split; i += gridDim.y) {
    const int g = split_runs[i];
    const int first = __ldg(p.item_table + g), n_c = __ldg(p.item_table + g + 1) - first;
    for (int f = slice * per_slice + threadIdx.x; f < (slice + 1) * per_slice; f += blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      const float4* src = reinterpret_cast<const float4*>(
                              p.partials + (int64_t(first) * tiles_xy + tile_xy) * slot_elems) + f;
      const int64_t stride4 = tiles_xy * slot_elems / 4;  // float4 between consecutive chunks
      // loads of 8 chunks are issued together (they are independent); the adds stay in chunk order
      int c2 = 0;
      for (; c2 + 8 <= n_c; c2 += 8) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldcs(src + (c2 + u) * stride4);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
        }
      }
      for (; c2 < n_c; ++c2) {
        const float4 v = __ldcs(src + c2 * stride4);
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
        __nv_bfloat16* base = g < p.n_out1 ? p.out + int64_t(g) * p.m_dim * p.n_dim
                                           : p.out_extra + int64_t(g - p.n_out1) * p.m_dim * p.n_dim;
        *reinterpret_cast<uint2*>(base + int64_t(m) * p.n_dim + n) = w;
      }
    }
  }
}

}  // namespace moe
