// Persistent row-grouped GEMM (see gemm.cuh). 320 threads: warp 0 TMA, warp 1 MMA, warps 2..9
// epilogue (two warps per TMEM lane quadrant, each taking half of the tile's column chunks).
#pragma once

namespace moe {

constexpr int ROWS_THREADS = 320;
constexpr int EPI_WARPS = 8;
// A gathered with cp.async needs many loads in flight, and a warp only keeps a few outstanding:
// three more producer warps (10..12) join warp 0, each copying 32 of a stage's 128 rows.
constexpr int GATHER_WARPS = 4;
constexpr int ROWS_THREADS_GATHER = ROWS_THREADS + (GATHER_WARPS - 1) * 32;
// The GLU-backward epilogue reads a tile of pre-activations [128 x 2 BN]: one more warp brings it
// into shared memory by TMA one tile ahead (with per-thread global loads the epilogue waited for
// them tile after tile: dHidden took 77 us with those loads, 50 us without).
__host__ __device__ constexpr bool epi_loads_aux(int epi) { return epi == EPI_GLUBWD; }
// The reducing epilogues hand their staged tiles to RED_WARPS more warps, which issue the atomic
// adds: those stall on the L2's atomic throughput, and the epilogue warps would otherwise stand
// still with them instead of draining the next accumulator.
constexpr int RED_WARPS = 4;
__host__ __device__ constexpr bool epi_reduces(int epi) {
  return epi == EPI_RAW_RED || epi == EPI_SCALE_RED;
}
__host__ __device__ constexpr int rows_threads(int epi, bool gather) {
  return (gather ? ROWS_THREADS_GATHER : ROWS_THREADS) + (epi_loads_aux(epi) ? 32 : 0) +
         (epi_reduces(epi) ? RED_WARPS * 32 : 0);
}

// Epilogues that leave through TMA stage the tile in shared memory one 64-column box (128 rows x
// 128 bytes, swizzled) at a time, in OUT_BOXES buffers used in turn.
constexpr int OUT_BOX_BYTES = BM * 128;
__host__ __device__ constexpr bool epi_uses_tma_store(int epi) {
  return epi == EPI_RAW || epi == EPI_SCALE;
}
// Epilogues that reduce into a token-major matrix stage the whole tile row by row (BN bf16 + 16
// bytes of padding per row, so that the 32 rows a warp writes at once spread over all banks) in
// OUT_BOXES buffers used in turn; the reducer warps read them back as whole rows.
__host__ __device__ constexpr int red_row_bytes(int bn) { return bn * 2 + 16; }
// OUT_BOXES = number of staging boxes. The stores are asynchronous: the epilogue warps only wait when a buffer
// comes round again, so the boxes in flight are what keeps HBM writing while the warps already
// work on the next tile. (With direct stores, and with two boxes, the time to write the output
// simply added to the rest of the kernel: down GEMM 24 us without its stores, 47 us with them.)

template <int BN, int STAGES, int EPI = EPI_GLU, int OUT_BOXES = 4>
struct RowsSmem {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;  // 1024-byte aligned
  static constexpr int RED_TILE_BYTES = (BM * red_row_bytes(BN) + 1023) / 1024 * 1024;
  static constexpr int STAGING_BYTES = epi_uses_tma_store(EPI) ? OUT_BOXES * OUT_BOX_BYTES
                                       : epi_reduces(EPI)      ? OUT_BOXES * RED_TILE_BYTES
                                                               : 0;
  static constexpr int AUX_OFFSET = STAGING_OFFSET + STAGING_BYTES;  // 1024-byte aligned
  static constexpr int AUX_TILE_BYTES = BM * 2 * BN * 2;             // [128 x 2 BN] bf16
  // (for the aux-loading epilogue OUT_BOXES is the number of pre-activation buffers, 1 or 2)
  static constexpr int AUX_BUFS = OUT_BOXES >= 2 ? 2 : 1;
  static constexpr int BAR_OFFSET = AUX_OFFSET + (epi_loads_aux(EPI) ? AUX_BUFS * AUX_TILE_BYTES : 0);
  // full, empty, tmem_full[2], tmem_empty[2], aux_full[2], aux_empty[2]
  static constexpr int N_BARS = 2 * STAGES + 8;
  static constexpr int MISC_OFFSET = BAR_OFFSET + 8 * N_BARS;      // tmem slot, abort flag
  static constexpr int PART_OFFSET = MISC_OFFSET + 16;             // float[128] dtw partials
  static constexpr int TOK_OFFSET = PART_OFFSET + 128 * 4;         // int[128] gathered row ids
  static constexpr int RED_TOK_OFFSET = TOK_OFFSET + 128 * 4;      // int[OUT_BOXES][128] tokens of the staged rows
  static constexpr int TOTAL = RED_TOK_OFFSET + (epi_reduces(EPI) ? OUT_BOXES * 128 * 4 : 0);
  static constexpr int DYNAMIC = TOTAL + 1024;  // slack for manual 1024-byte alignment
};

struct TileCoord {
  int m_tile, n0, group, z;
};

// t -> (group slice z, 128-row block, N chunk); N chunks of one row block are adjacent so its A
// tile is still in L2 for the next chunk.
__device__ __forceinline__ TileCoord decode_tile(const RowsArgs& p, int t, int m_tiles, int bn,
                                                 bool want_group = true) {
  TileCoord c;
  const int nc = t % p.n_chunks;
  const int rest = t / p.n_chunks;
  c.m_tile = rest % m_tiles;
  c.z = rest / m_tiles;
  c.n0 = nc * bn;
  c.group = !want_group ? -1 : p.n_fixed_groups > 0 ? c.z : __ldg(p.expert_ids + c.m_tile);
  return c;
}
// The owner of tile t alone (-1 past the end of the list). The producers ask for the next tile's
// owner while they work on the current one: the lookup is a global load whose latency would
// otherwise sit at the head of every tile.
__device__ __forceinline__ int tile_group(const RowsArgs& p, int t, int m_tiles, int total_tiles) {
  if (t >= total_tiles) return -1;
  const int rest = t / p.n_chunks;
  return p.n_fixed_groups > 0 ? rest / m_tiles : __ldg(p.expert_ids + rest % m_tiles);
}

// v[0..31] += bias[0..31] (bf16, 16-byte aligned; the same address in every lane: a broadcast load)
__device__ __forceinline__ void add_bias32(float* v, const __nv_bfloat16* bias) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(bias) + i);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
      v[8 * i + 2 * k] += f.x;
      v[8 * i + 2 * k + 1] += f.y;
    }
  }
}

template <int ACT, int BN>
__device__ __forceinline__ void epilogue_glu(uint32_t taddr, int c_lo, int c_hi, bool row_ok,
                                             __nv_bfloat16* out_row, __nv_bfloat16* raw_row,
                                             const __nv_bfloat16* bias) {
  constexpr int HALF = BN / 2;  // gate = accumulator cols [0, HALF), up = [HALF, BN)
#pragma unroll 1
  for (int c = c_lo; c < c_hi; ++c) {
    float g[32], u[32];
    tmem_ld32(taddr + c * 32, g);
    tmem_ld32(taddr + HALF + c * 32, u);
    tmem_ld_wait();
    if (bias != nullptr) {   // the kept pre-activations include it, as the backward expects
      add_bias32(g, bias + c * 32);
      add_bias32(u, bias + HALF + c * 32);
    }
    if (raw_row != nullptr && row_ok) {
      store_bf16x32(raw_row + c * 32, g);
      store_bf16x32(raw_row + HALF + c * 32, u);
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) g[i] = act_f<ACT>(g[i]) * u[i];
    if (row_ok) store_bf16x32(out_row + c * 32, g);
  }
}

// 32 bf16 of row `row`, columns [col, col + 32), from a tile that TMA loaded as 64-column boxes of
// 128 rows (128-byte swizzle): four 16-byte pieces at their swizzled positions.
__device__ __forceinline__ void load_tile_bf16x32(uint32_t tile, int row, int col, float* v) {
  const uint32_t base = tile + (col >> 6) * OUT_BOX_BYTES + row * 128;
  const int piece0 = (col & 63) >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t w[4];
    ld_shared_v4(base + (((piece0 + i) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[k]));
      v[8 * i + 2 * k] = f.x;
      v[8 * i + 2 * k + 1] = f.y;
    }
  }
}

// acc = G = dOut @ W_out^T for this row; a1_tile = the tile's [gate | up] pre-activations in shared
// memory; H = BN. Returns this thread's share of <G, hidden>.
template <int ACT, int BN>
__device__ __forceinline__ float epilogue_glubwd(uint32_t taddr, int c_lo, int c_hi, bool row_ok,
                                                 float w, uint32_t a1_tile, int row,
                                                 __nv_bfloat16* da1, __nv_bfloat16* hw) {
  float part = 0.f;
#pragma unroll 1
  for (int c = c_lo; c < c_hi; ++c) {
    float G[32], g[32], u[32];
    tmem_ld32(taddr + c * 32, G);
    load_tile_bf16x32(a1_tile, row, c * 32, g);
    load_tile_bf16x32(a1_tile, row, BN + c * 32, u);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float a, d;
      act_fd<ACT>(g[i], a, d);
      const float hid = a * u[i];
      part += G[i] * hid;
      const float dh = w * G[i];
      g[i] = dh * u[i] * d;  // d gate
      u[i] = dh * a;         // d up
      G[i] = w * hid;        // weighted hidden, the A operand of dW_out
    }
    if (row_ok) {
      store_bf16x32(da1 + c * 32, g);
      store_bf16x32(da1 + BN + c * 32, u);
      store_bf16x32(hw + c * 32, G);
    }
  }
  return part;
}

template <int BN, int STAGES, bool B_MN, int EPI, bool GATHER_A, int OUT_BOXES = 4>
__global__ void __launch_bounds__(rows_threads(EPI, GATHER_A), 1)
    rows_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmA2,
                     const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmB2,
                     const __grid_constant__ CUtensorMap tmOut, const RowsArgs p) {
  // The prologue below (barriers, TMEM, descriptor prefetch) touches nothing an earlier kernel
  // wrote, so it runs BEFORE the wait for the preceding kernels: under programmatic dependent launch
  // this CTA is resident while the previous grid's last CTAs still work.
  pdl_trigger();
  using L = RowsSmem<BN, STAGES, EPI, OUT_BOXES>;
  constexpr bool TMA_OUT = epi_uses_tma_store(EPI);
  static_assert(BN % 64 == 0 && BN <= 256, "BN must be a multiple of 64 up to 256");
  constexpr uint32_t TMEM_BUF = BN <= 128 ? 128 : 256;  // columns per accumulator buffer
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
  constexpr int AUX_WARP = 2 + EPI_WARPS + (GATHER_A ? GATHER_WARPS - 1 : 0);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::MISC_OFFSET);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* dtw_part = reinterpret_cast<float*>(smem + L::PART_OFFSET);
  int* tok_s = reinterpret_cast<int*>(smem + L::TOK_OFFSET);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmA2);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmB2);
    if constexpr (TMA_OUT) tma_prefetch_desc(&tmOut);
    for (int s = 0; s < STAGES; ++s) {
      // gathered A: every lane of warp 0 arrives (through its cp.async) next to the TMA transaction
      mbar_init(full_bar + s, GATHER_A ? GATHER_WARPS * 32 + 1 : 1);
      mbar_init(empty_bar + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + b, 1);
      mbar_init(tempty_bar + b, EPI_WARPS);
      // (the reducing epilogues use this pair for their staging buffers: filled by the epilogue
      // warps, drained by the reducer warps)
      mbar_init(afull_bar + b, epi_reduces(EPI) ? EPI_WARPS : 1);
      mbar_init(aempty_bar + b, epi_reduces(EPI) ? RED_WARPS : EPI_WARPS);
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
  const uint32_t tmem_base = *tmem_slot;

  // ------------------------------------------------------------ tile list
  // (every thread waits for the preceding kernels itself before its first read of their data; a
  // CTA beyond the end of the list runs no loop iteration and only gives its TMEM back)
  pdl_wait();
  const int live = p.n_fixed_groups > 0 ? p.rows_host : __ldg(p.n_post_pad);
  const int m_tiles = (live + BM - 1) / BM;
  const int total_tiles = m_tiles * p.n_chunks * (p.n_fixed_groups > 0 ? p.n_fixed_groups : 1);

  if (AUX_IN && warp == AUX_WARP) {
    // ------------------------------------------------ pre-activation tiles for the epilogue
    if (elect_one()) {
      int j = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x, ++j) {
        const TileCoord tc = decode_tile(p, t, m_tiles, BN);
        const int b = j % L::AUX_BUFS;
        const uint32_t use = uint32_t(j) / L::AUX_BUFS;
        if (use > 0 && !mbar_wait(aempty_bar + b, (use - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        uint8_t* dst = smem + L::AUX_OFFSET + b * L::AUX_TILE_BYTES;
        mbar_expect_tx(afull_bar + b, L::AUX_TILE_BYTES);
#pragma unroll
        for (int i = 0; i < 2 * BN / 64; ++i)  // 64-column boxes of [gate | up], rows past the end read 0
          tma_load_3d(dst + i * OUT_BOX_BYTES, &tmOut, afull_bar + b, 64 * i, tc.m_tile * BM, tc.z);
      }
    }
  } else if (GATHER_A && (warp == 0 || (warp >= 2 + EPI_WARPS && warp != AUX_WARP))) {
    // --------------------------------- producers, gathered A: four warps copy 32 rows each
    // Lane (r4 = lane / 8, c = lane % 8) moves 16-byte chunk c of rows r4, r4 + 4, ... of its
    // warp's 32 rows: eight lanes cover one row's 128-byte k slice, so global reads are whole
    // lines. The chunk lands at (c ^ (row & 7)), the 128-byte swizzle the UMMA descriptor expects.
    // Warp 0's lane 0 also issues the TMA loads of B.
    // Completion protocol: a lane's copies of stage i are known to have landed after
    // cp.async.wait_group; the lane then makes them visible to the async proxy (the tensor core
    // reads shared memory through it) with fence.proxy.async and arrives on the stage's barrier.
    // That hand-over trails the issue loop by one stage so the wait is normally already over.
    const int gw = warp == 0 ? 0 : warp - (1 + EPI_WARPS);
    uint32_t it = 0;
    int pending = -1;  // stage whose copies are issued but not yet handed over
    const int r4 = lane >> 3, c = lane & 7;
    int group_next = tile_group(p, blockIdx.x, m_tiles, total_tiles);
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      TileCoord tc = decode_tile(p, t, m_tiles, BN);
      tc.group = group_next;
      group_next = tile_group(p, t + gridDim.x, m_tiles, total_tiles);
      const int pair = __ldg(p.sorted_ids + int64_t(tc.m_tile) * BM + gw * 32 + lane);
      const int my_tok = pair < p.n_pairs ? pair / p.top_k : -1;  // token of row gw*32 + lane
      for (int kt = 0; kt < p.num_k; ++kt, ++it) {
        const int s = it % STAGES;
        const uint32_t use = it / STAGES;
        if (use > 0 && !mbar_wait(empty_bar + s, (use - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        }
        if (__any_sync(0xffffffffu, *abort_flag)) break;
        uint8_t* sA = smem + s * L::STAGE_BYTES;
        uint8_t* sB = sA + A_STAGE_BYTES;
        const int k0 = kt * BK;
        if (warp == 0 && lane == 0) {
          mbar_expect_tx(full_bar + s, L::B_STAGE_BYTES);
          // the tile's expert lives in the first weight stack or (shared experts) the second
          const bool first = tc.group < p.n_groups_b1;
          const CUtensorMap* mb = first ? &tmB : &tmB2;
          const int gb = first ? tc.group : tc.group - p.n_groups_b1;
          if constexpr (B_MN) {
            if (p.b_fused) {
              tma_load_4d(sB, mb, full_bar + s, 0, k0, tc.n0 / 64, gb);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sB + j * 8192, mb, full_bar + s, tc.n0 + 64 * j, k0, gb);
            }
          } else {
            tma_load_3d(sB, mb, full_bar + s, k0, tc.n0, gb);
          }
        }
        const int col = k0 + c * 8;
        const bool col_ok = col < p.a_cols;
        const uint32_t sA_u = smem_u32(sA);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int lrow = i * 4 + r4;
          const int tok = __shfl_sync(0xffffffffu, my_tok, lrow);
          const int row = gw * 32 + lrow;
          const bool ok = tok >= 0 && col_ok;
          const __nv_bfloat16* src = ok ? p.a_src + int64_t(tok) * p.a_cols + col : p.a_src;
          cp_async_16(sA_u + row * 128 + ((c ^ (row & 7)) << 4), src, ok ? 16u : 0u);
        }
        cp_async_commit();
        if (pending >= 0) {
          cp_async_wait<1>();
          fence_proxy_async();
          mbar_arrive(full_bar + pending);
        }
        pending = s;
      }
    }
    if (pending >= 0) {
      cp_async_wait<0>();
      fence_proxy_async();
      mbar_arrive(full_bar + pending);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      // Groups from a2_first_group on (the shared experts: every token, in token order) have no
      // rows in the slot-ordered buffer; their A rows are the token-major source itself, row =
      // slot - start of the group's run. The run start is fetched with the next tile's owner.
      auto run_start_of = [&](int group) {
        return (group >= p.a2_first_group && group >= 0) ? __ldg(p.a2_offsets + group) : 0;
      };
      int group_next = tile_group(p, blockIdx.x, m_tiles, total_tiles);
      int start_next = run_start_of(group_next);
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        TileCoord tc = decode_tile(p, t, m_tiles, BN);
        tc.group = group_next;
        const int a_start = start_next;
        const bool a_alt = tc.group >= p.a2_first_group;
        group_next = tile_group(p, t + gridDim.x, m_tiles, total_tiles);
        start_next = run_start_of(group_next);
        const int k_total = p.sum_groups > 0 ? p.sum_groups * p.num_k : p.num_k;
        for (int kt = 0; kt < k_total; ++kt, ++it) {
          const int s = it % STAGES;
          const uint32_t use = it / STAGES;
          if (use > 0 && !mbar_wait(empty_bar + s, (use - 1) & 1, p.status)) {
            *abort_flag = 1;
            atomicExch(p.status, ST_WAIT_TIMEOUT);
            break;
          }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + A_STAGE_BYTES;
          mbar_expect_tx(full_bar + s, L::STAGE_BYTES);
          const int g_sum = p.sum_groups > 0 ? kt / p.num_k : 0;
          const int k0 = (kt - g_sum * p.num_k) * BK;
          if (p.sum_groups > 0)
            tma_load_3d(sA, &tmA, full_bar + s, k0,
                        tc.m_tile * BM + __ldg(p.sum_offsets + g_sum), 0);
          else if (a_alt)
            tma_load_3d(sA, &tmA2, full_bar + s, k0, tc.m_tile * BM - a_start, 0);
          else
            tma_load_3d(sA, &tmA, full_bar + s, k0, tc.m_tile * BM, p.a_grouped ? tc.z : 0);
          // the tile's expert lives in the first weight stack or (shared experts) the second
          const bool first = tc.group < p.n_groups_b1;
          const CUtensorMap* mb = first ? &tmB : &tmB2;
          const int gb = p.sum_groups > 0 ? g_sum
                                          : first ? tc.group : tc.group - p.n_groups_b1;
          if constexpr (B_MN) {
            if (p.b_fused) {
              tma_load_4d(sB, mb, full_bar + s, 0, k0, tc.n0 / 64, gb);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sB + j * 8192, mb, full_bar + s, tc.n0 + 64 * j, k0, gb);
            }
          } else {
            tma_load_3d(sB, mb, full_bar + s, k0, tc.n0, gb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t it = 0;
      int j = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x, ++j) {
        const int b = j & 1;
        const uint32_t use = uint32_t(j) >> 1;
        if (use > 0 && !mbar_wait(tempty_bar + b, (use - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + b * TMEM_BUF;
        const int k_total = p.sum_groups > 0 ? p.sum_groups * p.num_k : p.num_k;
        for (int kt = 0; kt < k_total; ++kt, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar + s, (it / STAGES) & 1, p.status)) {
            *abort_flag = 1;
            atomicExch(p.status, ST_WAIT_TIMEOUT);
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * L::STAGE_BYTES);
          issue_stage_mmas<BN, false, B_MN>(sA, sA + A_STAGE_BYTES, d_tmem, kt == 0);
          umma_commit(empty_bar + s);  // stage reusable once these MMAs have read it
        }
        umma_commit(tfull_bar + b);
      }
    }
  } else if (epi_reduces(EPI) && warp >= 2 + EPI_WARPS) {
    // ------------------------------------------------------------------------ reducers
    // Staged tile -> token-major output: thread i takes the 16-byte pieces i, i + 128, ... of the
    // tile in row-major order, so a warp's adds cover whole rows (full lines for the L2's atomic
    // units); red.global is fire-and-forget, the waiting happens in the queues behind it.
    if constexpr (epi_reduces(EPI)) {
      static_assert(OUT_BOXES == 2, "two staging buffers (the barrier pairs are [2])");
      constexpr int ROWB = red_row_bytes(BN);
      int* tok_all = reinterpret_cast<int*>(smem + L::RED_TOK_OFFSET);
      const uint64_t keep = l2_policy_evict_last();
      int j = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++j) {
        const TileCoord tc = decode_tile(p, t, m_tiles, BN, false);
        const int b = j & 1;
        if (!mbar_wait(afull_bar + b, (uint32_t(j) >> 1) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        const int ncols = min(BN, p.n_dim - tc.n0);   // a multiple of 32
        const int ppr = ncols >> 3;                   // 16-byte pieces per row (<= 32)
        const uint32_t stg = smem_u32(smem + L::STAGING_OFFSET + b * L::RED_TILE_BYTES);
        const int* toks = tok_all + b * BM;
        __nv_bfloat16* dst0 = p.out + tc.n0 + lane * 8;
        // A warp takes every RED_WARPS-th row. The adds leave an SM through two independent
        // paths, each good for about 16 bytes per clock: vector red instructions (load/store
        // unit) and bulk reductions (copy engine). The rows are split between the two: of a
        // warp's 32 rows the odd ones go as one bulk reduction each (lane l issues row l's), the
        // even ones as red instructions, lane l piece l of the row, RED_UNROLL rows loaded before
        // the first add is issued.
        constexpr int RED_UNROLL = 8;
        constexpr int STEP = 2 * RED_WARPS;   // distance between two rows of the same kind
        static_assert(BM % (STEP * RED_UNROLL) == 0, "rows per reducer warp");
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
          for (int u = 0; u < RED_UNROLL; ++u) {
            const int r = r0 + u * STEP;
            tk[u] = lane < ppr ? toks[r] : -1;
            ld_shared_v4(stg + r * ROWB + (lane < ppr ? lane : 0) * 16, w[u][0], w[u][1], w[u][2],
                         w[u][3]);
          }
#pragma unroll
          for (int u = 0; u < RED_UNROLL; ++u)
            if (tk[u] >= 0)
              red_add_bf16x8(dst0 + int64_t(tk[u]) * p.ld_out, w[u][0], w[u][1], w[u][2], w[u][3],
                             keep);
        }
        bulk_wait_read<0>();   // the copy engine has read this thread's rows: the buffer may go back
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty_bar + b);
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ---------------------------------------------------------------------- epilogue
    const int ew = warp - 2;
    const int q = warp & 3;   // TMEM lane quadrant this warp may read
    const int half = ew >> 2; // which half of the column chunks
    const int row = q * 32 + lane;
    constexpr int NCH = (EPI == EPI_GLU ? BN / 2 : BN) / 32;
    static_assert(NCH % 2 == 0, "column chunks must split evenly over the two epilogue halves");
    const int c_lo = half * (NCH / 2), c_hi = c_lo + NCH / 2;

    // This row's pair id and router weight are two dependent global loads: they are issued two
    // tiles / one tile ahead so that their latency is spent under the previous tiles' work.
    const bool fixed = p.n_fixed_groups > 0;
    auto load_pair = [&](int t) {
      if (t >= total_tiles || fixed || p.sorted_ids == nullptr) return p.n_pairs;
      return __ldg(p.sorted_ids + int64_t((t / p.n_chunks) % m_tiles) * BM + row);
    };
    auto load_w = [&](int pr) {
      if (p.pair_w == nullptr) return 1.f;
      return pr < p.n_pairs ? __bfloat162float(__ldg(p.pair_w + pr)) : 0.f;
    };
    int pair = load_pair(blockIdx.x);
    int pair_n = load_pair(blockIdx.x + gridDim.x);
    float w = load_w(pair);

    int j = 0;
    [[maybe_unused]] uint32_t box_count = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++j) {
      const TileCoord tc = decode_tile(p, t, m_tiles, BN, false);
      const int b = j & 1;
      const float w_n = load_w(pair_n);                    // next tile's weight
      const int pair_nn = load_pair(t + 2 * gridDim.x);    // the pair id of the tile after that
      // A wait that gives up (status already flagged) falls through: the epilogue keeps its
      // barrier protocol intact and the host sees the status word.
      if (!mbar_wait(tfull_bar + b, (uint32_t(j) >> 1) & 1, p.status))
        atomicExch(p.status, ST_WAIT_TIMEOUT);
      tc_fence_after();
      const uint32_t taddr = tmem_base + b * TMEM_BUF + (uint32_t(q * 32) << 16);

      const int64_t grow = int64_t(tc.m_tile) * BM + row;
      const bool row_ok = !fixed || grow < p.rows_host;
      __nv_bfloat16* out_row = p.out + tc.z * p.out_gstride + grow * p.ld_out;

      // this tile's bias row
      // (the tile's owner is looked up only when there is a bias: the epilogue has no other use
      // for it, and the load would sit at the head of every tile)
      [[maybe_unused]] const __nv_bfloat16* bias_row = nullptr;
      if constexpr (EPI == EPI_GLU || EPI == EPI_SCALE || EPI == EPI_SCALE_RED) {
        if (p.bias != nullptr) {
          const int grp = fixed ? tc.z : __ldg(p.expert_ids + tc.m_tile);
          bias_row = p.bias + int64_t(grp) * p.n_dim;   // one row per group of both weight stacks
        }
      }
      if constexpr (EPI == EPI_GLU) {
        __nv_bfloat16* raw_row =
            p.out2 ? p.out2 + tc.z * p.out2_gstride + grow * BN : nullptr;
        switch (p.act) {
          case ACT_SILU: epilogue_glu<ACT_SILU, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          case ACT_GELU: epilogue_glu<ACT_GELU, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          case ACT_RELU: epilogue_glu<ACT_RELU, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          case ACT_SIGMOID: epilogue_glu<ACT_SIGMOID, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
          default: epilogue_glu<ACT_TANH, BN>(taddr, c_lo, c_hi, row_ok, out_row, raw_row, bias_row); break;
        }
      } else if constexpr (EPI == EPI_RAW || EPI == EPI_SCALE) {
        // The tile leaves as 64-column boxes: the eight warps fill one box in shared memory (warp
        // half h converts accumulator columns 32h..32h+31 of the box for its 32 rows, 16-byte
        // pieces at the swizzled position a TMA load would have put them), then one thread hands
        // the box to TMA, whose stores are whole 128-byte lines. OUT_BOXES buffers take turns;
        // before a buffer is filled again the issuing thread has waited for the store that last
        // read it.
        const bool issuer = warp == 2 && lane == 0;
        constexpr int NB = BN / 64;
        float v[2][32];  // the next box's accumulator columns are in flight while this one is packed
        tmem_ld32(taddr + half * 32, v[0]);
#pragma unroll
        for (int jb = 0; jb < NB; ++jb, ++box_count) {
          tmem_ld_wait();
          if (jb + 1 < NB) tmem_ld32(taddr + (jb + 1) * 64 + half * 32, v[(jb + 1) & 1]);
          float* cur = v[jb & 1];
          if constexpr (EPI == EPI_SCALE) {
            // (columns past n_dim belong to boxes that are never stored; n_dim is a multiple of 32)
            if (bias_row != nullptr && tc.n0 + jb * 64 + half * 32 < p.n_dim)
              add_bias32(cur, bias_row + tc.n0 + jb * 64 + half * 32);
#pragma unroll
            for (int i = 0; i < 32; ++i) cur[i] *= w;
          }
          const uint32_t buf = smem_u32(smem + L::STAGING_OFFSET + (box_count % OUT_BOXES) * OUT_BOX_BYTES);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t wd[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(cur[8 * i + 2 * k], cur[8 * i + 2 * k + 1]);
              wd[k] = *reinterpret_cast<uint32_t*>(&h2);
            }
            st_shared_v4(buf + row * 128 + (((half * 4 + i) ^ (row & 7)) << 4), wd[0], wd[1], wd[2],
                         wd[3]);
          }
          fence_proxy_async();
          // the buffer filled next was handed to TMA OUT_BOXES - 1 stores ago: wait for that read
          if (issuer) bulk_wait_read<OUT_BOXES - 2>();
          epi_bar_sync(EPI_WARPS * 32);
          if (issuer && tc.n0 + jb * 64 < p.n_dim) {
            tma_store_3d(&tmOut, smem + L::STAGING_OFFSET + (box_count % OUT_BOXES) * OUT_BOX_BYTES,
                         tc.n0 + jb * 64, tc.m_tile * BM, tc.z);
            bulk_commit();
          }
        }
      } else if constexpr (EPI == EPI_RAW_RED || EPI == EPI_SCALE_RED) {
        // The tile is staged row by row in shared memory (bf16, this row's weight and bias
        // applied) with the rows' tokens beside it, and handed to the reducer warps, which add
        // every row to row `token` of the token-major output (bf16 atomics performed in L2). Two
        // staging buffers take turns.
        constexpr int NB = BN / 64;
        constexpr int ROWB = red_row_bytes(BN);
        const int tok = fixed ? (row_ok ? int(grow) : -1)
                              : (pair < p.n_pairs ? pair / p.top_k : -1);
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
        fence_proxy_async();   // the copy engine reads the staged rows through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(afull_bar + b);   // (release: the staged rows are visible)
      } else {  // EPI_GLUBWD
        __nv_bfloat16* da1 = out_row;  // ld_out == 2 * BN
        __nv_bfloat16* hw = p.out2 + tc.z * p.out2_gstride + grow * BN;
        // this tile's pre-activations were brought in by the aux warp
        const int ab = j % L::AUX_BUFS;
        if (!mbar_wait(afull_bar + ab, (uint32_t(j) / L::AUX_BUFS) & 1, p.status))
          atomicExch(p.status, ST_WAIT_TIMEOUT);
        const uint32_t a1_tile = smem_u32(smem + L::AUX_OFFSET + ab * L::AUX_TILE_BYTES);
        float part;
        switch (p.act) {
          case ACT_SILU: part = epilogue_glubwd<ACT_SILU, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          case ACT_GELU: part = epilogue_glubwd<ACT_GELU, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          case ACT_RELU: part = epilogue_glubwd<ACT_RELU, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          case ACT_SIGMOID: part = epilogue_glubwd<ACT_SIGMOID, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
          default: part = epilogue_glubwd<ACT_TANH, BN>(taddr, c_lo, c_hi, row_ok, w, a1_tile, row, da1, hw); break;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(aempty_bar + ab);  // this warp is done with the tile's buffer
        // <G, hidden> of a row is split over the two column halves: fold half 1 into half 0
        // Barrier 1 hands half 1's partials to half 0, barrier 2 hands the buffer back; each half
        // only ever waits for the other one's previous step.
        if (p.dtw != nullptr) {
          if (half == 1) {
            if (j > 0) named_bar_sync(2, EPI_WARPS * 32);
            dtw_part[row] = part;
            named_bar_arrive(1, EPI_WARPS * 32);
          } else {
            named_bar_sync(1, EPI_WARPS * 32);
            if (row_ok && pair < p.n_pairs) p.dtw[pair] = __float2bfloat16(part + dtw_part[row]);
            if (t + int(gridDim.x) < total_tiles) named_bar_arrive(2, EPI_WARPS * 32);
          }
        }
      }
      // this warp has drained its share of accumulator buffer b
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar + b);
      pair = pair_n;
      pair_n = pair_nn;
      w = w_n;
    }
    // shared memory must outlive the last stores' reads
    if constexpr (TMA_OUT) {
      if (warp == 2 && lane == 0) bulk_wait_read<0>();
    }

  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace moe
