// Grouped bf16 GEMM for the MoE block on sm_100a: TMA -> 128B-swizzled shared memory ring ->
// tcgen05.mma with the fp32 accumulator in TMEM -> tcgen05.ld epilogue with the stage-specific
// math fused in (SwiGLU, router-weight scale, GLU backward, weight-gradient store).
//
// One CTA computes one 128 x BN output tile. Warp 0 issues TMA loads, warp 1 issues the MMAs and
// owns the TMEM allocation, warps 2..5 run the epilogue (one accumulator row per thread).
//
// Two tile schedules share the body:
//   ROWS  : "row-grouped". A is a [rows, K] activation buffer in expert-sorted slot order (runs padded
//           to 128 rows, so a tile never straddles two experts); the tile's expert picks the B
//           matrix out of a stacked weight tensor. Covers up/gate, down, dHidden and dX.
//   WGRAD : per-expert weight gradient C[e] = A_e^T @ B_e, where A_e, B_e are the expert's run of
//           rows in two slot-ordered buffers; the contraction runs over the run's rows.
#pragma once
#include "ptx.cuh"

namespace moe {

constexpr int BM = 128;  // UMMA M: one TMEM lane per output row
constexpr int BK = 64;   // 64 bf16 = one 128-byte swizzle span
constexpr int A_STAGE_BYTES = BM * BK * 2;

enum GemmMode { MODE_ROWS = 0, MODE_WGRAD = 1 };
enum GemmEpi { EPI_RAW = 0, EPI_GLU = 1, EPI_SCALE = 2, EPI_GLUBWD = 3, EPI_WGRAD = 4 };
enum Act { ACT_SILU = 0, ACT_GELU = 1, ACT_RELU = 2, ACT_SIGMOID = 3, ACT_TANH = 4 };

// Status codes a kernel can leave in the status word (0 = fine).
enum DevStatus { ST_OK = 0, ST_WAIT_TIMEOUT = 1, ST_BAD_EXPERT = 2 };

struct GemmArgs {
  // schedule
  const int32_t* expert_ids;   // ROWS: [tiles] owner of each 128-row block (ignored if fixed_group >= 0)
  const int32_t* n_post_pad;   // ROWS: device scalar, live padded rows
  const int32_t* pad_offsets;  // WGRAD: [G+1] run starts (multiples of 128)
  const int32_t* sorted_ids;   // slot -> pair id, sentinel n_pairs in pad slots (may be null)
  int32_t fixed_group;         // >= 0: every tile uses this group and rows_host rows (shared experts)
  int32_t rows_host;           // row count when fixed_group >= 0
  int32_t n_pairs;             // sentinel value in sorted_ids
  int32_t num_k;               // ROWS: K / 64
  int32_t m_dim, n_dim;        // WGRAD: rows / cols of one C[e]; ROWS: n_dim = valid output cols
  // epilogue
  __nv_bfloat16* out;          // main output
  int64_t ld_out;              // elements between rows of out
  __nv_bfloat16* out2;         // GLUBWD: w * hidden   [rows, H]
  __nv_bfloat16* dtw;          // GLUBWD: d(topk_w) flat [n_pairs] (may be null)
  const __nv_bfloat16* aux;    // GLUBWD: saved [gate | up] pre-activations [rows, 2H]
  const __nv_bfloat16* pair_w; // SCALE / GLUBWD: topk_w flat [n_pairs] (null -> weight 1)
  int32_t act;
  int32_t* status;
};

// MN-major 128B-swizzled operand as TMA lays it down in 64 x 64 boxes: 64 MN elements (128 B) per
// k row, 8 k rows per 1024-byte swizzle atom (SBO), next 64 MN elements one 8 KB box further (LBO);
// one UMMA K step (16) spans two atoms.
#define MN_LBO 8192u
#define MN_SBO 1024u
#define MN_KADV 2048u

__device__ __forceinline__ float act_fwd(float g, int act) {
  switch (act) {
    case ACT_SILU: return g / (1.f + __expf(-g));
    case ACT_GELU: return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
    case ACT_RELU: return fmaxf(g, 0.f);
    case ACT_SIGMOID: return 1.f / (1.f + __expf(-g));
    default: return 2.f / (1.f + __expf(-2.f * g)) - 1.f;
  }
}
__device__ __forceinline__ float act_bwd(float g, int act) {
  switch (act) {
    case ACT_SILU: {
      float s = 1.f / (1.f + __expf(-g));
      return s * (1.f + g * (1.f - s));
    }
    case ACT_GELU:
      return 0.5f * (1.f + erff(g * 0.7071067811865476f)) +
             g * 0.3989422804014327f * __expf(-0.5f * g * g);
    case ACT_RELU: return g > 0.f ? 1.f : 0.f;
    case ACT_SIGMOID: {
      float s = 1.f / (1.f + __expf(-g));
      return s * (1.f - s);
    }
    default: {
      float t = 2.f / (1.f + __expf(-2.f * g)) - 1.f;
      return 1.f - t * t;
    }
  }
}

// 32 fp32 -> 32 bf16, stored as four 16-byte vectors (dst 16-byte aligned).
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float* v) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    d4[q] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}
__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* src, float* v) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 r = __ldg(s4 + q);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&w[i]);
      float2 f = __bfloat1622float2(h);
      v[q * 8 + 2 * i] = f.x;
      v[q * 8 + 2 * i + 1] = f.y;
    }
  }
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], accum, then tmem base + abort flag
  static constexpr int TOTAL = BAR_OFFSET + 8 * (2 * STAGES + 1) + 16;
  static constexpr int DYNAMIC = TOTAL + 1024;  // slack for manual 1024-byte alignment
};

template <int BN, int STAGES, bool A_MN, bool B_MN, int MODE, int EPI>
__global__ void __launch_bounds__(192)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB, const GemmArgs p) {
  using L = GemmSmem<BN, STAGES>;
  constexpr uint32_t TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
  static_assert(BN % 64 == 0 && BN <= 256, "BN must be a multiple of 64 up to 256");

  // ------------------------------------------------------------ schedule (before any barrier)
  const int tile_m = blockIdx.x;
  const int n0 = blockIdx.y * BN;
  int group, num_k, row_begin = 0;
  if constexpr (MODE == MODE_ROWS) {
    const int live = p.fixed_group >= 0 ? p.rows_host : __ldg(p.n_post_pad);
    if (tile_m * BM >= live) return;
    group = p.fixed_group >= 0 ? p.fixed_group : __ldg(p.expert_ids + tile_m);
    num_k = p.num_k;
  } else {
    group = blockIdx.z;
    if (p.pad_offsets != nullptr) {
      row_begin = __ldg(p.pad_offsets + group);
      num_k = (__ldg(p.pad_offsets + group + 1) - row_begin) / BK;
    } else {  // one group spanning rows [0, rows_host); the ragged tail reads as zeros
      num_k = (p.rows_host + BK - 1) / BK;
    }
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      for (int kt = 0; kt < num_k; ++kt) {
        const int s = kt % STAGES;
        if (kt >= STAGES && !mbar_wait(empty_bar + s, ((kt / STAGES) - 1) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        if (*abort_flag) break;
        uint8_t* sA = smem + s * L::STAGE_BYTES;
        uint8_t* sB = sA + A_STAGE_BYTES;
        mbar_expect_tx(full_bar + s, L::STAGE_BYTES);
        const int k0 = kt * BK;
        if constexpr (MODE == MODE_ROWS) {
          static_assert(MODE != MODE_ROWS || !A_MN, "row-grouped A is K-major");
          tma_load_2d(sA, &tmA, full_bar + s, k0, tile_m * BM);
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * 8192, &tmB, full_bar + s, n0 + 64 * j, k0, group);
          } else {
            tma_load_3d(sB, &tmB, full_bar + s, k0, n0, group);
          }
        } else {
#pragma unroll
          for (int i = 0; i < BM / 64; ++i)
            tma_load_2d(sA + i * 8192, &tmA, full_bar + s, tile_m * BM + 64 * i, row_begin + k0);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(sB + j * 8192, &tmB, full_bar + s, n0 + 64 * j, row_begin + k0);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, A_MN, B_MN);
      for (int kt = 0; kt < num_k; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(full_bar + s, (kt / STAGES) & 1, p.status)) {
          *abort_flag = 1;
          atomicExch(p.status, ST_WAIT_TIMEOUT);
          break;
        }
        if (*abort_flag) break;
        tc_fence_after();
        const uint32_t sA = smem_u32(smem + s * L::STAGE_BYTES);
        const uint32_t sB = sA + A_STAGE_BYTES;
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; ++k16) {
          const uint64_t da = A_MN ? umma_desc(sA + k16 * MN_KADV, MN_LBO, MN_SBO)
                                   : umma_desc(sA + k16 * 32, 16, 1024);
          const uint64_t db = B_MN ? umma_desc(sB + k16 * MN_KADV, MN_LBO, MN_SBO)
                                   : umma_desc(sB + k16 * 32, 16, 1024);
          umma_f16(tmem_base, da, db, idesc, (kt | k16) != 0);
        }
        umma_commit(empty_bar + s);  // stage reusable once these MMAs have read it
      }
      umma_commit(accum_bar);
    }
  } else {
    // ---------------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int row = q * 32 + lane;
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
    bool have_acc = num_k > 0;
    if (have_acc) {
      if (!mbar_wait(accum_bar, 0, p.status)) {
        *abort_flag = 1;
        atomicExch(p.status, ST_WAIT_TIMEOUT);
        have_acc = false;
      }
      tc_fence_after();
    }
    const bool ok = !*abort_flag;

    if constexpr (EPI == EPI_WGRAD) {
      const int m = tile_m * BM + row;
      __nv_bfloat16* dst =
          p.out + (int64_t(group) * p.m_dim + m) * int64_t(p.n_dim) + n0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        if (have_acc) {
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        if (ok && m < p.m_dim && n0 + c * 32 < p.n_dim) store_bf16x32(dst + c * 32, v);
      }
    } else {
      const int64_t grow = int64_t(tile_m) * BM + row;
      const bool row_ok = ok && (p.fixed_group < 0 || grow < p.rows_host);
      int pair = p.n_pairs;
      if (p.sorted_ids != nullptr && p.fixed_group < 0) pair = __ldg(p.sorted_ids + grow);
      float w = 1.f;
      if (p.pair_w != nullptr) w = pair < p.n_pairs ? __bfloat162float(p.pair_w[pair]) : 0.f;

      if constexpr (EPI == EPI_GLU) {
        static_assert(EPI != EPI_GLU || BN == 256 || BN == 128 || BN == 64, "GLU tile");
        constexpr int HALF = BN / 2;  // gate = cols [0, HALF), up = cols [HALF, BN)
#pragma unroll 1
        for (int c = 0; c < HALF / 32; ++c) {
          float g[32], u[32];
          tmem_ld32(taddr + c * 32, g);
          tmem_ld32(taddr + HALF + c * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = act_fwd(g[i], p.act) * u[i];
          if (row_ok) store_bf16x32(p.out + grow * p.ld_out + c * 32, g);
        }
      } else if constexpr (EPI == EPI_RAW || EPI == EPI_SCALE) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          if constexpr (EPI == EPI_SCALE) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= w;
          }
          if (row_ok && n0 + c * 32 < p.n_dim) store_bf16x32(p.out + grow * p.ld_out + n0 + c * 32, v);
        }
      } else if constexpr (EPI == EPI_GLUBWD) {
        // acc = G = dOut @ W_out^T for this row; aux = [gate | up]; H = BN.
        const __nv_bfloat16* a1 = p.aux + grow * (2 * BN);
        __nv_bfloat16* da1 = p.out + grow * (2 * BN);
        __nv_bfloat16* hw = p.out2 + grow * BN;
        float part = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float G[32], g[32], u[32];
          tmem_ld32(taddr + c * 32, G);
          if (row_ok) {
            load_bf16x32(a1 + c * 32, g);
            load_bf16x32(a1 + BN + c * 32, u);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) g[i] = u[i] = 0.f;
          }
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float a = act_fwd(g[i], p.act);
            const float hid = a * u[i];
            part += G[i] * hid;
            const float dh = w * G[i];
            g[i] = dh * u[i] * act_bwd(g[i], p.act);  // d gate
            u[i] = dh * a;                             // d up
            G[i] = w * hid;                            // weighted hidden for dW_out
          }
          if (row_ok) {
            store_bf16x32(da1 + c * 32, g);
            store_bf16x32(da1 + BN + c * 32, u);
            store_bf16x32(hw + c * 32, G);
          }
        }
        if (row_ok && p.dtw != nullptr && pair < p.n_pairs) p.dtw[pair] = __float2bfloat16(part);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace moe
