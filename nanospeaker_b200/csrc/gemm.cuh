// Grouped bf16 GEMMs of the MoE block on sm_100a: TMA -> 128B-swizzled shared-memory ring ->
// tcgen05.mma with fp32 accumulators in TMEM -> tcgen05.ld epilogues with the stage math fused in
// (SwiGLU, router-weight scale, GLU backward, weight-gradient reduction).
//
// rows_gemm_kernel  : "row-grouped", persistent. A is a [rows, K] activation buffer in expert-sorted
//                     slot order (runs padded to 128 rows, so a 128-row tile never straddles two
//                     experts); the tile's expert picks B out of a stacked weight tensor. One CTA
//                     per SM walks the tile list; the accumulator is double-buffered in TMEM so the
//                     epilogue of tile i overlaps the loads and MMAs of tile i+1. Covers up/gate,
//                     down, dHidden (+GLU backward) and dX, for routed and shared experts.
// wgrad_gemm_kernel : per-expert weight gradient C[e] = A_e^T @ B_e; the contraction runs over the
//                     rows of the expert's run, split into chunks of ks_rows; a second small kernel
//                     sums the fp32 partials of split runs in chunk order (deterministic).
//
// Warp roles (both kernels): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2.. = epilogue (one accumulator row per thread; a warp may only read the TMEM lane
// quadrant 32*(warp%4)).
#pragma once
#include "pdl.cuh"
#include "ptx.cuh"

namespace moe {

constexpr int BM = 128;  // UMMA M: one TMEM lane per output row
constexpr int BK = 64;   // 64 bf16 = one 128-byte swizzle span
constexpr int A_STAGE_BYTES = BM * BK * 2;

// EPI_RAW_RED / EPI_SCALE_RED: as EPI_RAW / EPI_SCALE, but a row is not stored in slot order: it is
// added (bf16 atomics in L2, one bulk reduction per row and tile) to row `token` of a token-major
// matrix, which makes the GEMM also the combine.
enum GemmEpi { EPI_RAW = 0, EPI_GLU = 1, EPI_SCALE = 2, EPI_GLUBWD = 3, EPI_RAW_RED = 4,
               EPI_SCALE_RED = 5 };
enum Act { ACT_SILU = 0, ACT_GELU = 1, ACT_RELU = 2, ACT_SIGMOID = 3, ACT_TANH = 4 };

// Status codes a kernel can leave in the status word (0 = fine).
enum DevStatus { ST_OK = 0, ST_WAIT_TIMEOUT = 1, ST_BAD_EXPERT = 2 };

// MN-major 128B-swizzled operand as TMA lays it down in 64 x 64 boxes: 64 MN elements (128 B) per
// k row, 8 k rows per 1024-byte swizzle atom (SBO), next 64 MN elements one 8 KB box further (LBO);
// one UMMA K step (16) spans two atoms.
constexpr uint32_t MN_LBO = 8192u, MN_SBO = 1024u, MN_KADV = 2048u;

struct RowsArgs {
  // schedule
  const int32_t* expert_ids;   // routed: [tiles] owner of each 128-row block
  const int32_t* n_post_pad;   // routed: device scalar, live padded rows
  const int32_t* sorted_ids;   // routed: slot -> pair id, sentinel n_pairs in pad slots (may be null)
  int32_t n_fixed_groups;      // 0 = routed schedule; > 0 = groups 0..n-1, each over rows_host rows in
                               // token order (shared experts)
  int32_t rows_host;           // row count of the fixed-group schedule
  int32_t a_grouped;           // fixed schedule: A has a leading group dim ([G, rows, K])
  // gathered A (routed schedule only): row `slot` of the tile list is row sorted_ids[slot] / top_k
  // of the token-major matrix a_src [n_tokens, a_cols]; pad slots read as zero rows
  const __nv_bfloat16* a_src;
  int32_t a_cols;
  int32_t top_k;
  int32_t n_pairs;             // sentinel value in sorted_ids
  int32_t num_k;               // K / 64 (rounded up; the tail reads as zeros)
  int32_t n_dim;               // valid accumulator columns over all N chunks
  int32_t n_chunks;            // ceil(n_dim / BN)
  int32_t n_groups_total;      // CTA-pair kernels: number of runs in a2_offsets (both weight stacks)
  int32_t n_groups_b1;         // groups [0, n_groups_b1) read the first B stack, the rest the second
  int32_t a2_first_group;      // routed schedule: groups from here on read their A rows from the
                               // token-major second A map (row = slot - a2_offsets[group]);
                               // INT32_MAX = every group reads the slot-ordered buffer
  const int32_t* a2_offsets;   // [G + 1] run starts (pad_offsets), used with a2_first_group
  // group-summed fixed schedule (sum_groups > 0, n_fixed_groups == 1): ONE output row block per 128
  // token rows, accumulated over sum_groups groups -- C = sum_g A_g @ B_g with A_g = rows
  // [sum_offsets[g], sum_offsets[g] + rows_host) of the slot-ordered buffer (device offsets: the
  // dispatch's run starts) and B_g = group g of the weight stack. The k loop simply runs over
  // sum_groups * num_k stages.
  int32_t sum_groups;
  const int32_t* sum_offsets;
  int32_t b_fused;             // MN-major B: the maps are 4-D (64 n, k, n / 64, group) and one copy
                               // brings all BN / 64 boxes of a stage (a TMA instruction costs the
                               // issuing thread about as much as a whole stage of MMAs)
  // epilogue
  __nv_bfloat16* out;          // main output
  int64_t ld_out;              // elements between rows of out
  int64_t out_gstride;         // elements between fixed groups in out
  __nv_bfloat16* out2;         // GLU: raw [gate | up] rows (may be null); GLUBWD: w * hidden
  int64_t out2_gstride;
  __nv_bfloat16* dtw;          // GLUBWD: d(topk_w) flat [n_pairs] (may be null)
  const __nv_bfloat16* aux;    // GLUBWD: [gate | up] pre-activations [rows, 2H]
  int64_t aux_gstride;
  const __nv_bfloat16* pair_w; // SCALE / GLUBWD: topk_w flat [n_pairs] (null -> weight 1)
  const __nv_bfloat16* bias;   // GLU / SCALE: per-expert bias [all groups of both weight stacks, n_dim]
                               // added to the accumulator before the GLU / before the weight scale
                               // (null = none)
  int32_t act;
  int32_t* status;
};

struct WgradArgs {
  const int32_t* pad_offsets;  // routed: [G+1] run starts (multiples of 128); null = fixed rows
  int32_t n_groups;
  int32_t rows_host;           // fixed schedule: every group spans rows [0, rows_host)
  int32_t ks_rows;             // rows per split-K chunk (multiple of 64)
  int32_t a_grouped, b_grouped;  // fixed schedule: operand has a leading group dim
  int32_t a_fused, b_fused;    // the operand's map is 4-D (64 cols, row, col / 64, group): one copy
                               // brings all 64-column boxes of a stage
  // gathered operand (routed schedule only): its row `slot` is row sorted_ids[slot] / top_k of the
  // token-major matrix gather_src [n_tokens, m_dim or n_dim]; pad slots read as zero rows
  int32_t gather_a, gather_b;
  const __nv_bfloat16* gather_src;
  const int32_t* sorted_ids;
  int32_t top_k, n_pairs;
  int32_t m_dim, n_dim;        // rows / cols of one C[e]
  __nv_bfloat16* out;          // [n_out1, m_dim, n_dim]: groups [0, n_out1)
  __nv_bfloat16* out_extra;    // [G - n_out1, m_dim, n_dim]: the remaining groups (may be null)
  int32_t n_out1;
  float* partials;             // fp32 scratch for the partial tiles of split runs
  int32_t alt_which;           // 0 none; 1 / 2: runs from alt_first_group on read operand A / B from
  int32_t alt_first_group;     // the token-major alternative map, row = slot row - run start
  int32_t* item_table;         // scratch [G + 1]: first work item of every run, written by the GEMM
                               // pass for the reduction pass
  int32_t* status;
};

template <int ACT>
__device__ __forceinline__ float act_f(float g) {
  if constexpr (ACT == ACT_SILU) return __fdividef(g, 1.f + __expf(-g));
  if constexpr (ACT == ACT_GELU) return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
  if constexpr (ACT == ACT_RELU) return fmaxf(g, 0.f);
  if constexpr (ACT == ACT_SIGMOID) return __fdividef(1.f, 1.f + __expf(-g));
  return __fdividef(2.f, 1.f + __expf(-2.f * g)) - 1.f;
}
// (act(g), act'(g)) together: the backward needs both and they share the transcendental.
template <int ACT>
__device__ __forceinline__ void act_fd(float g, float& a, float& d) {
  if constexpr (ACT == ACT_SILU) {
    const float s = __fdividef(1.f, 1.f + __expf(-g));
    a = g * s;
    d = s * (1.f + g * (1.f - s));
  } else if constexpr (ACT == ACT_GELU) {
    const float cdf = 0.5f * (1.f + erff(g * 0.7071067811865476f));
    a = g * cdf;
    d = cdf + g * 0.3989422804014327f * __expf(-0.5f * g * g);
  } else if constexpr (ACT == ACT_RELU) {
    a = fmaxf(g, 0.f);
    d = g > 0.f ? 1.f : 0.f;
  } else if constexpr (ACT == ACT_SIGMOID) {
    a = __fdividef(1.f, 1.f + __expf(-g));
    d = a * (1.f - a);
  } else {
    a = __fdividef(2.f, 1.f + __expf(-2.f * g)) - 1.f;
    d = 1.f - a * a;
  }
}

// 256-bit global accesses (sm_100): one full 32-byte sector per thread and instruction, so a
// thread that owns 64 contiguous bytes of a row touches each sector exactly once.
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]),
               "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ void ld_global_nc_v8(const void* p, uint32_t* w) {
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]),
                 "=r"(w[7])
               : "l"(p));
}

// 32 fp32 -> 32 bf16 = 64 bytes, stored as two 32-byte vectors (dst 32-byte aligned).
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float* v) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 16 + 2 * i], v[q * 16 + 2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    st_global_v8(dst + q * 16, w);
  }
}
__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* src, float* v) {
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t w[8];
    ld_global_nc_v8(src + q * 16, w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&w[i]);
      float2 f = __bfloat1622float2(h);
      v[q * 16 + 2 * i] = f.x;
      v[q * 16 + 2 * i + 1] = f.y;
    }
  }
}
// 32 fp32 stored as four 32-byte vectors (dst 32-byte aligned).
__device__ __forceinline__ void store_f32x32(float* dst, const float* v) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    st_global_v8(dst + q * 8, reinterpret_cast<const uint32_t*>(v) + q * 8);
}

__device__ __forceinline__ void epi_bar_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}
// Named barrier `id` over nthreads threads in total: arrivers do not wait, syncers wait for all.
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Issue the four K=16 MMAs of one 64-wide k stage.
template <int BN, bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_stage_mmas(uint32_t sA, uint32_t sB, uint32_t d_tmem,
                                                 bool first_stage) {
  constexpr uint32_t idesc = umma_idesc(BM, BN, A_MN, B_MN);
#pragma unroll
  for (int k16 = 0; k16 < BK / 16; ++k16) {
    const uint64_t da = A_MN ? umma_desc(sA + k16 * MN_KADV, MN_LBO, MN_SBO)
                             : umma_desc(sA + k16 * 32, 16, 1024);
    const uint64_t db = B_MN ? umma_desc(sB + k16 * MN_KADV, MN_LBO, MN_SBO)
                             : umma_desc(sB + k16 * 32, 16, 1024);
    umma_f16(d_tmem, da, db, idesc, (first_stage && k16 == 0) ? 0u : 1u);
  }
}

}  // namespace moe

#include "gemm_rows.cuh"
#include "gemm_rows2.cuh"
#include "gemm_wgrad.cuh"
#include "gemm_wgrad2.cuh"
