// Host side of the grouped tcgen05 GEMMs: builds the TMA tensor maps for each stage's operands and
// launches the matching instantiation of grouped_gemm_kernel (gemm.cuh).
#include "gemm.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>

#include "../../include/moe_b200.h"

namespace moe {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// bf16 tensor map, 128-byte swizzle, zero fill out of bounds. dims/box innermost first;
// strides (bytes) for dims 1..rank-1.
static bool make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gd[5];
  cuuint64_t gs[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gd[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides[i];
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, cuuint32_t(rank), const_cast<void*>(base), gd, gs,
            bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [rows, cols] row-major activation buffer, K-major A operand: box = 64 cols x 128 rows.
static bool map_rows_kmajor(CUtensorMap* m, const void* base, int64_t rows, int64_t cols) {
  const uint64_t dims[2] = {uint64_t(cols), uint64_t(rows)};
  const uint64_t strides[1] = {uint64_t(cols) * 2};
  const uint32_t box[2] = {64, 128};
  return make_map(m, base, 2, dims, strides, box);
}
// [rows, cols] row-major buffer read as an MN-major operand (contraction over rows): 64 x 64 boxes.
static bool map_rows_mnmajor(CUtensorMap* m, const void* base, int64_t rows, int64_t cols) {
  const uint64_t dims[2] = {uint64_t(cols), uint64_t(rows)};
  const uint64_t strides[1] = {uint64_t(cols) * 2};
  const uint32_t box[2] = {64, 64};
  return make_map(m, base, 2, dims, strides, box);
}
// Stacked weights [G, k_dim, n_dim] with n contiguous (the reference's W_in / W_out layout used
// in the forward): MN-major B operand, 64 (n) x 64 (k) boxes.
static bool map_weight_mnmajor(CUtensorMap* m, const void* base, int64_t groups, int64_t k_dim,
                               int64_t n_dim) {
  const uint64_t dims[3] = {uint64_t(n_dim), uint64_t(k_dim), uint64_t(groups)};
  const uint64_t strides[2] = {uint64_t(n_dim) * 2, uint64_t(n_dim) * uint64_t(k_dim) * 2};
  const uint32_t box[3] = {64, 64, 1};
  return make_map(m, base, 3, dims, strides, box);
}
// Stacked weights [G, n_dim, k_dim] with k contiguous (the same tensors read "transposed" in the
// backward): K-major B operand, 64 (k) x BN (n) box.
static bool map_weight_kmajor(CUtensorMap* m, const void* base, int64_t groups, int64_t n_dim,
                              int64_t k_dim, int bn) {
  const uint64_t dims[3] = {uint64_t(k_dim), uint64_t(n_dim), uint64_t(groups)};
  const uint64_t strides[2] = {uint64_t(k_dim) * 2, uint64_t(n_dim) * uint64_t(k_dim) * 2};
  const uint32_t box[3] = {64, uint32_t(bn), 1};
  return make_map(m, base, 3, dims, strides, box);
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int MODE, int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, dim3 grid,
                  cudaStream_t st) {
  auto kern = grouped_gemm_kernel<BN, STAGES, A_MN, B_MN, MODE, EPI>;
  constexpr int smem = GemmSmem<BN, STAGES>::DYNAMIC;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (attr_err != cudaSuccess) return MOE_B200_ERR_CUDA;
  kern<<<grid, 192, smem, st>>>(tmA, tmB, args);
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static GemmArgs base_args(const int32_t* expert_ids, const int32_t* n_post_pad,
                          int32_t fixed_group, int64_t rows, int32_t* status) {
  GemmArgs a{};
  a.expert_ids = expert_ids;
  a.n_post_pad = n_post_pad;
  a.fixed_group = fixed_group;
  a.rows_host = int32_t(rows);
  a.status = status;
  return a;
}

}  // namespace moe

using namespace moe;

#define CHECK_SCHED()                                                                       \
  if (rows < 0 || n_groups < 1) return MOE_B200_ERR_SHAPE;                                  \
  if (rows == 0) return MOE_B200_OK;                                                        \
  if (!status) return MOE_B200_ERR_NULL;                                                    \
  if (fixed_group < 0 && (!expert_ids || !n_post_pad)) return MOE_B200_ERR_NULL;            \
  if (fixed_group >= n_groups) return MOE_B200_ERR_SHAPE;                                   \
  if (fixed_group < 0 && rows % 128 != 0) return MOE_B200_ERR_SHAPE;

extern "C" {

int moe_b200_up_gemm(const void* a, int64_t rows, int32_t d_model, const void* w_in,
                     int32_t n_groups, int32_t d_hidden, const int32_t* expert_ids,
                     const int32_t* n_post_pad, int32_t fixed_group, int32_t write_raw,
                     int32_t activation, void* out, int64_t ld_out, int32_t* status, void* stream) {
  CHECK_SCHED();
  if (d_hidden != 128 || d_model % 8 != 0 || d_model < 64) return MOE_B200_ERR_UNSUPPORTED;
  if (activation < 0 || activation > 4) return MOE_B200_ERR_UNSUPPORTED;
  if (!a || !w_in || !out) return MOE_B200_ERR_NULL;
  if (!aligned16(a) || !aligned16(w_in) || !aligned16(out) || ld_out % 8 != 0)
    return MOE_B200_ERR_ALIGN;
  CUtensorMap tmA, tmB;
  if (!map_rows_kmajor(&tmA, a, rows, d_model) ||
      !map_weight_mnmajor(&tmB, w_in, n_groups, d_model, 2 * d_hidden))
    return MOE_B200_ERR_TMA;
  GemmArgs g = base_args(expert_ids, n_post_pad, fixed_group, rows, status);
  g.num_k = (d_model + BK - 1) / BK;
  g.n_dim = 2 * d_hidden;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ld_out = ld_out;
  g.act = activation;
  const dim3 grid(unsigned((rows + BM - 1) / BM), 1, 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (write_raw) return launch<256, 3, false, true, MODE_ROWS, EPI_RAW>(tmA, tmB, g, grid, st);
  return launch<256, 3, false, true, MODE_ROWS, EPI_GLU>(tmA, tmB, g, grid, st);
}

int moe_b200_down_gemm(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                       int32_t n_groups, int32_t d_model, const int32_t* expert_ids,
                       const int32_t* n_post_pad, int32_t fixed_group, const int32_t* sorted_ids,
                       const void* pair_w, int64_t n_pairs, void* y, int32_t* status,
                       void* stream) {
  CHECK_SCHED();
  if (k_dim % 8 != 0 || k_dim < 64 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!hid || !w_out || !y) return MOE_B200_ERR_NULL;
  if (pair_w && fixed_group < 0 && !sorted_ids) return MOE_B200_ERR_NULL;
  if (!aligned16(hid) || !aligned16(w_out) || !aligned16(y)) return MOE_B200_ERR_ALIGN;
  CUtensorMap tmA, tmB;
  if (!map_rows_kmajor(&tmA, hid, rows, k_dim) ||
      !map_weight_mnmajor(&tmB, w_out, n_groups, k_dim, d_model))
    return MOE_B200_ERR_TMA;
  GemmArgs g = base_args(expert_ids, n_post_pad, fixed_group, rows, status);
  g.num_k = (k_dim + BK - 1) / BK;
  g.n_dim = d_model;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.pair_w = static_cast<const __nv_bfloat16*>(pair_w);
  g.out = static_cast<__nv_bfloat16*>(y);
  g.ld_out = d_model;
  const dim3 grid(unsigned((rows + BM - 1) / BM), unsigned((d_model + 191) / 192), 1);
  return launch<192, 2, false, true, MODE_ROWS, EPI_SCALE>(tmA, tmB, g, grid,
                                                           static_cast<cudaStream_t>(stream));
}

int moe_b200_dhidden_glu_bwd(const void* douts, int64_t rows, int32_t d_model, const void* w_out,
                             int32_t n_groups, int32_t d_hidden, const int32_t* expert_ids,
                             const int32_t* n_post_pad, int32_t fixed_group,
                             const int32_t* sorted_ids, const void* pair_w, int64_t n_pairs,
                             const void* a1, int32_t activation, void* da1, void* hidw, void* dtw,
                             int32_t* status, void* stream) {
  CHECK_SCHED();
  if (d_hidden != 128 || d_model % 8 != 0 || d_model < 64) return MOE_B200_ERR_UNSUPPORTED;
  if (activation < 0 || activation > 4) return MOE_B200_ERR_UNSUPPORTED;
  if (!douts || !w_out || !a1 || !da1 || !hidw) return MOE_B200_ERR_NULL;
  if (pair_w && fixed_group < 0 && !sorted_ids) return MOE_B200_ERR_NULL;
  if (!aligned16(douts) || !aligned16(w_out) || !aligned16(a1) || !aligned16(da1) ||
      !aligned16(hidw))
    return MOE_B200_ERR_ALIGN;
  CUtensorMap tmA, tmB;
  if (!map_rows_kmajor(&tmA, douts, rows, d_model) ||
      !map_weight_kmajor(&tmB, w_out, n_groups, d_hidden, d_model, 128))
    return MOE_B200_ERR_TMA;
  GemmArgs g = base_args(expert_ids, n_post_pad, fixed_group, rows, status);
  g.num_k = (d_model + BK - 1) / BK;
  g.n_dim = d_hidden;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.pair_w = static_cast<const __nv_bfloat16*>(pair_w);
  g.aux = static_cast<const __nv_bfloat16*>(a1);
  g.out = static_cast<__nv_bfloat16*>(da1);
  g.out2 = static_cast<__nv_bfloat16*>(hidw);
  g.dtw = static_cast<__nv_bfloat16*>(dtw);
  g.act = activation;
  const dim3 grid(unsigned((rows + BM - 1) / BM), 1, 1);
  return launch<128, 4, false, false, MODE_ROWS, EPI_GLUBWD>(tmA, tmB, g, grid,
                                                             static_cast<cudaStream_t>(stream));
}

int moe_b200_dx_gemm(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                     int32_t n_groups, int32_t d_model, const int32_t* expert_ids,
                     const int32_t* n_post_pad, int32_t fixed_group, void* ydx, int32_t* status,
                     void* stream) {
  CHECK_SCHED();
  if (d_hidden % 4 != 0 || d_hidden < 32 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!da1 || !w_in || !ydx) return MOE_B200_ERR_NULL;
  if (!aligned16(da1) || !aligned16(w_in) || !aligned16(ydx)) return MOE_B200_ERR_ALIGN;
  CUtensorMap tmA, tmB;
  if (!map_rows_kmajor(&tmA, da1, rows, 2 * d_hidden) ||
      !map_weight_kmajor(&tmB, w_in, n_groups, d_model, 2 * d_hidden, 192))
    return MOE_B200_ERR_TMA;
  GemmArgs g = base_args(expert_ids, n_post_pad, fixed_group, rows, status);
  g.num_k = (2 * d_hidden + BK - 1) / BK;
  g.n_dim = d_model;
  g.out = static_cast<__nv_bfloat16*>(ydx);
  g.ld_out = d_model;
  const dim3 grid(unsigned((rows + BM - 1) / BM), unsigned((d_model + 191) / 192), 1);
  return launch<192, 3, false, false, MODE_ROWS, EPI_RAW>(tmA, tmB, g, grid,
                                                          static_cast<cudaStream_t>(stream));
}

int moe_b200_wgrad(const void* a, int32_t m_dim, const void* b, int32_t n_dim, int64_t rows,
                   const int32_t* pad_offsets, int32_t n_groups, void* dw, int32_t* status,
                   void* stream) {
  if (rows < 0 || n_groups < 1 || m_dim < 1 || n_dim < 1) return MOE_B200_ERR_SHAPE;
  if (m_dim % 8 != 0 || n_dim % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!pad_offsets && n_groups != 1) return MOE_B200_ERR_SHAPE;
  if (!a || !b || !dw || !status) return MOE_B200_ERR_NULL;
  if (!aligned16(a) || !aligned16(b) || !aligned16(dw)) return MOE_B200_ERR_ALIGN;
  CUtensorMap tmA, tmB;
  // rows == 0 still launches: every C[e] must be written (with zeros)
  const int64_t map_rows = rows > 0 ? rows : 1;
  if (!map_rows_mnmajor(&tmA, a, map_rows, m_dim) || !map_rows_mnmajor(&tmB, b, map_rows, n_dim))
    return MOE_B200_ERR_TMA;
  GemmArgs g{};
  g.pad_offsets = pad_offsets;
  g.rows_host = int32_t(rows);
  g.fixed_group = pad_offsets ? -1 : 0;
  g.m_dim = m_dim;
  g.n_dim = n_dim;
  g.out = static_cast<__nv_bfloat16*>(dw);
  g.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_dim % 256 == 0) {
    const dim3 grid(unsigned((m_dim + BM - 1) / BM), unsigned(n_dim / 256), unsigned(n_groups));
    return launch<256, 3, true, true, MODE_WGRAD, EPI_WGRAD>(tmA, tmB, g, grid, st);
  }
  const dim3 grid(unsigned((m_dim + BM - 1) / BM), unsigned((n_dim + 191) / 192),
                  unsigned(n_groups));
  return launch<192, 3, true, true, MODE_WGRAD, EPI_WGRAD>(tmA, tmB, g, grid, st);
}

}  // extern "C"
