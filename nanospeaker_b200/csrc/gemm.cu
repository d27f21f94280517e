// Host side of the grouped tcgen05 GEMMs: builds the TMA tensor maps for each stage's operands and
// launches the matching instantiation of grouped_gemm_kernel (gemm.cuh).
#include "gemm.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "../../include/moe_b200.h"

// dHidden: ring stages / pre-activation buffers (32 KB / 64 KB each)
#ifndef MOE_DH_STAGES
#define MOE_DH_STAGES 4
#endif
#ifndef MOE_DH_AUX_BUFS
#define MOE_DH_AUX_BUFS 1
#endif
#ifndef MOE_PAIR_WGRAD_STAGES
#define MOE_PAIR_WGRAD_STAGES 6   // 32 KB per stage and CTA
#endif
#ifndef MOE_PAIR_UP_STAGES
#define MOE_PAIR_UP_STAGES 6
#endif
#ifndef MOE_PAIR_DX_STAGES
#define MOE_PAIR_DX_STAGES 4
#endif

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

// [groups, rows, cols] row-major activation buffer as the K-major A operand: 64 cols x 128 rows.
static bool map_rows_kmajor(CUtensorMap* m, const void* base, int64_t groups, int64_t rows,
                            int64_t cols) {
  const uint64_t dims[3] = {uint64_t(cols), uint64_t(rows), uint64_t(groups)};
  const uint64_t strides[2] = {uint64_t(cols) * 2, uint64_t(cols) * uint64_t(rows) * 2};
  const uint32_t box[3] = {64, 128, 1};
  return make_map(m, base, 3, dims, strides, box);
}
// [groups, rows, cols] buffer read as an MN-major operand (contraction over rows): 64 x 64 boxes.
// When cols is a multiple of 64 the map is 4-D (64 cols, row, col / 64, group) with `boxes` boxes
// per copy (*fused = 1): one TMA instruction then fills a whole stage of the operand.
static bool map_rows_mnmajor(CUtensorMap* m, const void* base, int64_t groups, int64_t rows,
                             int64_t cols, int boxes, int32_t* fused) {
  if (cols % 64 == 0) {
    const uint64_t dims[4] = {64, uint64_t(rows), uint64_t(cols / 64), uint64_t(groups)};
    const uint64_t strides[3] = {uint64_t(cols) * 2, 128, uint64_t(cols) * uint64_t(rows) * 2};
    const uint32_t box[4] = {64, 64, uint32_t(boxes), 1};
    *fused = 1;
    return make_map(m, base, 4, dims, strides, box);
  }
  const uint64_t dims[3] = {uint64_t(cols), uint64_t(rows), uint64_t(groups)};
  const uint64_t strides[2] = {uint64_t(cols) * 2, uint64_t(cols) * uint64_t(rows) * 2};
  const uint32_t box[3] = {64, 64, 1};
  *fused = 0;
  return make_map(m, base, 3, dims, strides, box);
}
// Stacked weights [G, k_dim, n_dim] with n contiguous (the reference's W_in / W_out layout used
// in the forward): MN-major B operand, 64 (n) x 64 (k) boxes; 4-D with `boxes` boxes per copy when
// n_dim is a multiple of 64, as above.
static bool map_weight_mnmajor(CUtensorMap* m, const void* base, int64_t groups, int64_t k_dim,
                               int64_t n_dim, int boxes, int32_t* fused) {
  return map_rows_mnmajor(m, base, groups, k_dim, n_dim, boxes, fused);
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

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// Persistent launch: one CTA per SM (fewer if the tile list is shorter than that).
template <int BN, int STAGES, bool B_MN, int EPI, bool GATHER_A = false, int OUT_BOXES = 4>
static int launch_rows(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmB2,
                       const CUtensorMap& tmOut, const RowsArgs& args, int64_t max_tiles,
                       cudaStream_t st, const CUtensorMap* tmA2 = nullptr) {
  auto kern = rows_gemm_kernel<BN, STAGES, B_MN, EPI, GATHER_A, OUT_BOXES>;
  constexpr int smem = RowsSmem<BN, STAGES, EPI, OUT_BOXES>::DYNAMIC;
  static_assert(smem <= 232448, "shared memory of a row GEMM exceeds the 227 KB per-CTA limit");
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (attr_err != cudaSuccess) return MOE_B200_ERR_CUDA;
  const int64_t sms = sm_count();
  const unsigned grid = unsigned(max_tiles < sms ? max_tiles : sms);
  const cudaError_t err = launch_pdl(kern, dim3(grid), dim3(rows_threads(EPI, GATHER_A)),
                                     size_t(smem), st, tmA, tmA2 ? *tmA2 : tmA, tmB, tmB2, tmOut,
                                     args);
  return err == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

// CTA-pair launch (rows_gemm2_kernel): as many clusters of two as can be resident at once (a
// 148-SM part need not fit 74 of them: SMs pair up inside their processing cluster), fewer when
// the unit list is shorter.
template <int BN, int STAGES, bool B_MN, int EPI>
static int launch_rows2(const CUtensorMap& tmA, const CUtensorMap& tmA2, const CUtensorMap& tmB,
                        const CUtensorMap& tmB2, const CUtensorMap& tmOut, const RowsArgs& args,
                        int64_t max_units, cudaStream_t st) {
  auto kern = rows_gemm2_kernel<BN, STAGES, B_MN, EPI>;
  constexpr int smem = Rows2Smem<BN, STAGES, EPI>::DYNAMIC;
  static_assert(smem <= 232448, "shared memory of a row GEMM exceeds the 227 KB per-CTA limit");
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  static int max_clusters = 0;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (attr_err != cudaSuccess) return;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(sm_count() / 2 * 2));
    cfg.blockDim = dim3(rows_threads(EPI, false));
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    attr_err = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
  });
  if (attr_err != cudaSuccess || max_clusters < 1) return MOE_B200_ERR_CUDA;
  int64_t clusters = std::min<int64_t>(max_clusters, sm_count() / 2);
  if (max_units < clusters) clusters = max_units;
  const cudaError_t err = launch_pdl_pairs(kern, dim3(unsigned(2 * clusters)),
                                           dim3(rows_threads(EPI, false)), size_t(smem), st, tmA,
                                           tmA2, tmB, tmB2, tmOut, args);
  return err == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

// Upper bound on the pair units of a routed launch: every run may end in a half-empty pair.
static int64_t max_pair_units(int64_t rows, int n_groups_total, int n_chunks) {
  return ((rows / BM + n_groups_total + 1) / 2) * n_chunks;
}

template <int BN, int STAGES, int GATHER>
static int launch_wgrad_g(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmAlt,
                          const WgradArgs& args, int tiles_x, int tiles_y, int64_t max_items,
                          cudaStream_t st) {
  auto kern = wgrad_gemm_kernel<BN, STAGES, GATHER>;
  constexpr int smem = WgradSmem<BN, STAGES>::DYNAMIC;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (attr_err != cudaSuccess) return MOE_B200_ERR_CUDA;
  const int64_t tiles = max_items * tiles_x * tiles_y, sms = sm_count();
  const unsigned grid = unsigned(tiles < sms ? tiles : sms);
  const int threads = GATHER ? WGRAD_THREADS_GATHER : WGRAD_THREADS;
  const cudaError_t err =
      launch_pdl(kern, dim3(grid), dim3(threads), size_t(smem), st, tmA, tmB, tmAlt, args, tiles_x,
                 tiles_y);
  return err == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

// The weight gradient on CTA pairs (gemm_wgrad2.cuh): clusters of two, one per SM pair.
template <int BN, int STAGES>
static int launch_wgrad2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmAlt,
                         const WgradArgs& args, int tiles_x, int tiles_y, int64_t max_items,
                         cudaStream_t st) {
  auto kern = wgrad_gemm2_kernel<BN, STAGES>;
  constexpr int smem = Wgrad2Smem<BN, STAGES>::DYNAMIC;
  static_assert(smem <= 232448, "shared memory of the pair weight gradient exceeds the CTA limit");
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  static int max_clusters = 0;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (attr_err != cudaSuccess) return;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(sm_count() / 2 * 2));
    cfg.blockDim = dim3(WGRAD_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    attr_err = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
  });
  if (attr_err != cudaSuccess || max_clusters < 1) return MOE_B200_ERR_CUDA;
  const int64_t units = max_items * ((tiles_x + 1) / 2) * tiles_y;
  int64_t clusters = std::min<int64_t>(max_clusters, sm_count() / 2);
  if (units < clusters) clusters = units;
  const cudaError_t err =
      launch_pdl_pairs(kern, dim3(unsigned(2 * clusters)), dim3(WGRAD_THREADS), size_t(smem), st,
                       tmA, tmB, tmAlt, args, tiles_x, tiles_y);
  return err == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

template <int BN, int STAGES>
static int launch_wgrad(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmAlt,
                        const WgradArgs& args, int tiles_x, int tiles_y, int64_t max_items,
                        cudaStream_t st) {
  if (args.gather_a)
    return launch_wgrad_g<BN, STAGES, 1>(tmA, tmB, tmAlt, args, tiles_x, tiles_y, max_items, st);
  if (args.gather_b)
    return launch_wgrad_g<BN, STAGES, 2>(tmA, tmB, tmAlt, args, tiles_x, tiles_y, max_items, st);
  return launch_wgrad_g<BN, STAGES, 0>(tmA, tmB, tmAlt, args, tiles_x, tiles_y, max_items, st);
}

// inputs feed TMA (16 bytes); outputs are written with 32-byte vectors
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

static RowsArgs base_args(const int32_t* expert_ids, const int32_t* n_post_pad,
                          int32_t n_fixed_groups, int64_t rows, int32_t* status) {
  RowsArgs a{};
  a.expert_ids = expert_ids;
  a.n_post_pad = n_post_pad;
  a.n_fixed_groups = n_fixed_groups;
  a.rows_host = int32_t(rows);
  a.a2_first_group = INT32_MAX;
  a.status = status;
  return a;
}

// Token-major A rows for the groups of the second weight stack (the shared experts): the map over
// a_tokens [n_tokens, k_dim] and the schedule fields that switch those groups over to it.
static int use_token_rows(RowsArgs* g, CUtensorMap* tmA2, const void* a_tokens, int64_t n_tokens,
                          const int32_t* pad_offsets, int32_t n_groups, int32_t n_extra,
                          int32_t n_fixed_groups, int32_t gather_top_k, int32_t k_dim) {
  if (!a_tokens) return MOE_B200_OK;
  if (n_extra < 1 || n_fixed_groups > 0 || gather_top_k > 0 || n_tokens < 1) return MOE_B200_ERR_SHAPE;
  if (!pad_offsets) return MOE_B200_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(a_tokens) & 15u) != 0) return MOE_B200_ERR_ALIGN;
  if (!map_rows_kmajor(tmA2, a_tokens, 1, n_tokens, k_dim)) return MOE_B200_ERR_TMA;
  g->a2_first_group = n_groups;
  g->a2_offsets = pad_offsets;
  return MOE_B200_OK;
}

// Upper bound on the tile count of a row-grouped launch (the live count is on the device).
static int64_t max_tiles(int64_t rows, int n_chunks, int n_fixed_groups) {
  return (rows + BM - 1) / BM * n_chunks * (n_fixed_groups > 0 ? n_fixed_groups : 1);
}

}  // namespace moe

using namespace moe;

#define CHECK_SCHED()                                                                        \
  if (rows < 0 || n_groups < 1 || n_fixed_groups < 0) return MOE_B200_ERR_SHAPE;             \
  if (rows == 0) return MOE_B200_OK;                                                         \
  if (rows > (int64_t(1) << 30)) return MOE_B200_ERR_SHAPE;                                  \
  if (!status) return MOE_B200_ERR_NULL;                                                     \
  if (n_fixed_groups == 0 && (!expert_ids || !n_post_pad)) return MOE_B200_ERR_NULL;         \
  if (n_fixed_groups > n_groups) return MOE_B200_ERR_SHAPE;                                  \
  if (n_fixed_groups == 0 && rows % 128 != 0) return MOE_B200_ERR_SHAPE;

// A second weight stack (the shared experts') serves expert ids >= n_groups on the routed schedule.
#define CHECK_EXTRA()                                                               \
  if (n_extra < 0 || (n_extra > 0 && (!w_extra || n_fixed_groups > 0)))            \
    return n_extra < 0 || n_fixed_groups > 0 ? MOE_B200_ERR_SHAPE : MOE_B200_ERR_NULL; \
  if (n_extra > 0 && !aligned16(w_extra)) return MOE_B200_ERR_ALIGN;

extern "C" {

int moe_b200_up_gemm(const void* a, int64_t rows, int32_t d_model, const void* w_in,
                     int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_hidden, const int32_t* expert_ids,
                     const int32_t* n_post_pad, int32_t n_fixed_groups,
                     const int32_t* sorted_ids, int32_t gather_top_k, int64_t n_pairs,
                     int32_t activation, void* hid, void* raw, const void* a_tokens,
                     int64_t n_tokens, const int32_t* pad_offsets, const void* bias,
                     int32_t* status, void* stream) {
  CHECK_SCHED();
  if (bias && (n_fixed_groups > 0 || (reinterpret_cast<uintptr_t>(bias) & 15u) != 0))
    return n_fixed_groups > 0 ? MOE_B200_ERR_SHAPE : MOE_B200_ERR_ALIGN;
  if (d_hidden != 128 || d_model % 8 != 0 || d_model < 64) return MOE_B200_ERR_UNSUPPORTED;
  if (activation < 0 || activation > 4) return MOE_B200_ERR_UNSUPPORTED;
  if (!a || !w_in || !hid) return MOE_B200_ERR_NULL;
  if (gather_top_k < 0 || (gather_top_k > 0 && (n_fixed_groups > 0 || !sorted_ids || n_pairs < 0)))
    return MOE_B200_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(w_in) || !aligned16(hid) || !aligned16(raw))
    return MOE_B200_ERR_ALIGN;
  CHECK_EXTRA();
  CUtensorMap tmA, tmB, tmB2;
  int32_t fused = 0;
  if (!map_weight_mnmajor(&tmB, w_in, n_groups, d_model, 2 * d_hidden, 4, &fused))
    return MOE_B200_ERR_TMA;
  tmB2 = tmB;
  if (n_extra > 0 && !map_weight_mnmajor(&tmB2, w_extra, n_extra, d_model, 2 * d_hidden, 4, &fused))
    return MOE_B200_ERR_TMA;
  if (gather_top_k > 0)
    tmA = tmB;  // unused: A rows are gathered with cp.async
  else if (!map_rows_kmajor(&tmA, a, 1, rows, d_model))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(expert_ids, n_post_pad, n_fixed_groups, rows, status);
  g.num_k = (d_model + BK - 1) / BK;
  g.n_dim = 2 * d_hidden;
  g.n_chunks = 1;
  g.b_fused = fused;
  g.out = static_cast<__nv_bfloat16*>(hid);
  g.ld_out = d_hidden;
  g.out_gstride = rows * int64_t(d_hidden);
  g.out2 = static_cast<__nv_bfloat16*>(raw);
  g.out2_gstride = rows * int64_t(2 * d_hidden);
  g.act = activation;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.n_groups_b1 = n_extra > 0 ? n_groups : INT32_MAX;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.a_src = static_cast<const __nv_bfloat16*>(a);
  g.a_cols = d_model;
  g.top_k = gather_top_k;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t tiles = max_tiles(rows, 1, n_fixed_groups);
  CUtensorMap tmA2 = tmA;
  const int rc2 = use_token_rows(&g, &tmA2, a_tokens, n_tokens, pad_offsets, n_groups, n_extra,
                                 n_fixed_groups, gather_top_k, d_model);
  if (rc2 != MOE_B200_OK) return rc2;
  if (gather_top_k > 0)
    return launch_rows<256, 4, true, EPI_GLU, true>(tmA, tmB, tmB2, tmB, g, tiles, st);
#ifndef MOE_NO_PAIR_UP
  // Routed schedule with the run table at hand: CTA pairs, each CTA loading half of the expert's
  // weight tile (the 4-D weight maps then bring 2 of the 4 64-column boxes per copy).
  if (n_fixed_groups == 0 && pad_offsets != nullptr && fused) {
    int32_t f2 = 0;
    CUtensorMap hB, hB2;
    if (!map_weight_mnmajor(&hB, w_in, n_groups, d_model, 2 * d_hidden, 2, &f2)) return MOE_B200_ERR_TMA;
    hB2 = hB;
    if (n_extra > 0 && !map_weight_mnmajor(&hB2, w_extra, n_extra, d_model, 2 * d_hidden, 2, &f2))
      return MOE_B200_ERR_TMA;
    g.a2_offsets = pad_offsets;
    g.n_groups_total = n_groups + n_extra;
    return launch_rows2<256, MOE_PAIR_UP_STAGES, true, EPI_GLU>(
        tmA, tmA2, hB, hB2, hB, g, max_pair_units(rows, n_groups + n_extra, 1), st);
  }
#endif
  return launch_rows<256, 4, true, EPI_GLU>(tmA, tmB, tmB2, tmB, g, tiles, st, &tmA2);
}

int moe_b200_down_gemm(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                       int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model, const int32_t* expert_ids,
                       const int32_t* n_post_pad, int32_t n_fixed_groups,
                       const int32_t* sorted_ids, const void* pair_w, int64_t n_pairs, void* y,
                       const void* bias, int32_t* status, void* stream) {
  CHECK_SCHED();
  if (bias && (n_fixed_groups > 0 || (reinterpret_cast<uintptr_t>(bias) & 15u) != 0))
    return n_fixed_groups > 0 ? MOE_B200_ERR_SHAPE : MOE_B200_ERR_ALIGN;
  if (k_dim % 8 != 0 || k_dim < 64 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!hid || !w_out || !y) return MOE_B200_ERR_NULL;
  if (pair_w && n_fixed_groups == 0 && !sorted_ids) return MOE_B200_ERR_NULL;
  if (!aligned16(hid) || !aligned16(w_out) || !aligned16(y)) return MOE_B200_ERR_ALIGN;
  CHECK_EXTRA();
  const int gdim = n_fixed_groups > 0 ? n_fixed_groups : 1;
  CUtensorMap tmA, tmB, tmB2, tmOut;
  int32_t fused = 0;
  if (!map_rows_kmajor(&tmA, hid, gdim, rows, k_dim) ||
      !map_weight_mnmajor(&tmB, w_out, n_groups, k_dim, d_model, 3, &fused) ||
      !map_rows_kmajor(&tmOut, y, gdim, rows, d_model))  // stored as 64-column x 128-row boxes
    return MOE_B200_ERR_TMA;
  tmB2 = tmB;
  if (n_extra > 0 && !map_weight_mnmajor(&tmB2, w_extra, n_extra, k_dim, d_model, 3, &fused))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(expert_ids, n_post_pad, n_fixed_groups, rows, status);
  g.a_grouped = n_fixed_groups > 0;
  g.num_k = (k_dim + BK - 1) / BK;
  g.n_dim = d_model;
  g.n_chunks = (d_model + 191) / 192;
  g.b_fused = fused;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.pair_w = static_cast<const __nv_bfloat16*>(pair_w);
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.out = static_cast<__nv_bfloat16*>(y);
  g.ld_out = d_model;
  g.out_gstride = rows * int64_t(d_model);
  g.n_groups_b1 = n_extra > 0 ? n_groups : INT32_MAX;
  return launch_rows<192, 4, true, EPI_SCALE, false, 4>(
      tmA, tmB, tmB2, tmOut, g, max_tiles(rows, g.n_chunks, n_fixed_groups), static_cast<cudaStream_t>(stream));
}

int moe_b200_dhidden_glu_bwd(const void* douts, int64_t rows, int32_t d_model, const void* w_out,
                             int32_t n_groups, const void* w_extra, int32_t n_extra,
                             int32_t d_hidden, const int32_t* expert_ids,
                             const int32_t* n_post_pad, int32_t n_fixed_groups,
                             const int32_t* sorted_ids, int32_t gather_top_k, const void* pair_w,
                             int64_t n_pairs, const void* a1, int32_t activation, void* da1,
                             void* hidw, void* dtw, const void* dout_tokens, int64_t n_tokens,
                             const int32_t* pad_offsets, int32_t* status, void* stream) {
  CHECK_SCHED();
  if (gather_top_k < 0 || (gather_top_k > 0 && (n_fixed_groups > 0 || !sorted_ids)))
    return MOE_B200_ERR_SHAPE;
  if (d_hidden != 128 || d_model % 8 != 0 || d_model < 64) return MOE_B200_ERR_UNSUPPORTED;
  if (activation < 0 || activation > 4) return MOE_B200_ERR_UNSUPPORTED;
  if (!douts || !w_out || !a1 || !da1 || !hidw) return MOE_B200_ERR_NULL;
  if (pair_w && n_fixed_groups == 0 && !sorted_ids) return MOE_B200_ERR_NULL;
  if (!aligned16(douts) || !aligned16(w_out) || !aligned16(a1) || !aligned16(da1) ||
      !aligned16(hidw))
    return MOE_B200_ERR_ALIGN;
  CHECK_EXTRA();
  CUtensorMap tmA, tmB, tmB2;
  if (!map_weight_kmajor(&tmB, w_out, n_groups, d_hidden, d_model, 128)) return MOE_B200_ERR_TMA;
  tmB2 = tmB;
  if (n_extra > 0 && !map_weight_kmajor(&tmB2, w_extra, n_extra, d_hidden, d_model, 128))
    return MOE_B200_ERR_TMA;
  if (gather_top_k > 0)
    tmA = tmB;  // unused: dOut rows are gathered with cp.async
  else if (!map_rows_kmajor(&tmA, douts, 1, rows, d_model))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(expert_ids, n_post_pad, n_fixed_groups, rows, status);
  g.num_k = (d_model + BK - 1) / BK;
  g.n_dim = d_hidden;
  g.n_chunks = 1;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.pair_w = static_cast<const __nv_bfloat16*>(pair_w);
  g.aux = static_cast<const __nv_bfloat16*>(a1);
  g.aux_gstride = rows * int64_t(2 * d_hidden);
  g.out = static_cast<__nv_bfloat16*>(da1);
  g.ld_out = 2 * d_hidden;
  g.out_gstride = rows * int64_t(2 * d_hidden);
  g.out2 = static_cast<__nv_bfloat16*>(hidw);
  g.out2_gstride = rows * int64_t(d_hidden);
  g.dtw = static_cast<__nv_bfloat16*>(dtw);
  g.act = activation;
  g.n_groups_b1 = n_extra > 0 ? n_groups : INT32_MAX;
  g.a_src = static_cast<const __nv_bfloat16*>(douts);
  g.a_cols = d_model;
  g.top_k = gather_top_k;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t tiles = max_tiles(rows, 1, n_fixed_groups);
  // the pre-activations reach the epilogue through shared memory: 64-column x 128-row boxes
  CUtensorMap tmAux;
  if (!map_rows_kmajor(&tmAux, a1, n_fixed_groups > 0 ? n_fixed_groups : 1, rows, 2 * d_hidden))
    return MOE_B200_ERR_TMA;
  CUtensorMap tmA2 = tmA;
  const int rc2 = use_token_rows(&g, &tmA2, dout_tokens, n_tokens, pad_offsets, n_groups, n_extra,
                                 n_fixed_groups, gather_top_k, d_model);
  if (rc2 != MOE_B200_OK) return rc2;
  if (gather_top_k > 0)
    return launch_rows<128, 3, false, EPI_GLUBWD, true>(tmA, tmB, tmB2, tmAux, g, tiles, st);
  return launch_rows<128, MOE_DH_STAGES, false, EPI_GLUBWD, false, MOE_DH_AUX_BUFS>(
      tmA, tmB, tmB2, tmAux, g, tiles, st, &tmA2);
}

int moe_b200_dx_gemm(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                     int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model, const int32_t* expert_ids,
                     const int32_t* n_post_pad, int32_t n_fixed_groups, void* ydx,
                     int32_t* status, void* stream) {
  CHECK_SCHED();
  if (d_hidden % 4 != 0 || d_hidden < 32 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!da1 || !w_in || !ydx) return MOE_B200_ERR_NULL;
  if (!aligned16(da1) || !aligned16(w_in) || !aligned16(ydx)) return MOE_B200_ERR_ALIGN;
  CHECK_EXTRA();
  const int gdim = n_fixed_groups > 0 ? n_fixed_groups : 1;
  CUtensorMap tmA, tmB, tmB2, tmOut;
  if (!map_rows_kmajor(&tmA, da1, gdim, rows, 2 * d_hidden) ||
      !map_weight_kmajor(&tmB, w_in, n_groups, d_model, 2 * d_hidden, 192) ||
      !map_rows_kmajor(&tmOut, ydx, gdim, rows, d_model))  // stored as 64-column x 128-row boxes
    return MOE_B200_ERR_TMA;
  tmB2 = tmB;
  if (n_extra > 0 && !map_weight_kmajor(&tmB2, w_extra, n_extra, d_model, 2 * d_hidden, 192))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(expert_ids, n_post_pad, n_fixed_groups, rows, status);
  g.a_grouped = n_fixed_groups > 0;
  g.num_k = (2 * d_hidden + BK - 1) / BK;
  g.n_dim = d_model;
  g.n_chunks = (d_model + 191) / 192;
  g.out = static_cast<__nv_bfloat16*>(ydx);
  g.ld_out = d_model;
  g.out_gstride = rows * int64_t(d_model);
  g.n_groups_b1 = n_extra > 0 ? n_groups : INT32_MAX;
  return launch_rows<192, 4, false, EPI_RAW, false, 3>(
      tmA, tmB, tmB2, tmOut, g, max_tiles(rows, g.n_chunks, n_fixed_groups), static_cast<cudaStream_t>(stream));
}

// The group-summed row GEMMs: out[t] = sum_g A[run_offsets[g] + t] @ B_g, plain stores. They give
// the token-major accumulators of the atomic combine their initial value -- the shared experts'
// contribution, whose rows are in token order -- so that no fill pass is needed and only the routed
// experts' rows go through the L2's atomic units.
static int sum_checks(const void* a, const void* w, const void* out, const int32_t* run_offsets,
                      int64_t rows, int32_t n_sum, int64_t n_tokens, const int32_t* status) {
  if (rows < 1 || n_sum < 1 || n_tokens < 1 || rows > (int64_t(1) << 30) || n_tokens > rows)
    return MOE_B200_ERR_SHAPE;
  if (!a || !w || !out || !run_offsets || !status) return MOE_B200_ERR_NULL;
  if (!aligned16(a) || !aligned16(w) || !aligned16(out)) return MOE_B200_ERR_ALIGN;
  return MOE_B200_OK;
}

int moe_b200_down_gemm_sum(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                           int32_t n_sum, int32_t d_model, const int32_t* run_offsets,
                           int64_t n_tokens, void* out, int32_t* status, void* stream) {
  const int rc = sum_checks(hid, w_out, out, run_offsets, rows, n_sum, n_tokens, status);
  if (rc != MOE_B200_OK) return rc;
  if (k_dim % 8 != 0 || k_dim < 64 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB, tmOut;
  int32_t fused = 0;
  if (!map_rows_kmajor(&tmA, hid, 1, rows, k_dim) ||
      !map_weight_mnmajor(&tmB, w_out, n_sum, k_dim, d_model, 3, &fused) ||
      !map_rows_kmajor(&tmOut, out, 1, n_tokens, d_model))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(nullptr, nullptr, 1, n_tokens, status);
  g.sum_groups = n_sum;
  g.sum_offsets = run_offsets;
  g.num_k = (k_dim + BK - 1) / BK;
  g.n_dim = d_model;
  g.n_chunks = (d_model + 191) / 192;
  g.b_fused = fused;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ld_out = d_model;
  g.n_groups_b1 = INT32_MAX;
  return launch_rows<192, 4, true, EPI_SCALE, false, 4>(
      tmA, tmB, tmB, tmOut, g, max_tiles(n_tokens, g.n_chunks, 1), static_cast<cudaStream_t>(stream));
}

int moe_b200_dx_gemm_sum(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                         int32_t n_sum, int32_t d_model, const int32_t* run_offsets,
                         int64_t n_tokens, void* out, int32_t* status, void* stream) {
  const int rc = sum_checks(da1, w_in, out, run_offsets, rows, n_sum, n_tokens, status);
  if (rc != MOE_B200_OK) return rc;
  if (d_hidden % 4 != 0 || d_hidden < 32 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB, tmOut;
  if (!map_rows_kmajor(&tmA, da1, 1, rows, 2 * d_hidden) ||
      !map_weight_kmajor(&tmB, w_in, n_sum, d_model, 2 * d_hidden, 192) ||
      !map_rows_kmajor(&tmOut, out, 1, n_tokens, d_model))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(nullptr, nullptr, 1, n_tokens, status);
  g.sum_groups = n_sum;
  g.sum_offsets = run_offsets;
  g.num_k = (2 * d_hidden + BK - 1) / BK;
  g.n_dim = d_model;
  g.n_chunks = (d_model + 191) / 192;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ld_out = d_model;
  g.n_groups_b1 = INT32_MAX;
  return launch_rows<192, 4, false, EPI_RAW, false, 3>(
      tmA, tmB, tmB, tmOut, g, max_tiles(n_tokens, g.n_chunks, 1), static_cast<cudaStream_t>(stream));
}

// Ring stages / staging buffers of the two accumulating row GEMMs (shared memory per CTA: stages x
// 40 KB + buffers x 50 KB at 192-column tiles).
#ifndef MOE_RED_DOWN_STAGES
#define MOE_RED_DOWN_STAGES 3
#endif
#ifndef MOE_RED_DOWN_BUFS
#define MOE_RED_DOWN_BUFS 2
#endif
#ifndef MOE_RED_DX_STAGES
#define MOE_RED_DX_STAGES 3
#endif
#ifndef MOE_RED_DX_BUFS
#define MOE_RED_DX_BUFS 2
#endif

// Where an accumulating GEMM adds its rows: routed schedule -> row sorted_ids[slot] / top_k of
// acc [n_tokens, d_model]; fixed schedule -> row `row` (every group adds to the same rows).
static int check_acc(int32_t n_fixed_groups, int64_t rows, const int32_t* sorted_ids, int32_t top_k,
                     int64_t n_pairs, const void* acc, int64_t n_tokens, int32_t d_model) {
  if (!acc) return MOE_B200_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(acc) & 15u) != 0) return MOE_B200_ERR_ALIGN;
  if (d_model % 32 != 0 || n_tokens < 1) return MOE_B200_ERR_SHAPE;
  if (n_fixed_groups > 0) return rows <= n_tokens ? MOE_B200_OK : MOE_B200_ERR_SHAPE;
  if (!sorted_ids) return MOE_B200_ERR_NULL;
  if (top_k < 1 || n_pairs < 0 || n_pairs > n_tokens * int64_t(top_k)) return MOE_B200_ERR_SHAPE;
  return MOE_B200_OK;
}

int moe_b200_down_gemm_acc(const void* hid, int64_t rows, int32_t k_dim, const void* w_out,
                           int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model,
                           const int32_t* expert_ids, const int32_t* n_post_pad,
                           int32_t n_fixed_groups, const int32_t* sorted_ids, const void* pair_w,
                           int64_t n_pairs, int32_t top_k, void* acc, int64_t n_tokens,
                           const void* bias, int32_t* status, void* stream) {
  CHECK_SCHED();
  if (bias && (n_fixed_groups > 0 || (reinterpret_cast<uintptr_t>(bias) & 15u) != 0))
    return n_fixed_groups > 0 ? MOE_B200_ERR_SHAPE : MOE_B200_ERR_ALIGN;
  if (k_dim % 8 != 0 || k_dim < 64 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!hid || !w_out) return MOE_B200_ERR_NULL;
  if (!aligned16(hid) || !aligned16(w_out)) return MOE_B200_ERR_ALIGN;
  const int rca = check_acc(n_fixed_groups, rows, sorted_ids, top_k, n_pairs, acc, n_tokens, d_model);
  if (rca != MOE_B200_OK) return rca;
  CHECK_EXTRA();
  const int gdim = n_fixed_groups > 0 ? n_fixed_groups : 1;
  CUtensorMap tmA, tmB, tmB2;
  int32_t fused = 0;
  if (!map_rows_kmajor(&tmA, hid, gdim, rows, k_dim) ||
      !map_weight_mnmajor(&tmB, w_out, n_groups, k_dim, d_model, 3, &fused))
    return MOE_B200_ERR_TMA;
  tmB2 = tmB;
  if (n_extra > 0 && !map_weight_mnmajor(&tmB2, w_extra, n_extra, k_dim, d_model, 3, &fused))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(expert_ids, n_post_pad, n_fixed_groups, rows, status);
  g.a_grouped = n_fixed_groups > 0;
  g.num_k = (k_dim + BK - 1) / BK;
  g.n_dim = d_model;
  g.n_chunks = (d_model + 191) / 192;
  g.b_fused = fused;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.top_k = top_k;
  g.pair_w = static_cast<const __nv_bfloat16*>(pair_w);
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.out = static_cast<__nv_bfloat16*>(acc);
  g.ld_out = d_model;
  g.n_groups_b1 = n_extra > 0 ? n_groups : INT32_MAX;
  return launch_rows<192, MOE_RED_DOWN_STAGES, true, EPI_SCALE_RED, false, MOE_RED_DOWN_BUFS>(
      tmA, tmB, tmB2, tmB, g, max_tiles(rows, g.n_chunks, n_fixed_groups),
      static_cast<cudaStream_t>(stream));
}

int moe_b200_dx_gemm_acc(const void* da1, int64_t rows, int32_t d_hidden, const void* w_in,
                         int32_t n_groups, const void* w_extra, int32_t n_extra, int32_t d_model,
                         const int32_t* expert_ids, const int32_t* n_post_pad,
                         int32_t n_fixed_groups, const int32_t* sorted_ids, int64_t n_pairs,
                         int32_t top_k, void* acc, int64_t n_tokens, const int32_t* pad_offsets,
                         int32_t* status, void* stream) {
  CHECK_SCHED();
  if (d_hidden % 4 != 0 || d_hidden < 32 || d_model % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (!da1 || !w_in) return MOE_B200_ERR_NULL;
  if (!aligned16(da1) || !aligned16(w_in)) return MOE_B200_ERR_ALIGN;
  const int rca = check_acc(n_fixed_groups, rows, sorted_ids, top_k, n_pairs, acc, n_tokens, d_model);
  if (rca != MOE_B200_OK) return rca;
  CHECK_EXTRA();
  const int gdim = n_fixed_groups > 0 ? n_fixed_groups : 1;
  CUtensorMap tmA, tmB, tmB2;
  if (!map_rows_kmajor(&tmA, da1, gdim, rows, 2 * d_hidden) ||
      !map_weight_kmajor(&tmB, w_in, n_groups, d_model, 2 * d_hidden, 192))
    return MOE_B200_ERR_TMA;
  tmB2 = tmB;
  if (n_extra > 0 && !map_weight_kmajor(&tmB2, w_extra, n_extra, d_model, 2 * d_hidden, 192))
    return MOE_B200_ERR_TMA;
  RowsArgs g = base_args(expert_ids, n_post_pad, n_fixed_groups, rows, status);
  g.a_grouped = n_fixed_groups > 0;
  g.num_k = (2 * d_hidden + BK - 1) / BK;
  g.n_dim = d_model;
  g.n_chunks = (d_model + 191) / 192;
  g.sorted_ids = sorted_ids;
  g.n_pairs = int32_t(n_pairs);
  g.top_k = top_k;
  g.out = static_cast<__nv_bfloat16*>(acc);
  g.ld_out = d_model;
  g.n_groups_b1 = n_extra > 0 ? n_groups : INT32_MAX;
#ifndef MOE_NO_PAIR_DX
  // Routed schedule with the run table at hand: CTA pairs, each CTA loading 96 of the 192 weight
  // rows of the tile.
  if (n_fixed_groups == 0 && pad_offsets != nullptr) {
    CUtensorMap hB, hB2;
    if (!map_weight_kmajor(&hB, w_in, n_groups, d_model, 2 * d_hidden, 96)) return MOE_B200_ERR_TMA;
    hB2 = hB;
    if (n_extra > 0 && !map_weight_kmajor(&hB2, w_extra, n_extra, d_model, 2 * d_hidden, 96))
      return MOE_B200_ERR_TMA;
    g.a2_offsets = pad_offsets;
    g.n_groups_total = n_groups + n_extra;
    return launch_rows2<192, MOE_PAIR_DX_STAGES, false, EPI_RAW_RED>(
        tmA, tmA, hB, hB2, hB, g, max_pair_units(rows, n_groups + n_extra, g.n_chunks),
        static_cast<cudaStream_t>(stream));
  }
#endif
  return launch_rows<192, MOE_RED_DX_STAGES, false, EPI_RAW_RED, false, MOE_RED_DX_BUFS>(
      tmA, tmB, tmB2, tmB, g, max_tiles(rows, g.n_chunks, n_fixed_groups),
      static_cast<cudaStream_t>(stream));
}

// The scratch buffer starts with the item table ([G + 1] int32), the partial tiles follow.
constexpr size_t WGRAD_TABLE_BYTES = 4096;
static_assert((WGRAD_MAX_GROUPS + 1) * sizeof(int32_t) <= WGRAD_TABLE_BYTES, "item table too small");

static int64_t wgrad_items(int64_t rows, int n_groups, int routed, int ks_rows) {
  return routed ? rows / ks_rows + n_groups : int64_t(n_groups) * wgrad_chunks(int(rows), ks_rows);
}

// Rows per split-K chunk when the caller leaves the choice to the library: expert runs are cut at
// 3072 rows (measured at T=16384, 78 experts: dW_in 98 / 82 / 78 / 72 / 75 / 89 us for chunks of
// 1024 / 1536 / 2048 / 3072 / 4096 / 8192 rows -- shorter chunks mean more fp32 partial tiles,
// longer ones a longer tail); on the fixed schedule (few groups, every row) the chunks are sized so that the
// work items fill the SMs about once.
static int auto_ks_rows(int32_t m_dim, int32_t n_dim, int64_t rows, int n_groups, int routed) {
  if (routed) return 3072;
  const int bn = n_dim % 256 == 0 ? 256 : 192;
  const int64_t tiles = int64_t((m_dim + BM - 1) / BM) * ((n_dim + bn - 1) / bn) * n_groups;
  int64_t splits = sm_count() / (tiles > 0 ? tiles : 1);
  if (splits < 1) splits = 1;
  int64_t ks = ((rows + splits - 1) / splits + 63) / 64 * 64;
  if (ks < 256) ks = 256;
  return int(ks);
}

int moe_b200_wgrad_scratch_bytes(int32_t m_dim, int32_t n_dim, int64_t rows, int32_t n_groups,
                                 int32_t routed, int32_t ks_rows, size_t* partial_bytes) {
  if (m_dim < 1 || n_dim < 1 || rows < 0 || n_groups < 1 || ks_rows < 0 || ks_rows % 64 != 0 ||
      !partial_bytes)
    return MOE_B200_ERR_SHAPE;
  if (ks_rows == 0) ks_rows = auto_ks_rows(m_dim, n_dim, rows, n_groups, routed);
  const int bn = n_dim % 256 == 0 ? 256 : 192;
  const int64_t tiles_xy = int64_t((m_dim + BM - 1) / BM) * ((n_dim + bn - 1) / bn);
  *partial_bytes = WGRAD_TABLE_BYTES + size_t(wgrad_items(rows, n_groups, routed, ks_rows)) *
                                           size_t(tiles_xy) * BM * bn * sizeof(float);
  return MOE_B200_OK;
}

int moe_b200_wgrad(const void* a, int32_t a_grouped, int32_t m_dim, const void* b,
                   int32_t b_grouped, int32_t n_dim, int64_t rows, const int32_t* pad_offsets,
                   int32_t n_groups, int32_t ks_rows, const int32_t* sorted_ids,
                   int32_t gather_top_k, int64_t n_pairs, int32_t gather_which, void* dw,
                   int32_t n_first, void* dw_extra, void* partials, size_t partial_bytes,
                   const void* alt, int64_t alt_rows, int32_t alt_which, int32_t* status,
                   void* stream) {
  if (rows < 0 || rows > (int64_t(1) << 30) || n_groups < 1 || n_groups > WGRAD_MAX_GROUPS ||
      m_dim < 1 || n_dim < 1)
    return MOE_B200_ERR_SHAPE;
  if (ks_rows < 0 || ks_rows % 64 != 0) return MOE_B200_ERR_SHAPE;
  if (m_dim % 8 != 0 || n_dim % 32 != 0) return MOE_B200_ERR_UNSUPPORTED;
  if (pad_offsets && (a_grouped || b_grouped)) return MOE_B200_ERR_SHAPE;
  if (pad_offsets && rows % 128 != 0) return MOE_B200_ERR_SHAPE;
  if (gather_which < 0 || gather_which > 2) return MOE_B200_ERR_SHAPE;
  if (gather_which && (!pad_offsets || !sorted_ids || gather_top_k < 1 || n_pairs < 0))
    return MOE_B200_ERR_SHAPE;
  if (!a || !b || !dw || !status || !partials) return MOE_B200_ERR_NULL;
  if (n_first < 1 || n_first > n_groups || (n_first < n_groups && !dw_extra))
    return MOE_B200_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(b) || !aligned16(dw) || !aligned16(partials) ||
      !aligned16(dw_extra))
    return MOE_B200_ERR_ALIGN;
  const int routed = pad_offsets != nullptr;
  if (ks_rows == 0) ks_rows = auto_ks_rows(m_dim, n_dim, rows, n_groups, routed);
  size_t need_p = 0;
  moe_b200_wgrad_scratch_bytes(m_dim, n_dim, rows, n_groups, routed, ks_rows, &need_p);
  if (partial_bytes < need_p) return MOE_B200_ERR_SCRATCH;
  CUtensorMap tmA, tmB;
  // rows == 0 still launches: every C[e] must be written (with zeros)
  const int64_t map_rows = rows > 0 ? rows : 1;
  // a gathered operand is token-major and copied with cp.async: it gets the other one's map
  // CTA pairs: plain operands, 256-column tiles, at least two 128-row tiles of C; each CTA of a
  // pair loads half of the B tile, so B's map has 128-column boxes
  static const bool no_pair_wgrad = getenv("MOE_NO_PAIR_WGRAD") != nullptr;
  bool pairs = !no_pair_wgrad && gather_which == 0 && n_dim % 256 == 0 && m_dim > BM &&
               m_dim % 64 == 0;
  const int bn_boxes = n_dim % 256 == 0 ? (pairs ? 2 : 4) : 3;
  int32_t a_fused = 0, b_fused = 0;
  if (gather_which != 1 &&
      !map_rows_mnmajor(&tmA, a, a_grouped ? n_groups : 1, map_rows, m_dim, BM / 64, &a_fused))
    return MOE_B200_ERR_TMA;
  if (gather_which != 2 &&
      !map_rows_mnmajor(&tmB, b, b_grouped ? n_groups : 1, map_rows, n_dim, bn_boxes, &b_fused))
    return MOE_B200_ERR_TMA;
  if (gather_which == 1) tmA = tmB;
  if (gather_which == 2) tmB = tmA;
  // runs [n_first, n_groups) may read one operand from a token-major matrix (row = slot - run start)
  CUtensorMap tmAlt = tmA;
  if (alt) {
    if (alt_which < 1 || alt_which > 2 || !routed || gather_which || n_first >= n_groups || alt_rows < 1)
      return MOE_B200_ERR_SHAPE;
    if (!aligned16(alt)) return MOE_B200_ERR_ALIGN;
    int32_t alt_fused = 0;
    if (!map_rows_mnmajor(&tmAlt, alt, 1, alt_rows, alt_which == 1 ? m_dim : n_dim,
                          alt_which == 1 ? BM / 64 : bn_boxes, &alt_fused))
      return MOE_B200_ERR_TMA;
    if (alt_fused != (alt_which == 1 ? a_fused : b_fused)) return MOE_B200_ERR_TMA;
  }
  if (pairs && !(a_fused && b_fused)) {   // the pair kernel takes 4-D maps only: remake B's
    pairs = false;
    if (!map_rows_mnmajor(&tmB, b, b_grouped ? n_groups : 1, map_rows, n_dim, 4, &b_fused))
      return MOE_B200_ERR_TMA;
    if (alt && alt_which == 2) {
      int32_t alt_fused = 0;
      if (!map_rows_mnmajor(&tmAlt, alt, 1, alt_rows, n_dim, 4, &alt_fused) || alt_fused != b_fused)
        return MOE_B200_ERR_TMA;
    }
  }
  WgradArgs g{};
  g.alt_which = alt ? alt_which : 0;
  g.alt_first_group = n_first;
  g.pad_offsets = pad_offsets;
  g.n_groups = n_groups;
  g.rows_host = int32_t(rows);
  g.ks_rows = ks_rows;
  g.a_grouped = a_grouped;
  g.b_grouped = b_grouped;
  g.a_fused = a_fused;
  g.b_fused = b_fused;
  g.m_dim = m_dim;
  g.n_dim = n_dim;
  g.out = static_cast<__nv_bfloat16*>(dw);
  g.out_extra = static_cast<__nv_bfloat16*>(dw_extra);
  g.n_out1 = n_first;
  g.item_table = static_cast<int32_t*>(partials);
  g.partials = reinterpret_cast<float*>(static_cast<char*>(partials) + WGRAD_TABLE_BYTES);
  g.status = status;
  g.gather_a = gather_which == 1;
  g.gather_b = gather_which == 2;
  g.gather_src = static_cast<const __nv_bfloat16*>(gather_which == 1 ? a : b);
  g.sorted_ids = sorted_ids;
  g.top_k = gather_top_k;
  g.n_pairs = int32_t(n_pairs);
  const unsigned items = unsigned(wgrad_items(rows, n_groups, routed, ks_rows));
  // the second pass can be skipped when no run can have more than one chunk
  const bool may_split = rows > ks_rows;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned tx = unsigned((m_dim + BM - 1) / BM);
  // reduce CTAs per tile slice: they share the split runs (at most rows / ks_rows of them)
  const unsigned gy = unsigned(std::min<int64_t>(n_groups, std::min<int64_t>(8, rows / ks_rows + 1)));
  int rc;
  if (n_dim % 256 == 0) {
    const unsigned ty = unsigned(n_dim / 256);
    rc = pairs ? launch_wgrad2<256, MOE_PAIR_WGRAD_STAGES>(tmA, tmB, tmAlt, g, int(tx), int(ty),
                                                           items, st)
               : launch_wgrad<256, 4>(tmA, tmB, tmAlt, g, int(tx), int(ty), items, st);
    if (rc == MOE_B200_OK && may_split)
      launch_pdl(wgrad_reduce_kernel<256>, dim3(tx * ty * WGRAD_REDUCE_SPLIT, gy), dim3(256), 0, st,
                 g, int(tx), int(ty));
  } else {
    const unsigned ty = unsigned((n_dim + 191) / 192);
    rc = launch_wgrad<192, 5>(tmA, tmB, tmAlt, g, int(tx), int(ty), items, st);
    if (rc == MOE_B200_OK && may_split)
      launch_pdl(wgrad_reduce_kernel<192>, dim3(tx * ty * WGRAD_REDUCE_SPLIT, gy), dim3(256), 0, st,
                 g, int(tx), int(ty));
  }
  if (rc != MOE_B200_OK) return rc;
  return cudaGetLastError() == cudaSuccess ? MOE_B200_OK : MOE_B200_ERR_CUDA;
}

}  // extern "C"
