// Pieces shared by the routing kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

constexpr int MAX_EXPERTS = 256;  // router + dispatch kernels keep per-expert state on chip
constexpr int MAX_TOPK = 16;
constexpr int ALIGN_M = 128;     // expert runs are padded to whole 128-row GEMM tiles

// Order-preserving map fp32 -> uint32 (larger float -> larger key); NaN sorts above +inf and
// -0.0 ties with +0.0, so ties between equal values fall to the lowest expert index below.
__device__ __forceinline__ uint32_t float_key(float f) {
  if (f != f) return 0xFFFFFFFFu;
  if (f == 0.f) f = 0.f;
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

}  // namespace moe

#include <cuda_bf16.h>

namespace moe {
// router_fused.cu: router top-k in chunked mode (block b owns tokens [b * tokens_per_block, ...))
// that also leaves the dispatch's per-block histograms and the sentinel fill. Returns an error code
// of include/moe_b200.h.
// With `sc` given and the whole input in one block (n_blocks == 1), the four-lanes-per-token kernel
// also runs the dispatch's second pass itself and *did_scatter is set: no further launch is needed.
struct ScatterArgs {
  int32_t* counts;
  int32_t* pad_offsets;
  int32_t* n_post_pad;
  int32_t* expert_ids;
  int64_t n_tiles_cap;
  int32_t* inv_ids;
};
int launch_router_fused_chunked(const __nv_bfloat16* logits, int ld, const float* bias,
                                const float* noise,
                                int64_t n_tokens, int n_experts, int top_k, int n_shared,
                                int normalize, int full_softmax, __nv_bfloat16* w_all,
                                int64_t* idx_all, float* colsum, int tokens_per_block, int n_blocks,
                                int32_t* block_hist, int32_t* sorted_ids, int64_t l_cap,
                                cudaStream_t st, const ScatterArgs* sc = nullptr,
                                bool* did_scatter = nullptr);
}  // namespace moe
