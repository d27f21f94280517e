// Pieces shared by the routing kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

constexpr int MAX_EXPERTS = 256;  // router + dispatch kernels keep per-expert state on chip
constexpr int MAX_TOPK = 16;

// Order-preserving map fp32 -> uint32 (larger float -> larger key); NaN sorts above +inf and
// -0.0 ties with +0.0, so ties between equal values fall to the lowest expert index below.
__device__ __forceinline__ uint32_t float_key(float f) {
  if (f != f) return 0xFFFFFFFFu;
  if (f == 0.f) f = 0.f;
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}


}  // namespace moe
