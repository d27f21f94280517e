// Programmatic dependent launch. Every kernel of the library starts with pdl_trigger() + pdl_wait()
// and is launched with launch_pdl(): the next kernel in the stream may then be scheduled while this
// one still runs (its CTAs become resident as SMs free up and park in pdl_wait()), which hides the
// launch latency between two dependent kernels. pdl_wait() returns once the preceding kernel has
// completed and its writes are visible; it must be executed by every CTA before any global access
// and before exit, otherwise a later kernel could overtake an earlier one it depends on.
#pragma once

#include <cuda_runtime.h>

#include <utility>

namespace moe {

__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // A debug build (-DMOE_B200_DEBUG_NO_PDL) launches every kernel fully serialised; the kernels'
  // pdl_wait() is then a no-op.
#ifdef MOE_B200_DEBUG_NO_PDL
  cfg.numAttrs = 0;
#else
  cfg.numAttrs = 1;
#endif
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// The same launch for kernels that run as clusters of two CTAs (grid.x a multiple of 2).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl_pairs(void (*kern)(KArgs...), dim3 grid, dim3 block,
                                           size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
#ifdef MOE_B200_DEBUG_NO_PDL
  cfg.numAttrs = 1;
#else
  cfg.numAttrs = 2;
#endif
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

}  // namespace moe
