// ABI version and error text for the C interface declared in include/moe_b200.h.
#include "../../include/moe_b200.h"

extern "C" {

int32_t moe_b200_abi_version(void) { return 2; }

const char* moe_b200_error_string(int32_t code) {
  switch (code) {
    case MOE_B200_OK: return "ok";
    case MOE_B200_ERR_SHAPE: return "bad shape: a size is negative, zero or inconsistent";
    case MOE_B200_ERR_NULL: return "a required pointer is NULL";
    case MOE_B200_ERR_ALIGN: return "a pointer or row stride is not aligned (16 bytes for inputs, 32 for GEMM operands and outputs)";
    case MOE_B200_ERR_SCRATCH: return "scratch buffer missing or too small";
    case MOE_B200_ERR_UNSUPPORTED: return "shape or activation not covered by the sm_100a kernels";
    case MOE_B200_ERR_TMA: return "cuTensorMapEncodeTiled refused a tensor map";
    case MOE_B200_ERR_CUDA: return "kernel launch failed";
    case MOE_B200_ERR_TOO_LARGE:
      return "problem larger than the fixed built-in scratch of the no-allocation entry point";
    default: return "unknown moe_b200 error code";
  }
}

}  // extern "C"
