// Activations shared by the GEMM epilogues and the stand-alone element-wise kernels.
#pragma once

#include <cuda_runtime.h>

#include "../../include/tfcc_b200.h"

namespace tfccb200 {

// 0.5 * v * (1 + erf(v / sqrt(2))) with the reference's mixed precision
// (tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:214-220).  There the literal 0.5 is a double,
// so 0.5 * v * e is evaluated in double and rounded to float once.  Both factors are floats
// (e = 1 + erf(float) is a float sum), so their product is exact in double and the single
// rounding equals one float multiplication; halving e first is exact too.  No double
// arithmetic is needed for the same bits.
__device__ __forceinline__ float gelu_erf(float v) {
  const float e = 1.0f + erff(v / 1.4142135623730951f);
  return __fmul_rn(v, 0.5f * e);
}

__device__ __forceinline__ float apply_activation(float v, int activation) {
  return activation == TFCCB200_ACT_GELU_ERF ? gelu_erf(v) : v;
}

}  // namespace tfccb200
