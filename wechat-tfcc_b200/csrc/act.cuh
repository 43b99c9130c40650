// Activations shared by the GEMM epilogues and the stand-alone element-wise kernels.
#pragma once

#include <cuda_runtime.h>

#include "../../include/tfcc_b200.h"

namespace tfccb200 {

// 0.5 * v * (1 + erf(v / sqrt(2))) with the reference's mixed precision
// (tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:214-220): the literal 0.5 is a double there,
// so the two outer products are carried out in double and rounded to float once.
__device__ __forceinline__ float gelu_erf(float v) {
  const float e = 1.0f + erff(v / 1.4142135623730951f);
  return static_cast<float>(__dmul_rn(__dmul_rn(0.5, static_cast<double>(v)), static_cast<double>(e)));
}

__device__ __forceinline__ float apply_activation(float v, int activation) {
  return activation == TFCCB200_ACT_GELU_ERF ? gelu_erf(v) : v;
}

}  // namespace tfccb200
