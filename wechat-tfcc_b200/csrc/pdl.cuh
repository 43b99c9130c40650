// Programmatic dependent launch: a kernel launched through launch_after_previous() may
// begin (block scheduling, shared-memory set-up, barrier and tensor-memory initialisation)
// while the kernel before it in the stream is still draining.  It must not touch global
// memory before pdl_wait(), which returns once every earlier kernel in the stream has
// completed and its stores are visible.  pdl_release() tells the runtime that the NEXT
// kernel in the stream may start its own preamble; it implies nothing about this kernel's
// results (the next kernel's pdl_wait() still waits for this one to finish).
// In operator sequences of latency-bound kernels (an encoder block is ~16 launches of
// 3-50 us) this hides the launch gap and most of each kernel's preamble.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace tfccb200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// TFCCB200_PDL=0 launches everything with full stream serialisation (for A/B timing).
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("TFCCB200_PDL");
    return !(v && v[0] == '0');
  }();
  return on;
}

// Launch `kernel` so that it may overlap the tail of the previous kernel in `stream`.
// The kernel must call pdl_wait() before its first global-memory access.
template <typename... Params, typename... Args>
cudaError_t launch_after_previous(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(std::forward<Args>(args))...);
}

}  // namespace tfccb200
