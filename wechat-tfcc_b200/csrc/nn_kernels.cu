// The element-wise and row-wise steps that sit between the matmuls of an attention / FFN
// block: row softmax with a fused pre-scale, erf-GELU, layer normalisation with a fused
// residual add, and the two 4-D permutations attention needs.  Formulas follow the
// reference's CPU kernels:
//   softmaxV2      tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:138-155
//   geluAccurate   tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:214-220
//   layer norm     tfcc/mkl/interfaces/tfcc_mklnormalizationinterface.cpp:29-62
//   transpose      tfcc/cuda/interfaces/tfcc_cudabasicinterface.cu:83-100 (same index map)
// All are HBM-bound: one read and one write of the tensor, 128-bit accesses where the row
// length allows.
#include <cuda_runtime.h>
#include <stdint.h>

#include "act.cuh"
#include "internal.h"
#include "pdl.cuh"

namespace tfccb200 {

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row; the row lives in registers (up to kMaxPerLane values per lane).
constexpr int kMaxPerLane = 32;  // rows up to 1024 columns

template <int PER_LANE>
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const float* __restrict__ src, unsigned rows, unsigned cols, float scale,
                    float* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  const unsigned row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const unsigned lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* p = src + static_cast<size_t>(row) * cols;
  float v[PER_LANE];
  float mx = -3.402823466e+38f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const unsigned c = lane + 32 * i;
    v[i] = c < cols ? p[c] * scale : -3.402823466e+38f;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const unsigned c = lane + 32 * i;
    v[i] = c < cols ? expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
  float* q = dst + static_cast<size_t>(row) * cols;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const unsigned c = lane + 32 * i;
    if (c < cols) q[c] = v[i] / sum;
  }
}

// The same with 128-bit loads and stores, for rows whose length is a multiple of 4 and whose
// base is 16-byte aligned: a quarter of the memory instructions, and the division by the row
// sum stays a division (the reference divides).
template <int VECS>
__global__ void __launch_bounds__(256)
softmax_rows_vec_kernel(const float4* __restrict__ src, unsigned rows, unsigned vecs, float scale,
                        float4* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  const unsigned row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const unsigned lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float4* p = src + static_cast<size_t>(row) * vecs;
  constexpr float kLowest = -3.402823466e+38f;
  float4 v[VECS];
  float mx = kLowest;
#pragma unroll
  for (int i = 0; i < VECS; ++i) {
    const unsigned c = lane + 32 * i;
    if (c < vecs) {
      const float4 t = __ldcs(p + c);
      v[i] = make_float4(t.x * scale, t.y * scale, t.z * scale, t.w * scale);
    } else {
      v[i] = make_float4(kLowest, kLowest, kLowest, kLowest);
    }
    mx = fmaxf(fmaxf(mx, v[i].x), fmaxf(v[i].y, fmaxf(v[i].z, v[i].w)));
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VECS; ++i) {
    const unsigned c = lane + 32 * i;
    if (c < vecs) {
      v[i] = make_float4(expf(v[i].x - mx), expf(v[i].y - mx), expf(v[i].z - mx), expf(v[i].w - mx));
      sum += v[i].x; sum += v[i].y; sum += v[i].z; sum += v[i].w;
    }
  }
  sum = warp_sum(sum);
  float4* q = dst + static_cast<size_t>(row) * vecs;
#pragma unroll
  for (int i = 0; i < VECS; ++i) {
    const unsigned c = lane + 32 * i;
    if (c < vecs) q[c] = make_float4(v[i].x / sum, v[i].y / sum, v[i].z / sum, v[i].w / sum);
  }
}

// Any row length: one CTA per row, three passes over the row (it stays in L1/L2).
__global__ void __launch_bounds__(256)
softmax_long_rows_kernel(const float* __restrict__ src, unsigned cols, float scale,
                         float* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  __shared__ float red[8];
  __shared__ float bcast;
  const float* p = src + static_cast<size_t>(blockIdx.x) * cols;
  float* q = dst + static_cast<size_t>(blockIdx.x) * cols;
  const unsigned lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  float mx = -3.402823466e+38f;
  for (unsigned c = threadIdx.x; c < cols; c += 256) mx = fmaxf(mx, p[c] * scale);
  mx = warp_max(mx);
  if (lane == 0) red[w] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    bcast = m;
  }
  __syncthreads();
  mx = bcast;
  float sum = 0.f;
  for (unsigned c = threadIdx.x; c < cols; c += 256) {
    const float e = expf(p[c] * scale - mx);
    q[c] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red[w] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += red[i];
    bcast = s;
  }
  __syncthreads();
  sum = bcast;
  for (unsigned c = threadIdx.x; c < cols; c += 256) q[c] /= sum;
}

// dst = layer_norm(x (+ residual)) * gamma + beta, one warp per row, two-pass mean / variance.
template <int PER_LANE>
__global__ void __launch_bounds__(256)
layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ residual,
                  const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                  unsigned rows, unsigned cols, float* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  const unsigned row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const unsigned lane = threadIdx.x & 31;
  if (row >= rows) return;
  const size_t off = static_cast<size_t>(row) * cols;
  float v[PER_LANE];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const unsigned c = lane + 32 * i;
    float t = 0.f;
    if (c < cols) {
      t = x[off + c];
      if (residual) t += residual[off + c];
    }
    v[i] = t;
    sum += t;
  }
  const float mean = warp_sum(sum) / static_cast<float>(cols);
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const unsigned c = lane + 32 * i;
    const float d = c < cols ? v[i] - mean : 0.f;
    var += d * d;
  }
  var = warp_sum(var) / static_cast<float>(cols);
  const float inv = 1.0f / sqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const unsigned c = lane + 32 * i;
    if (c < cols) dst[off + c] = (v[i] - mean) * (inv * gamma[c]) + beta[c];
  }
}

// Rows longer than a warp's registers hold (the reference's _cuda_layer_normalize_large,
// tfcc/cuda/interfaces/tfcc_cudanormalizationinterface.cu:85): one CTA per row, three passes
// over the row (mean, variance about the mean, output); the row stays in L1/L2 between them.
__global__ void __launch_bounds__(256)
layer_norm_long_rows_kernel(const float* __restrict__ x, const float* __restrict__ residual,
                            const float* __restrict__ gamma, const float* __restrict__ beta,
                            float eps, unsigned cols, float* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  __shared__ float red[8];
  __shared__ float bcast;
  const size_t off = static_cast<size_t>(blockIdx.x) * cols;
  const unsigned lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  auto block_sum = [&](float v) {
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int i = 0; i < 8; ++i) s += red[i];
      bcast = s;
    }
    __syncthreads();
    return bcast;
  };
  auto value = [&](unsigned c) { return residual ? x[off + c] + residual[off + c] : x[off + c]; };
  float sum = 0.f;
  for (unsigned c = threadIdx.x; c < cols; c += 256) sum += value(c);
  const float mean = block_sum(sum) / static_cast<float>(cols);
  float var = 0.f;
  for (unsigned c = threadIdx.x; c < cols; c += 256) {
    const float d = value(c) - mean;
    var += d * d;
  }
  var = block_sum(var) / static_cast<float>(cols);
  const float inv = 1.0f / sqrtf(var + eps);
  for (unsigned c = threadIdx.x; c < cols; c += 256)
    dst[off + c] = (value(c) - mean) * (inv * gamma[c]) + beta[c];
}

// Same, for rows that are whole float4 vectors at 16-byte aligned addresses: VPL vectors per
// lane, all loads of a row issued before the first use.
template <int VPL>
__global__ void __launch_bounds__(256)
layer_norm_vec_kernel(const float4* __restrict__ x, const float4* __restrict__ residual,
                      const float4* __restrict__ gamma, const float4* __restrict__ beta, float eps,
                      unsigned rows, unsigned vecs, float4* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  const unsigned row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const unsigned lane = threadIdx.x & 31;
  if (row >= rows) return;
  const size_t off = static_cast<size_t>(row) * vecs;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[VPL], r[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const unsigned c = lane + 32 * i;
    v[i] = c < vecs ? __ldcs(x + off + c) : zero;
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const unsigned c = lane + 32 * i;
    r[i] = (residual && c < vecs) ? __ldcs(residual + off + c) : zero;
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    v[i].x += r[i].x; v[i].y += r[i].y; v[i].z += r[i].z; v[i].w += r[i].w;
    sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float n = static_cast<float>(vecs * 4);
  const float mean = warp_sum(sum) / n;
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    if (lane + 32 * i < vecs) {
      const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
      var += (a * a + b * b) + (c * c + d * d);
    }
  }
  var = warp_sum(var) / n;
  const float inv = 1.0f / sqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const unsigned c = lane + 32 * i;
    if (c < vecs) {
      const float4 g = __ldg(gamma + c), bt = __ldg(beta + c);
      float4 o;
      o.x = (v[i].x - mean) * (inv * g.x) + bt.x;
      o.y = (v[i].y - mean) * (inv * g.y) + bt.y;
      o.z = (v[i].z - mean) * (inv * g.z) + bt.z;
      o.w = (v[i].w - mean) * (inv * g.w) + bt.w;
      dst[off + c] = o;
    }
  }
}

// Element-wise, may run in place (src == dst).
__global__ void __launch_bounds__(256)
gelu_kernel(const float* src, size_t n, float* dst) {
  pdl_release();
  pdl_wait();
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += gridDim.x * 256ull)
    dst[i] = gelu_erf(src[i]);
}
__global__ void __launch_bounds__(256)
gelu_vec_kernel(const float4* src, size_t n4, float4* dst) {
  pdl_release();
  pdl_wait();
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n4; i += gridDim.x * 256ull) {
    float4 v = src[i];
    v.x = gelu_erf(v.x); v.y = gelu_erf(v.y); v.z = gelu_erf(v.z); v.w = gelu_erf(v.w);
    dst[i] = v;
  }
}

// [d0,d1,d2,d3] -> [d0,d2,d1,d3]: rows of d3 contiguous floats move as a whole.
__global__ void __launch_bounds__(256)
permute_0213_kernel(const float* __restrict__ src, unsigned d0, unsigned d1, unsigned d2,
                    unsigned d3, float* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  const size_t total = static_cast<size_t>(d0) * d1 * d2 * d3;
  for (size_t o = blockIdx.x * 256ull + threadIdx.x; o < total; o += gridDim.x * 256ull) {
    const unsigned i3 = o % d3;
    size_t r = o / d3;
    const unsigned i1 = r % d1;  // destination order: [d0][d2][d1][d3]
    r /= d1;
    const unsigned i2 = r % d2;
    const unsigned i0 = r / d2;
    dst[o] = src[((static_cast<size_t>(i0) * d1 + i1) * d2 + i2) * d3 + i3];
  }
}

// Same with d3 a multiple of 4 and 16-byte aligned tensors: one float4 per thread step.
__global__ void __launch_bounds__(256)
permute_0213_vec_kernel(const float4* __restrict__ src, unsigned d0, unsigned d1, unsigned d2,
                        unsigned v3, float4* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  const size_t total = static_cast<size_t>(d0) * d1 * d2 * v3;
  for (size_t o = blockIdx.x * 256ull + threadIdx.x; o < total; o += gridDim.x * 256ull) {
    const unsigned i3 = o % v3;
    size_t r = o / v3;
    const unsigned i1 = r % d1;  // destination order: [d0][d2][d1][v3]
    r /= d1;
    const unsigned i2 = r % d2;
    const unsigned i0 = r / d2;
    dst[o] = __ldcs(src + ((static_cast<size_t>(i0) * d1 + i1) * d2 + i2) * v3 + i3);
  }
}

// [batch, r, c] -> [batch, c, r] through a padded 32x32 tile in shared memory.
__global__ void __launch_bounds__(256)
transpose_last2_kernel(const float* __restrict__ src, unsigned r, unsigned c,
                       float* __restrict__ dst) {
  pdl_release();
  pdl_wait();
  __shared__ float tile[32][33];
  const size_t base = static_cast<size_t>(blockIdx.z) * r * c;
  const unsigned r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  const unsigned tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const unsigned rr = r0 + ty + 8 * i, cc = c0 + tx;
    if (rr < r && cc < c) tile[ty + 8 * i][tx] = src[base + static_cast<size_t>(rr) * c + cc];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const unsigned cc = c0 + ty + 8 * i, rr = r0 + tx;
    if (rr < r && cc < c) dst[base + static_cast<size_t>(cc) * r + rr] = tile[tx][ty + 8 * i];
  }
}

int done(unsigned launches = 1) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch(launches);
  return TFCCB200_OK;
}

unsigned flat_grid(size_t n, int sm_count) {
  size_t blocks = (n + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count) * 16;
  if (blocks > cap) blocks = cap;
  return static_cast<unsigned>(blocks ? blocks : 1);
}

}  // namespace

int softmax_f32(cudaStream_t stream, const float* src, unsigned rows, unsigned cols, float scale,
                float* dst) {
  const unsigned blocks = (rows + 7) / 8;
  if (cols % 4 == 0 && cols >= 128 && cols <= 1024 &&
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
    const unsigned vecs = cols / 4;
#define TFCCB200_SOFTMAXV(V)                                                                  \
  launch_after_previous(softmax_rows_vec_kernel<V>, dim3(blocks), dim3(256), 0, stream,       \
                        reinterpret_cast<const float4*>(src), rows, vecs, scale,              \
                        reinterpret_cast<float4*>(dst))
    if (vecs <= 32) TFCCB200_SOFTMAXV(1);
    else if (vecs <= 64) TFCCB200_SOFTMAXV(2);
    else if (vecs <= 128) TFCCB200_SOFTMAXV(4);
    else TFCCB200_SOFTMAXV(8);
#undef TFCCB200_SOFTMAXV
    return done();
  }
#define TFCCB200_SOFTMAX(P)                                                                   \
  launch_after_previous(softmax_rows_kernel<P>, dim3(blocks), dim3(256), 0, stream, src, rows, cols,  \
                        scale, dst)
  if (cols <= 32) TFCCB200_SOFTMAX(1);
  else if (cols <= 64) TFCCB200_SOFTMAX(2);
  else if (cols <= 128) TFCCB200_SOFTMAX(4);
  else if (cols <= 256) TFCCB200_SOFTMAX(8);
  else if (cols <= 512) TFCCB200_SOFTMAX(16);
  else if (cols <= 1024) TFCCB200_SOFTMAX(32);
  else launch_after_previous(softmax_long_rows_kernel, dim3(rows), dim3(256), 0, stream, src, cols,
                             scale, dst);
#undef TFCCB200_SOFTMAX
  return done();
}

int layer_norm_f32(cudaStream_t stream, const float* x, const float* residual, const float* gamma,
                   const float* beta, float eps, unsigned rows, unsigned cols, float* dst) {
  if (cols > 32u * kMaxPerLane) {
    launch_after_previous(layer_norm_long_rows_kernel, dim3(rows), dim3(256), 0, stream, x, residual,
                          gamma, beta, eps, cols, dst);
    return done();
  }
  const unsigned blocks = (rows + 7) / 8;
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (cols % 4 == 0 && a16(x) && a16(residual) && a16(gamma) && a16(beta) && a16(dst)) {
    const unsigned vecs = cols / 4;
#define TFCCB200_LNV(V)                                                                       \
  launch_after_previous(layer_norm_vec_kernel<V>, dim3(blocks), dim3(256), 0, stream,         \
                        reinterpret_cast<const float4*>(x),                                   \
                        reinterpret_cast<const float4*>(residual),                            \
                        reinterpret_cast<const float4*>(gamma),                               \
                        reinterpret_cast<const float4*>(beta), eps, rows, vecs,               \
                        reinterpret_cast<float4*>(dst))
    if (vecs <= 32) TFCCB200_LNV(1);
    else if (vecs <= 64) TFCCB200_LNV(2);
    else if (vecs <= 128) TFCCB200_LNV(4);
    else if (vecs <= 192) TFCCB200_LNV(6);
    else TFCCB200_LNV(8);
#undef TFCCB200_LNV
    return done();
  }
#define TFCCB200_LN(P)                                                                        \
  launch_after_previous(layer_norm_kernel<P>, dim3(blocks), dim3(256), 0, stream, x, residual,   \
                        gamma, beta, eps, rows, cols, dst)
  if (cols <= 128) TFCCB200_LN(4);
  else if (cols <= 256) TFCCB200_LN(8);
  else if (cols <= 512) TFCCB200_LN(16);
  else if (cols <= 768) TFCCB200_LN(24);
  else TFCCB200_LN(32);
#undef TFCCB200_LN
  return done();
}

int gelu_f32(cudaStream_t stream, const float* src, size_t n, float* dst) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  if (n % 4 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
    launch_after_previous(gelu_vec_kernel, dim3(flat_grid(n / 4, di->sm_count)), dim3(256), 0, stream,
                          reinterpret_cast<const float4*>(src), n / 4,
                          reinterpret_cast<float4*>(dst));
    return done();
  }
  launch_after_previous(gelu_kernel, dim3(flat_grid(n, di->sm_count)), dim3(256), 0, stream, src, n,
                        dst);
  return done();
}

int permute_0213_f32(cudaStream_t stream, const float* src, unsigned d0, unsigned d1, unsigned d2,
                     unsigned d3, float* dst) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  const size_t n = static_cast<size_t>(d0) * d1 * d2 * d3;
  if (d3 % 4 == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
    launch_after_previous(permute_0213_vec_kernel, dim3(flat_grid(n / 4, di->sm_count)), dim3(256), 0,
                          stream, reinterpret_cast<const float4*>(src), d0, d1, d2, d3 / 4,
                          reinterpret_cast<float4*>(dst));
    return done();
  }
  launch_after_previous(permute_0213_kernel, dim3(flat_grid(n, di->sm_count)), dim3(256), 0,
                        stream, src, d0, d1, d2, d3, dst);
  return done();
}

int transpose_last2_f32(cudaStream_t stream, const float* src, unsigned batch, unsigned r,
                        unsigned c, float* dst) {
  if (batch > 65535 || (r + 31) / 32 > 65535) return TFCCB200_EOVERFLOW;
  dim3 grid((c + 31) / 32, (r + 31) / 32, batch);
  launch_after_previous(transpose_last2_kernel, grid, dim3(256), 0, stream, src, r, c, dst);
  return done();
}

}  // namespace tfccb200
