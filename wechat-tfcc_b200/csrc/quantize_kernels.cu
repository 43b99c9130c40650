// quantize / dequantize / requantize on the device, with the reference's exact scalar math
// (double precision, C round() = half away from zero, clamp to the integer type):
//   get_quantized_scale_info / get_dequantized_scale_info / quantize_one
//   (tfcc/core/utils/tfcc_quantizationutils.h:45-79) and the element loops of
//   tfcc/mkl/kernel/tfcc_mklquantizationkernel.hpp:21-64.
// The (min, max) ranges stay on the device: every thread derives scale and offset from the
// two floats itself (IEEE double arithmetic gives the host's bits), so no host round trip or
// synchronisation is needed between the range reduction and the conversion.
#include <cuda_runtime.h>

#include "internal.h"
#include "pdl.cuh"

namespace tfccb200 {

namespace {

template <class T>
struct Limits;
template <> struct Limits<int8_t> { static constexpr long long lo = -128, hi = 127; };
template <> struct Limits<uint8_t> { static constexpr long long lo = 0, hi = 255; };
template <> struct Limits<int16_t> { static constexpr long long lo = -32768, hi = 32767; };
template <> struct Limits<uint16_t> { static constexpr long long lo = 0, hi = 65535; };
template <> struct Limits<int32_t> { static constexpr long long lo = -2147483648LL, hi = 2147483647LL; };
template <> struct Limits<uint32_t> { static constexpr long long lo = 0, hi = 4294967295LL; };

template <class T>
__device__ __forceinline__ void quantized_scale_info(float min_value, float max_value,
                                                     double* scale, long long* offset) {
  const long long step_cnt = 1LL << (sizeof(T) * 8);
  const double range_adjust = step_cnt / (step_cnt - 1.0);
  const double range = (max_value - min_value) * range_adjust;  // float subtraction, as the reference
  const double range_scale = step_cnt / range;
  *scale = range_scale;
  *offset = static_cast<long long>(round(__dmul_rn(static_cast<double>(min_value), range_scale)));
}

template <class T>
__device__ __forceinline__ void dequantized_scale_info(float min_value, float max_value,
                                                       double* scale, double* min_rounded) {
  const long long step_cnt = 1LL << (sizeof(T) * 8);
  const double range_adjust = step_cnt / (step_cnt - 1.0);
  const double range = (max_value - min_value) * range_adjust;
  *scale = range / step_cnt;
  *min_rounded = min_value;
}

template <class T>
__device__ __forceinline__ T quantize_value(double real, double scale, long long offset) {
  long long q = static_cast<long long>(round(__dmul_rn(real, scale))) - offset;
  q += Limits<T>::lo;
  q = max(q, Limits<T>::lo);
  q = min(q, Limits<T>::hi);
  return static_cast<T>(q);
}

// ---- min / max of a float tensor -------------------------------------------------------
// Floats are mapped to unsigned keys whose order is the floats' order, so that integer
// atomics can combine the per-block results; out[0..1] hold keys between the init and the
// decode kernels and floats afterwards.
__device__ __forceinline__ unsigned float_key(float f) {
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// ---- element-wise skeleton -----------------------------------------------------------------
// dst[i] = f(src[i]) for n elements.  These passes are bound by memory bandwidth, so the bulk
// moves in the widest words both sides allow: a thread takes E = 16 / max(sizeof) adjacent
// elements per step -- one 128-bit word on the wider side, 32 to 128 bits on the narrower --
// consecutive threads take consecutive words (every warp instruction reads or writes one
// contiguous run), and four steps' loads are requested before the first is used.  Pointers that
// are not aligned to those words, and the ragged end, go element by element.
template <int BYTES> struct WordOf;
template <> struct WordOf<4> { using type = uint32_t; };
template <> struct WordOf<8> { using type = uint2; };
template <> struct WordOf<16> { using type = uint4; };

template <class TI, class TO, class F>
__device__ __forceinline__ void map_elements(const TI* __restrict__ src, TO* __restrict__ dst,
                                             size_t n, F f) {
  constexpr int kWide = sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO);
  constexpr int E = 16 / kWide;
  using WI = typename WordOf<E * sizeof(TI)>::type;
  using WO = typename WordOf<E * sizeof(TO)>::type;
  constexpr int U = 4;
  const size_t tid = blockIdx.x * 256ull + threadIdx.x, stride = gridDim.x * 256ull;
  size_t done = 0;
  if ((reinterpret_cast<uintptr_t>(src) & (sizeof(WI) - 1)) == 0 &&
      (reinterpret_cast<uintptr_t>(dst) & (sizeof(WO) - 1)) == 0) {
    const size_t steps = n / E;
    const WI* in = reinterpret_cast<const WI*>(src);
    WO* out = reinterpret_cast<WO*>(dst);
    auto convert = [&](const WI& w) {
      WO o;
      const TI* e = reinterpret_cast<const TI*>(&w);
      TO* q = reinterpret_cast<TO*>(&o);
#pragma unroll
      for (int v = 0; v < E; ++v) q[v] = f(e[v]);
      return o;
    };
    size_t i = tid;
    for (; i + (U - 1) * stride < steps; i += U * stride) {
      WI w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) w[u] = __ldcs(in + i + u * stride);
#pragma unroll
      for (int u = 0; u < U; ++u) out[i + u * stride] = convert(w[u]);
    }
    for (; i < steps; i += stride) out[i] = convert(__ldcs(in + i));
    done = steps * E;
  }
  for (size_t i = done + tid; i < n; i += stride) dst[i] = f(src[i]);
}

__global__ void minmax_init_kernel(unsigned* out) {
  out[0] = 0xffffffffu;  // larger than every key
  out[1] = 0u;
}

__global__ void __launch_bounds__(256)
minmax_reduce_kernel(const float* __restrict__ src, size_t n, unsigned* out) {
  float lo = 3.402823466e+38f, hi = -3.402823466e+38f;  // std::numeric_limits<float>::max / lowest
  const size_t tid = blockIdx.x * 256ull + threadIdx.x, stride = gridDim.x * 256ull;
  size_t done = 0;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {  // 128-bit loads, four in flight
    const size_t steps = n / 4;
    const float4* in = reinterpret_cast<const float4*>(src);
    auto take = [&](const float4& v) {
      lo = fminf(fminf(lo, v.x), fminf(v.y, fminf(v.z, v.w)));
      hi = fmaxf(fmaxf(hi, v.x), fmaxf(v.y, fmaxf(v.z, v.w)));
    };
    size_t i = tid;
    for (; i + 3 * stride < steps; i += 4 * stride) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcs(in + i + u * stride);
#pragma unroll
      for (int u = 0; u < 4; ++u) take(v[u]);
    }
    for (; i < steps; i += stride) take(__ldcs(in + i));
    done = steps * 4;
  }
  for (size_t i = done + tid; i < n; i += stride) {
    const float v = src[i];
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  __shared__ float slo[8], shi[8];
  if ((threadIdx.x & 31) == 0) {
    slo[threadIdx.x >> 5] = lo;
    shi[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) {
      lo = fminf(lo, slo[w]);
      hi = fmaxf(hi, shi[w]);
    }
    atomicMin(out, float_key(lo));
    atomicMax(out + 1, float_key(hi));
  }
}

__global__ void minmax_decode_kernel(unsigned* out) {
  const float lo = key_float(out[0]), hi = key_float(out[1]);
  reinterpret_cast<float*>(out)[0] = lo;
  reinterpret_cast<float*>(out)[1] = hi;
}

// ---- scalars of the quantized matmul from device-resident ranges -----------------------------
// offA = round(minA * scaleA) - lowest(u8), offB = round(minB * scaleB) - lowest(s8) and the
// float range of the int32 result, as tfcc::mkl::quantization::matmul derives them on the
// host (tfcc/mkl/operations/tfcc_mklquantization.cpp:181-193,
// get_quantization_range_for_multiplication, tfcc/core/utils/tfcc_quantizationutils.h:23-43):
// same double / float operations, none of them fused.
__global__ void qmatmul_params_kernel(const float* __restrict__ minA, const float* __restrict__ maxA,
                                      const float* __restrict__ minB, const float* __restrict__ maxB,
                                      int32_t* __restrict__ offsets, float* __restrict__ minC,
                                      float* __restrict__ maxC) {
  // one thread in front of the product: it is launched to overlap the tail of the kernel before
  // it, and lets the product's own preamble (barriers, tensor memory) run beside it
  pdl_release();
  pdl_wait();
  double scale;
  long long off;
  quantized_scale_info<uint8_t>(*minA, *maxA, &scale, &off);
  offsets[0] = static_cast<int32_t>(off - Limits<uint8_t>::lo);
  quantized_scale_info<int8_t>(*minB, *maxB, &scale, &off);
  offsets[1] = static_cast<int32_t>(off - Limits<int8_t>::lo);
  const float a_level = __fdiv_rn(__fsub_rn(*maxA, *minA), 255.0f);
  const float b_level = __fdiv_rn(__fsub_rn(*maxB, *minB), 255.0f);
  const float c_level = __fmul_rn(a_level, b_level);
  *minC = __fmul_rn(c_level, static_cast<float>(Limits<int32_t>::lo));
  *maxC = __fmul_rn(c_level, static_cast<float>(Limits<int32_t>::hi));
}

// ---- element kernels ---------------------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(256)
quantize_kernel(const float* __restrict__ src, size_t n, const float* __restrict__ pmin,
                const float* __restrict__ pmax, T* __restrict__ dst) {
  const float mn = *pmin, mx = *pmax;
  const bool degenerate = mn >= mx;  // also the "all values equal" case of quantize(a)
  double scale = 0;
  long long offset = 0;
  if (!degenerate) quantized_scale_info<T>(mn, mx, &scale, &offset);
  map_elements(src, dst, n, [&](float v) {
    return degenerate ? static_cast<T>(Limits<T>::lo)
                      : quantize_value<T>(static_cast<double>(v), scale, offset);
  });
}

// quantize with the row sums of the quantized values produced in the same pass: the
// `quantize<u8>(x)` followed by `reduce_sum(q, row)` of a quantized dense layer
// (tfcc/test/quantization.cpp:105-121) without reading q back.  One CTA of 256 threads per row
// group; a thread converts four adjacent floats per step (one 128-bit load) and keeps its share
// of the row's integer sum; warps combine with shuffles, the row's warps through shared memory.
template <class T, int TPR>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const float* __restrict__ src, unsigned rows, unsigned cols,
                     const float* __restrict__ pmin, const float* __restrict__ pmax,
                     T* __restrict__ dst, int32_t* __restrict__ row_sums) {
  constexpr int kRowsPerCta = 256 / TPR;
  __shared__ int32_t warp_sums[8];
  const float mn = *pmin, mx = *pmax;
  const bool degenerate = mn >= mx;
  double scale = 0;
  long long offset = 0;
  if (!degenerate) quantized_scale_info<T>(mn, mx, &scale, &offset);
  const unsigned row = blockIdx.x * kRowsPerCta + threadIdx.x / TPR;
  const unsigned t = threadIdx.x % TPR;
  int32_t s = 0;
  if (row < rows) {
    const float* p = src + static_cast<size_t>(row) * cols;
    T* q = dst + static_cast<size_t>(row) * cols;
    auto one = [&](float v) {
      const T r = degenerate ? static_cast<T>(Limits<T>::lo)
                             : quantize_value<T>(static_cast<double>(v), scale, offset);
      s += static_cast<int32_t>(r);
      return r;
    };
    const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0 &&
                     (reinterpret_cast<uintptr_t>(q) & (4 * sizeof(T) - 1)) == 0;
    if (vec) {
      auto put = [&](unsigned i, const float4& v) {
        T r[4] = {one(v.x), one(v.y), one(v.z), one(v.w)};
        if constexpr (sizeof(T) == 1) {
          reinterpret_cast<uint32_t*>(q)[i] = *reinterpret_cast<const uint32_t*>(r);
        } else {
          reinterpret_cast<uint2*>(q)[i] = *reinterpret_cast<const uint2*>(r);
        }
      };
      const unsigned vecs = cols / 4;
      unsigned i = t;
      for (; i + 3 * TPR < vecs; i += 4 * TPR) {  // four loads requested before the first is used
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const float4*>(p) + i + u * TPR);
#pragma unroll
        for (int u = 0; u < 4; ++u) put(i + u * TPR, v[u]);
      }
      for (; i < vecs; i += TPR) put(i, __ldcs(reinterpret_cast<const float4*>(p) + i));
    } else {
      for (unsigned i = t; i < cols; i += TPR) q[i] = one(p[i]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if constexpr (TPR == 32) {
    if (t == 0 && row < rows) row_sums[row] = s;
  } else {
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
    __syncthreads();
    if (t == 0 && row < rows) {
      int32_t total = 0;
#pragma unroll
      for (int w = 0; w < TPR / 32; ++w) total += warp_sums[(threadIdx.x >> 5) + w];
      row_sums[row] = total;
    }
  }
}

template <class T>
__global__ void __launch_bounds__(256)
dequantize_kernel(const T* __restrict__ src, size_t n, const float* __restrict__ pmin,
                  const float* __restrict__ pmax, float* __restrict__ dst) {
  const float mn = *pmin, mx = *pmax;
  const bool degenerate = mn >= mx;
  double scale = 0, min_rounded = 0;
  if (!degenerate) dequantized_scale_info<T>(mn, mx, &scale, &min_rounded);
  map_elements(src, dst, n, [&](T q) {
    const double off = static_cast<double>(q) - static_cast<double>(Limits<T>::lo);
    // separate multiply and add, each rounded: the reference's expression is not fused
    return degenerate ? mn : static_cast<float>(__dadd_rn(min_rounded, __dmul_rn(off, scale)));
  });
}

template <class TI, class TO>
__global__ void __launch_bounds__(256)
requantize_kernel(const TI* __restrict__ src, size_t n, const float* __restrict__ pmin_in,
                  const float* __restrict__ pmax_in, const float* __restrict__ pmin_out,
                  const float* __restrict__ pmax_out, TO* __restrict__ dst) {
  const float min_in = *pmin_in, max_in = *pmax_in, min_out = *pmin_out, max_out = *pmax_out;
  // the three cases of _requantize_helper (tfcc/mkl/interfaces/tfcc_mklquantizationinterface.cpp:114-140)
  if (min_out >= max_out) {
    map_elements(src, dst, n, [](TI) { return static_cast<TO>(Limits<TO>::lo); });
    return;
  }
  double in_scale, in_min, out_scale;
  long long out_offset;
  dequantized_scale_info<TI>(min_in, max_in, &in_scale, &in_min);
  quantized_scale_info<TO>(min_out, max_out, &out_scale, &out_offset);
  if (min_in >= max_in) {
    const TO q = quantize_value<TO>(static_cast<double>(min_in), out_scale, out_offset);
    map_elements(src, dst, n, [q](TI) { return q; });
    return;
  }
  map_elements(src, dst, n, [&](TI v) {
    const double off = static_cast<double>(v) - static_cast<double>(Limits<TI>::lo);
    return quantize_value<TO>(__dadd_rn(in_min, __dmul_rn(off, in_scale)), out_scale, out_offset);
  });
}

unsigned grid_for(size_t n, int sm_count) {
  size_t blocks = (n + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count) * 8;
  if (blocks > cap) blocks = cap;
  return static_cast<unsigned>(blocks ? blocks : 1);
}

template <class F>
int dispatch_type(int type, F&& f) {
  switch (type) {
    case TFCCB200_TYPE_S8: return f(int8_t());
    case TFCCB200_TYPE_U8: return f(uint8_t());
    case TFCCB200_TYPE_S16: return f(int16_t());
    case TFCCB200_TYPE_U16: return f(uint16_t());
    case TFCCB200_TYPE_S32: return f(int32_t());
    case TFCCB200_TYPE_U32: return f(uint32_t());
    default: return TFCCB200_EINVAL;
  }
}

int finish(unsigned launches) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch(launches);
  return TFCCB200_OK;
}

}  // namespace

int minmax_f32(cudaStream_t stream, const float* src, size_t n, float* out) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  unsigned* keys = reinterpret_cast<unsigned*>(out);
  minmax_init_kernel<<<1, 1, 0, stream>>>(keys);
  minmax_reduce_kernel<<<grid_for(n, di->sm_count), 256, 0, stream>>>(src, n, keys);
  minmax_decode_kernel<<<1, 1, 0, stream>>>(keys);
  return finish(3);
}

int quantize_f32(cudaStream_t stream, const float* src, size_t n, const float* pmin,
                 const float* pmax, void* dst, int dst_type) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  const unsigned grid = grid_for(n, di->sm_count);
  return dispatch_type(dst_type, [&](auto tag) {
    using T = decltype(tag);
    quantize_kernel<T><<<grid, 256, 0, stream>>>(src, n, pmin, pmax, static_cast<T*>(dst));
    return finish(1);
  });
}

int quantized_matmul_params_dev(cudaStream_t stream, const float* minA, const float* maxA,
                                const float* minB, const float* maxB, int32_t* offsets,
                                float* minC, float* maxC) {
  cudaError_t e = launch_after_previous(qmatmul_params_kernel, dim3(1), dim3(1), 0, stream, minA, maxA,
                                        minB, maxB, offsets, minC, maxC);
  if (e != cudaSuccess) return static_cast<int>(e);
  return finish(1);
}

int quantize_rows_f32(cudaStream_t stream, const float* src, unsigned rows, unsigned cols,
                      const float* pmin, const float* pmax, void* dst, int dst_type,
                      int32_t* row_sums) {
  auto run = [&](auto tag) {
    using T = decltype(tag);
    T* out = static_cast<T*>(dst);
    if (cols <= 256) {
      quantize_rows_kernel<T, 32><<<(rows + 7) / 8, 256, 0, stream>>>(src, rows, cols, pmin, pmax,
                                                                      out, row_sums);
    } else if (cols <= 1024) {
      quantize_rows_kernel<T, 128><<<(rows + 1) / 2, 256, 0, stream>>>(src, rows, cols, pmin, pmax,
                                                                       out, row_sums);
    } else {
      quantize_rows_kernel<T, 256><<<rows, 256, 0, stream>>>(src, rows, cols, pmin, pmax, out,
                                                             row_sums);
    }
    return finish(1);
  };
  switch (dst_type) {  // the types reduce_sum exists for
    case TFCCB200_TYPE_S8: return run(int8_t());
    case TFCCB200_TYPE_U8: return run(uint8_t());
    case TFCCB200_TYPE_S16: return run(int16_t());
    default: return TFCCB200_EINVAL;
  }
}

int dequantize_f32(cudaStream_t stream, const void* src, int src_type, size_t n, const float* pmin,
                   const float* pmax, float* dst) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  const unsigned grid = grid_for(n, di->sm_count);
  return dispatch_type(src_type, [&](auto tag) {
    using T = decltype(tag);
    dequantize_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(src), n, pmin, pmax, dst);
    return finish(1);
  });
}

int requantize(cudaStream_t stream, const void* src, int src_type, size_t n, const float* pmin_in,
               const float* pmax_in, const float* pmin_out, const float* pmax_out, void* dst,
               int dst_type) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  const unsigned grid = grid_for(n, di->sm_count);
  return dispatch_type(src_type, [&](auto in_tag) {
    using TI = decltype(in_tag);
    return dispatch_type(dst_type, [&](auto out_tag) {
      using TO = decltype(out_tag);
      requantize_kernel<TI, TO><<<grid, 256, 0, stream>>>(static_cast<const TI*>(src), n, pmin_in,
                                                          pmax_in, pmin_out, pmax_out,
                                                          static_cast<TO*>(dst));
      return finish(1);
    });
  });
}

}  // namespace tfccb200
