// extern "C" surface of libtfcc_b200: argument checks, kernel-path choice and
// the host-buffer convenience forms.  Nothing here throws.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <limits>
#include <mutex>
#include <vector>

#include "internal.h"

namespace tfccb200 {

namespace {
std::atomic<unsigned long long> g_launches{0};
constexpr int kMaxDevices = 64;
DeviceInfo g_info[kMaxDevices];
std::once_flag g_info_once[kMaxDevices];
cudaError_t g_info_err[kMaxDevices];
}  // namespace

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

const DeviceInfo* current_device_info(cudaError_t* err) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *err = (e != cudaSuccess) ? e : cudaErrorInvalidDevice;
    return nullptr;
  }
  std::call_once(g_info_once[dev], [dev] {
    cudaDeviceProp prop;
    g_info_err[dev] = cudaGetDeviceProperties(&prop, dev);
    if (g_info_err[dev] == cudaSuccess) {
      g_info[dev].sm_count = prop.multiProcessorCount;
      g_info[dev].cc_major = prop.major;
      g_info[dev].cc_minor = prop.minor;
      g_info[dev].l2_bytes = static_cast<size_t>(prop.l2CacheSize);
    }
  });
  if (g_info_err[dev] != cudaSuccess) {
    *err = g_info_err[dev];
    return nullptr;
  }
  return &g_info[dev];
}

namespace {

// A rank-2 B next to a batched, densely packed A is one tall GEMM: the batch
// folds into M (the reference CUDA backend does the same before cublasGemmEx,
// tfcc/cuda/interfaces/tfcc_cudablasinterface.cu:224-236).
template <class Args>
void fold_batch(Args& a) {
  if (a.batch > 1 && a.strideB == 0 && a.strideA == a.M * a.K && a.strideC == a.M * a.N &&
      static_cast<unsigned long long>(a.M) * a.batch <= 0xffffffffull) {
    a.M *= a.batch;
    a.batch = 1;
  }
}

bool shape_overflows(unsigned M, unsigned N, unsigned K, unsigned batch) {
  // TFCC's Shape keeps the element count of a tensor in 32 bits
  // (tfcc/core/framework/tfcc_shape.h:24-81).
  const unsigned long long lim = 0xffffffffull;
  return static_cast<unsigned long long>(M) * K > lim ||
         static_cast<unsigned long long>(K) * N > lim ||
         static_cast<unsigned long long>(M) * N * batch > lim;
}

int pick_sgemm_path(const SgemmArgs& a) {
  // Few rows and a B of at most 16 MB (it stays in L2 for the other row groups): one launch of
  // the CUDA-core kernel that adds its K slices inside a cluster.
  // (B is re-read by every group of 8 rows, so with more than 16 rows it has to be smaller:
  // measured 32x512x2048 7.7 us against 12.3 on the tensor cores, 32x768x3072 18.4 against 15.8.)
  const unsigned long long b_elems = static_cast<unsigned long long>(a.K) * a.N;
  if (a.M <= 32 && b_elems >= (1ull << 14) && b_elems <= (a.M <= 16 ? (1ull << 22) : (1ull << 21)) &&
      cluster_simt_sgemm_supported(a))
    return TFCCB200_PATH_CLUSTER_SIMT;
  // Up to 16 rows the streaming kernel wins wherever the weights dominate the traffic (measured
  // 16x4096x16384: 73 us against 99 us on the tensor-core path, 12x4096x4096: 25 against 37);
  // from 17 rows on its FMA work per weight outgrows what the bandwidth leaves time for
  // (32x4096x16384: 121 against 99), so those go to the tensor cores.
  if (a.M <= 16 && skinny_sgemm_supported(a) &&
      static_cast<unsigned long long>(a.K) * a.N >= (1ull << 16))
    return TFCCB200_PATH_SKINNY;
  const unsigned long long macs = static_cast<unsigned long long>(a.M) * a.N * a.K * a.batch;
  if (umma_sgemm_supported(a) && macs >= (1ull << 22) && a.K >= 32 && a.N >= 64) {
    cudaError_t e;
    const DeviceInfo* di = current_device_info(&e);
    const int sms = di ? di->sm_count : 148;
    const bool fp32 = a.precision == TFCCB200_PRECISION_FP32;
    return umma_plan(a.M, a.N, a.K, a.batch, sms, a.precision == TFCCB200_PRECISION_BF16 ? 2 : 4, -1,
                     fp32, fp32 && stream_k_scratch_ok(a, sms))
               .pair ? TFCCB200_PATH_UMMA2
                                                             : TFCCB200_PATH_UMMA;
  }
  return TFCCB200_PATH_SIMT;
}

int run_sgemm(SgemmArgs a, int path) {
  if (!a.A || !a.B || !a.C) return TFCCB200_EINVAL;
  if (a.M == 0 || a.N == 0 || a.K == 0 || a.batch == 0) return TFCCB200_EINVAL;
  if (a.precision != TFCCB200_PRECISION_FP32 && a.precision != TFCCB200_PRECISION_TF32 &&
      a.precision != TFCCB200_PRECISION_BF16)
    return TFCCB200_EINVAL;
  if (shape_overflows(a.M, a.N, a.K, a.batch)) return TFCCB200_EOVERFLOW;
  if (a.batch == 1) a.strideA = a.strideB = 0, a.strideC = a.M * a.N;
  fold_batch(a);
  if (path == TFCCB200_PATH_AUTO) path = pick_sgemm_path(a);
  // The bfloat16 mode exists on the tensor-core paths only, for pitches that are multiples of
  // 8 elements; anything else is computed in fp32, which is within every bfloat16 tolerance.
  if (a.precision == TFCCB200_PRECISION_BF16 &&
      ((path != TFCCB200_PATH_UMMA && path != TFCCB200_PATH_UMMA2) || a.K % 8 || a.N % 8))
    a.precision = TFCCB200_PRECISION_FP32;
  switch (path) {
    case TFCCB200_PATH_SIMT: return simt_sgemm(a);
    case TFCCB200_PATH_SKINNY: return skinny_sgemm(a);
    case TFCCB200_PATH_CLUSTER_SIMT: return cluster_simt_sgemm(a);
    case TFCCB200_PATH_UMMA: return umma_sgemm(a, false);
    case TFCCB200_PATH_UMMA2: return umma_sgemm(a, true);
    default: return TFCCB200_EINVAL;
  }
}

int pick_qgemm_path(const QgemmArgs& a) {
  const unsigned long long macs = static_cast<unsigned long long>(a.M) * a.N * a.K * a.batch;
  if (umma_qgemm_supported(a) && macs >= (1ull << 22) && a.K >= 128 && a.N >= 128) {
    cudaError_t e;
    const DeviceInfo* di = current_device_info(&e);
    const int sms = di ? di->sm_count : 148;
    return umma_qgemm_prefers_pair(a.M, a.N, a.K, a.batch, sms) ? TFCCB200_PATH_UMMA2
                                                                  : TFCCB200_PATH_UMMA;
  }
  return TFCCB200_PATH_SIMT;
}

int run_qgemm(QgemmArgs a, int path) {
  if (!a.A || !a.B || !a.C || !a.rsA || !a.rsB) return TFCCB200_EINVAL;
  if (a.M == 0 || a.N == 0 || a.K == 0 || a.batch == 0) return TFCCB200_EINVAL;
  if (shape_overflows(a.M, a.N, a.K, a.batch)) return TFCCB200_EOVERFLOW;
  if (a.batch == 1) a.strideA = a.strideB = 0, a.strideC = a.M * a.N;
  // Same fold as the reference: a single B matrix turns the batch into rows
  // (tfcc/mkl/operations/tfcc_mklquantization.cpp:140-145).
  if (a.batch > 1 && a.strideB == 0 && a.strideA == a.M * a.K && a.strideC == a.M * a.N &&
      a.strideRsB == 0 && (a.strideRsA == a.M) &&
      static_cast<unsigned long long>(a.M) * a.batch <= 0xffffffffull) {
    a.M *= a.batch;
    a.batch = 1;
  }
  if (path == TFCCB200_PATH_AUTO) path = pick_qgemm_path(a);
  switch (path) {
    case TFCCB200_PATH_SIMT: return simt_qgemm(a);
    case TFCCB200_PATH_UMMA: return umma_qgemm(a, false);
    case TFCCB200_PATH_UMMA2: return umma_qgemm(a, true);
    default: return TFCCB200_EINVAL;
  }
}

template <class T>
int reduce_sum_checked(void* stream, const T* src, unsigned batch, unsigned rows, unsigned cols,
                       int row_flag, int32_t* dst) {
  if (!src || !dst || batch == 0 || rows == 0 || cols == 0) return TFCCB200_EINVAL;
  if (static_cast<unsigned long long>(batch) * rows * cols > 0xffffffffull)
    return TFCCB200_EOVERFLOW;
  return reduce_sum<T>(static_cast<cudaStream_t>(stream), src, batch, rows, cols, row_flag, dst);
}

// get_quantized_scale_info<T> of the reference for 8-bit T: scale = 256 /
// ((max - min) * 256/255) in double, offset = round(min * scale).
int64_t quantized_offset_8bit(float minv, float maxv) {
  const double step_cnt = 256.0;
  const double range_adjust = step_cnt / (step_cnt - 1.0);
  const double range = (static_cast<double>(maxv - minv)) * range_adjust;
  const double range_scale = step_cnt / range;
  return static_cast<int64_t>(std::round(minv * range_scale));
}

// Scoped helpers for the host-buffer entry points.
struct ScopedStream {
  cudaStream_t s = nullptr;
  cudaError_t create() { return cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking); }
  ~ScopedStream() {
    if (s) cudaStreamDestroy(s);
  }
};
struct ScopedEvent {
  cudaEvent_t e = nullptr;
  cudaError_t create() { return cudaEventCreateWithFlags(&e, cudaEventDisableTiming); }
  ~ScopedEvent() {
    if (e) cudaEventDestroy(e);
  }
};

// The staging buffers of the host-buffer entry points come from a stream-ordered pool that
// belongs to this library (one per device, created on first use, kept until the process
// exits).  Its release threshold is unlimited, so the pool keeps the memory between calls
// instead of returning it to the driver at every synchronisation; the device's default pool
// and its settings are left alone.
cudaError_t staging_pool(cudaMemPool_t* out) {
  static std::mutex mu;
  static cudaMemPool_t pools[kMaxDevices] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t pool = nullptr;
    if ((e = cudaMemPoolCreate(&pool, &props)) != cudaSuccess) return e;
    unsigned long long threshold = ~0ull;
    if ((e = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold)) !=
        cudaSuccess) {
      cudaMemPoolDestroy(pool);
      return e;
    }
    pools[dev] = pool;
  }
  *out = pools[dev];
  return cudaSuccess;
}

struct DeviceBuffer {
  void* p = nullptr;
  cudaStream_t s;
  explicit DeviceBuffer(cudaStream_t st) : s(st) {}
  cudaError_t alloc(size_t bytes) {
    cudaMemPool_t pool;
    cudaError_t e = staging_pool(&pool);
    if (e != cudaSuccess) return e;
    return cudaMallocFromPoolAsync(&p, bytes ? bytes : 16, pool, s);
  }
  ~DeviceBuffer() {
    if (p) cudaFreeAsync(p, s);
  }
};

// Leaving a host-buffer call early must not leave copies in flight: they touch the caller's
// host buffers, and the staging buffers are freed in the caller's stream order only.  While
// armed, the destructor waits for every stream the call has used.
struct JoinStreams {
  cudaStream_t streams[3] = {nullptr, nullptr, nullptr};
  int count = 0;
  bool armed = true;
  void add(cudaStream_t st) { streams[count++] = st; }
  ~JoinStreams() {
    if (!armed) return;
    for (int i = 0; i < count; ++i) cudaStreamSynchronize(streams[i]);
  }
};

}  // namespace
}  // namespace tfccb200

using namespace tfccb200;

extern "C" {

const char* tfccb200_strerror(int status) {
  switch (status) {
    case TFCCB200_OK: return "ok";
    case TFCCB200_EINVAL: return "invalid argument";
    case TFCCB200_EALIGN: return "operand alignment not supported by the requested kernel path";
    case TFCCB200_EWORKSPACE: return "workspace missing, misaligned or too small";
    case TFCCB200_EOVERFLOW: return "element count exceeds the 32-bit shape limit";
    case TFCCB200_EUNSUPPORTED: return "requested kernel path cannot run this problem";
    case TFCCB200_EDEVICE: return "a kernel abandoned a bounded wait";
    case TFCCB200_ESTATICLIMIT:
      return "problem needs more scratch than the library's built-in 20 MiB array holds";
    default:
      if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
      return "unknown status";
  }
}

int tfccb200_version(void) { return 100; }

void tfccb200_test_flag_wait(unsigned long long timeout_ns, unsigned expect_extra) {
  set_test_flag_wait(timeout_ns, expect_extra);
}

unsigned long long tfccb200_launch_count(void) {
  return g_launches.load(std::memory_order_relaxed);
}

int tfccb200_sgemm_ex(void* stream, const float* A, unsigned strideA, const float* B,
                      unsigned strideB, float* C, unsigned strideC, const float* bias, unsigned M,
                      unsigned N, unsigned K, unsigned batch, int precision_mode, int path,
                      void* workspace, size_t workspace_bytes, int* device_status) {
  return tfccb200_sgemm_act(stream, A, strideA, B, strideB, C, strideC, bias, M, N, K, batch,
                            precision_mode, path, TFCCB200_ACT_NONE, workspace, workspace_bytes,
                            device_status);
}

int tfccb200_sgemm_act(void* stream, const float* A, unsigned strideA, const float* B,
                       unsigned strideB, float* C, unsigned strideC, const float* bias, unsigned M,
                       unsigned N, unsigned K, unsigned batch, int precision_mode, int path,
                       int activation, void* workspace, size_t workspace_bytes,
                       int* device_status) {
  if (activation != TFCCB200_ACT_NONE && activation != TFCCB200_ACT_GELU_ERF)
    return TFCCB200_EINVAL;
  SgemmArgs a = {};
  a.activation = activation;
  a.stream = static_cast<cudaStream_t>(stream);
  a.A = A; a.B = B; a.C = C; a.bias = bias;
  a.strideA = strideA; a.strideB = strideB; a.strideC = strideC;
  a.M = M; a.N = N; a.K = K; a.batch = batch;
  a.precision = precision_mode;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.status = device_status;
  return run_sgemm(a, path);
}

int tfccb200_sgemm(void* stream, const float* A, unsigned strideA, const float* B,
                   unsigned strideB, float* C, unsigned strideC, const float* bias, unsigned M,
                   unsigned N, unsigned K, unsigned batch, int precision_mode, void* workspace,
                   size_t workspace_bytes, int* device_status) {
  return tfccb200_sgemm_ex(stream, A, strideA, B, strideB, C, strideC, bias, M, N, K, batch,
                           precision_mode, TFCCB200_PATH_AUTO, workspace, workspace_bytes,
                           device_status);
}

size_t tfccb200_sgemm_workspace(unsigned M, unsigned N, unsigned K, unsigned batch,
                                int precision_mode) {
  (void)precision_mode;
  if (M == 0 || N == 0 || K == 0 || batch == 0) return 0;
  cudaError_t e;
  const DeviceInfo* di = current_device_info(&e);
  const int sms = di ? di->sm_count : 148;
  // The M <= 8 streaming kernel keeps its per-slice partial sums in scratch (the bound covers
  // both the batched and the batch-folded reading of the problem); the fp32 tensor-core
  // kernel keeps the partial tiles of a k-shared last wave there.
  size_t need = 0;
  if (precision_mode == TFCCB200_PRECISION_FP32 &&
      static_cast<unsigned long long>(M) * N * K * batch >= (1ull << 22))  // tensor-core sized
    need = umma_stream_k_workspace(sms);
  if (precision_mode == TFCCB200_PRECISION_BF16)  // dense upper bound: both operands batched
    need = bf16_staging_bytes(M, N, K, batch, M * K, K * N);
  if (M <= 32) need = std::max(need, skinny_sgemm_workspace(M, N, K, batch, sms));
  if (static_cast<unsigned long long>(M) * batch <= 32) {
    const size_t folded = skinny_sgemm_workspace(M * batch, N, K, 1, sms);
    if (folded > need) need = folded;
  }
  return need;
}

int tfccb200_sgemm_path(unsigned M, unsigned N, unsigned K, unsigned batch, unsigned strideA,
                        unsigned strideB, int precision_mode) {
  SgemmArgs a = {};
  a.A = a.B = reinterpret_cast<const float*>(16);
  a.C = reinterpret_cast<float*>(16);
  a.strideA = strideA; a.strideB = strideB; a.strideC = M * N;
  a.M = M; a.N = N; a.K = K; a.batch = batch;
  a.precision = precision_mode;
  if (M == 0 || N == 0 || K == 0 || batch == 0) return TFCCB200_EINVAL;
  if (a.batch == 1) a.strideA = a.strideB = 0;
  fold_batch(a);
  return pick_sgemm_path(a);
}

int tfccb200_qgemm_u8s8s32_ex(void* stream, const uint8_t* A, unsigned strideA,
                              const int32_t* rsA, unsigned strideRsA, int32_t offA,
                              const int8_t* B, unsigned strideB, const int32_t* rsB,
                              unsigned strideRsB, int32_t offB, int32_t* C, unsigned strideC,
                              unsigned M, unsigned N, unsigned K, unsigned batch, int path,
                              int* device_status) {
  QgemmArgs a = {};
  a.stream = static_cast<cudaStream_t>(stream);
  a.A = A; a.B = B; a.C = C; a.rsA = rsA; a.rsB = rsB;
  a.strideA = strideA; a.strideB = strideB; a.strideC = strideC;
  a.strideRsA = strideRsA; a.strideRsB = strideRsB;
  a.offA = offA; a.offB = offB;
  a.M = M; a.N = N; a.K = K; a.batch = batch;
  a.status = device_status;
  return run_qgemm(a, path);
}

int tfccb200_qgemm_u8s8s32(void* stream, const uint8_t* A, unsigned strideA, const int32_t* rsA,
                           unsigned strideRsA, int32_t offA, const int8_t* B, unsigned strideB,
                           const int32_t* rsB, unsigned strideRsB, int32_t offB, int32_t* C,
                           unsigned strideC, unsigned M, unsigned N, unsigned K, unsigned batch,
                           int* device_status) {
  return tfccb200_qgemm_u8s8s32_ex(stream, A, strideA, rsA, strideRsA, offA, B, strideB, rsB,
                                   strideRsB, offB, C, strideC, M, N, K, batch,
                                   TFCCB200_PATH_AUTO, device_status);
}

int tfccb200_qgemm_u8s8s32_dev(void* stream, const uint8_t* A, unsigned strideA, const int32_t* rsA,
                               unsigned strideRsA, const float* minA, const float* maxA,
                               const int8_t* B, unsigned strideB, const int32_t* rsB,
                               unsigned strideRsB, const float* minB, const float* maxB, int32_t* C,
                               unsigned strideC, float* minC, float* maxC, int32_t* offsets,
                               unsigned M, unsigned N, unsigned K, unsigned batch, int path,
                               int* device_status) {
  if (!minA || !maxA || !minB || !maxB || !minC || !maxC || !offsets) return TFCCB200_EINVAL;
  if (!A || !B || !C || !rsA || !rsB || M == 0 || N == 0 || K == 0 || batch == 0)
    return TFCCB200_EINVAL;
  int st = quantized_matmul_params_dev(static_cast<cudaStream_t>(stream), minA, maxA, minB, maxB,
                                       offsets, minC, maxC);
  if (st != TFCCB200_OK) return st;
  QgemmArgs a = {};
  a.stream = static_cast<cudaStream_t>(stream);
  a.A = A; a.B = B; a.C = C; a.rsA = rsA; a.rsB = rsB;
  a.strideA = strideA; a.strideB = strideB; a.strideC = strideC;
  a.strideRsA = strideRsA; a.strideRsB = strideRsB;
  a.dev_offsets = offsets;
  a.M = M; a.N = N; a.K = K; a.batch = batch;
  a.status = device_status;
  return run_qgemm(a, path);
}

int tfccb200_quantized_matmul_params(float minA, float maxA, float minB, float maxB,
                                     int32_t* offA, int32_t* offB, float* minC, float* maxC) {
  if (!offA || !offB || !minC || !maxC) return TFCCB200_EINVAL;
  int64_t oa = quantized_offset_8bit(minA, maxA);
  int64_t ob = quantized_offset_8bit(minB, maxB);
  oa -= static_cast<int64_t>(std::numeric_limits<uint8_t>::lowest());
  ob -= static_cast<int64_t>(std::numeric_limits<int8_t>::lowest());
  *offA = static_cast<int32_t>(oa);
  *offB = static_cast<int32_t>(ob);
  // One quantization level of each operand, in float as the reference computes it.
  const float a_level = (maxA - minA) / 255;
  const float b_level = (maxB - minB) / 255;
  const float c_level = a_level * b_level;
  *minC = c_level * static_cast<int64_t>(std::numeric_limits<int32_t>::lowest());
  *maxC = c_level * static_cast<int64_t>(std::numeric_limits<int32_t>::max());
  return TFCCB200_OK;
}

int tfccb200_reduce_sum_u8(void* stream, const uint8_t* src, unsigned batch, unsigned rows,
                           unsigned cols, int row_flag, int32_t* dst) {
  return reduce_sum_checked<uint8_t>(stream, src, batch, rows, cols, row_flag, dst);
}
int tfccb200_reduce_sum_s8(void* stream, const int8_t* src, unsigned batch, unsigned rows,
                           unsigned cols, int row_flag, int32_t* dst) {
  return reduce_sum_checked<int8_t>(stream, src, batch, rows, cols, row_flag, dst);
}
int tfccb200_reduce_sum_s16(void* stream, const int16_t* src, unsigned batch, unsigned rows,
                            unsigned cols, int row_flag, int32_t* dst) {
  return reduce_sum_checked<int16_t>(stream, src, batch, rows, cols, row_flag, dst);
}

int tfccb200_softmax_f32(void* stream, const float* src, unsigned rows, unsigned cols, float scale,
                         float* dst) {
  if (!src || !dst || rows == 0 || cols == 0) return TFCCB200_EINVAL;
  return softmax_f32(static_cast<cudaStream_t>(stream), src, rows, cols, scale, dst);
}

int tfccb200_layer_norm_f32(void* stream, const float* x, const float* residual,
                            const float* gamma, const float* beta, float eps, unsigned rows,
                            unsigned cols, float* dst) {
  if (!x || !gamma || !beta || !dst || rows == 0 || cols == 0) return TFCCB200_EINVAL;
  return layer_norm_f32(static_cast<cudaStream_t>(stream), x, residual, gamma, beta, eps, rows,
                        cols, dst);
}

int tfccb200_attention_f32(void* stream, const float* q, const float* k, const float* v,
                           float* out, unsigned batch, unsigned seq, unsigned heads, unsigned dim,
                           unsigned ld_qkv, unsigned ld_out, float scale, int* device_status) {
  if (!q || !k || !v || !out || batch == 0 || seq == 0 || heads == 0 || dim == 0)
    return TFCCB200_EINVAL;
  if (static_cast<unsigned long long>(batch) * seq * ld_qkv > 0xffffffffull ||
      static_cast<unsigned long long>(batch) * seq * ld_out > 0xffffffffull)
    return TFCCB200_EOVERFLOW;
  AttentionArgs a = {};
  a.stream = static_cast<cudaStream_t>(stream);
  a.q = q; a.k = k; a.v = v; a.out = out;
  a.batch = batch; a.seq = seq; a.heads = heads; a.dim = dim;
  a.ld = ld_qkv;
  a.batch_stride = static_cast<unsigned long long>(seq) * ld_qkv;
  a.ld_out = ld_out;
  a.scale = scale;
  a.status = device_status;
  return attention_f32(a);
}

int tfccb200_gelu_f32(void* stream, const float* src, size_t n, float* dst) {
  if (!src || !dst || n == 0) return TFCCB200_EINVAL;
  return gelu_f32(static_cast<cudaStream_t>(stream), src, n, dst);
}

int tfccb200_permute_0213_f32(void* stream, const float* src, unsigned d0, unsigned d1,
                              unsigned d2, unsigned d3, float* dst) {
  if (!src || !dst || d0 == 0 || d1 == 0 || d2 == 0 || d3 == 0) return TFCCB200_EINVAL;
  if (static_cast<unsigned long long>(d0) * d1 * d2 * d3 > 0xffffffffull) return TFCCB200_EOVERFLOW;
  return permute_0213_f32(static_cast<cudaStream_t>(stream), src, d0, d1, d2, d3, dst);
}

int tfccb200_transpose_last2_f32(void* stream, const float* src, unsigned batch, unsigned r,
                                 unsigned c, float* dst) {
  if (!src || !dst || batch == 0 || r == 0 || c == 0) return TFCCB200_EINVAL;
  return transpose_last2_f32(static_cast<cudaStream_t>(stream), src, batch, r, c, dst);
}

int tfccb200_minmax_f32(void* stream, const float* src, size_t n, float* minmax) {
  if (!src || !minmax || n == 0) return TFCCB200_EINVAL;
  return minmax_f32(static_cast<cudaStream_t>(stream), src, n, minmax);
}

int tfccb200_quantize_f32(void* stream, const float* src, size_t n, const float* min_value,
                          const float* max_value, void* dst, int dst_type) {
  if (!src || !min_value || !max_value || !dst || n == 0) return TFCCB200_EINVAL;
  return quantize_f32(static_cast<cudaStream_t>(stream), src, n, min_value, max_value, dst,
                      dst_type);
}

int tfccb200_quantize_rowsum_f32(void* stream, const float* src, unsigned rows, unsigned cols,
                                 const float* min_value, const float* max_value, void* dst,
                                 int dst_type, int32_t* row_sums) {
  if (!src || !min_value || !max_value || !dst || !row_sums || rows == 0 || cols == 0)
    return TFCCB200_EINVAL;
  if (static_cast<unsigned long long>(rows) * cols > 0xffffffffull) return TFCCB200_EOVERFLOW;
  return quantize_rows_f32(static_cast<cudaStream_t>(stream), src, rows, cols, min_value,
                           max_value, dst, dst_type, row_sums);
}

int tfccb200_dequantize_f32(void* stream, const void* src, int src_type, size_t n,
                            const float* min_value, const float* max_value, float* dst) {
  if (!src || !min_value || !max_value || !dst || n == 0) return TFCCB200_EINVAL;
  return dequantize_f32(static_cast<cudaStream_t>(stream), src, src_type, n, min_value, max_value,
                        dst);
}

int tfccb200_requantize(void* stream, const void* src, int src_type, size_t n,
                        const float* min_input, const float* max_input, const float* min_output,
                        const float* max_output, void* dst, int dst_type) {
  if (!src || !min_input || !max_input || !min_output || !max_output || !dst || n == 0)
    return TFCCB200_EINVAL;
  return requantize(static_cast<cudaStream_t>(stream), src, src_type, n, min_input, max_input,
                    min_output, max_output, dst, dst_type);
}

int tfccb200_sgemm_nsplit_push_ex(void* stream, const float* A, const float* B_shard,
                                  float* const* C_ranks, unsigned num_ranks, unsigned rank,
                                  const float* bias_shard, unsigned M, unsigned N_shard,
                                  unsigned K, int precision_mode, float* C_multicast,
                                  void* workspace, size_t workspace_bytes, unsigned max_ctas,
                                  int* device_status) {
  if (!A || !B_shard || !C_ranks || num_ranks == 0 || num_ranks > 8 || rank >= num_ranks)
    return TFCCB200_EINVAL;
  if (M == 0 || N_shard == 0 || K == 0) return TFCCB200_EINVAL;
  if (precision_mode != TFCCB200_PRECISION_FP32 && precision_mode != TFCCB200_PRECISION_TF32)
    return TFCCB200_EINVAL;
  const unsigned long long n_total = static_cast<unsigned long long>(N_shard) * num_ranks;
  if (n_total > 0xffffffffull || shape_overflows(M, static_cast<unsigned>(n_total), K, 1))
    return TFCCB200_EOVERFLOW;
  if (!C_ranks[rank]) return TFCCB200_EINVAL;
  SgemmArgs a = {};
  a.stream = static_cast<cudaStream_t>(stream);
  a.A = A; a.B = B_shard; a.bias = bias_shard;
  a.M = M; a.N = N_shard; a.K = K; a.batch = 1;
  a.strideC = 0;
  a.precision = precision_mode;
  a.status = device_status;
  a.workspace = workspace;
  a.workspace_bytes = workspace ? workspace_bytes : 0;
  a.max_ctas = max_ctas;
  for (unsigned d = 0; d < num_ranks; ++d) {
    if (!C_ranks[d]) continue;  // that rank's copy is not written by this call
    if (reinterpret_cast<uintptr_t>(C_ranks[d]) & 15u) return TFCCB200_EALIGN;
    a.dst[a.num_dst++] = C_ranks[d];
  }
  a.C = C_ranks[rank];
  if (C_multicast && (reinterpret_cast<uintptr_t>(C_multicast) & 15u)) return TFCCB200_EALIGN;
  a.mc_dst = C_multicast;
  a.ldc = n_total;
  a.col_offset = rank * N_shard;
  if (!umma_sgemm_supported(a)) return TFCCB200_EALIGN;  // N_shard % 4, K % 4, 16-byte bases
  cudaError_t e;
  const DeviceInfo* di = current_device_info(&e);
  if (!di) return static_cast<int>(e);
  const int sms = umma_sm_budget(di->sm_count, max_ctas);
  return umma_sgemm(a, umma_plan(M, N_shard, K, 1, sms, 4, -1, false,
                                 stream_k_scratch_ok(a, sms)).pair);
}

int tfccb200_sgemm_nsplit_push(void* stream, const float* A, const float* B_shard,
                               float* const* C_ranks, unsigned num_ranks, unsigned rank,
                               const float* bias_shard, unsigned M, unsigned N_shard, unsigned K,
                               int precision_mode, float* C_multicast, void* workspace,
                               size_t workspace_bytes, int* device_status) {
  return tfccb200_sgemm_nsplit_push_ex(stream, A, B_shard, C_ranks, num_ranks, rank, bias_shard,
                                       M, N_shard, K, precision_mode, C_multicast, workspace,
                                       workspace_bytes, 0, device_status);
}

int tfccb200_qgemm_nsplit_push(void* stream, const uint8_t* A, const int32_t* rsA, int32_t offA,
                               const int8_t* B_shard, const int32_t* rsB_shard, int32_t offB,
                               int32_t* const* C_ranks, unsigned num_ranks, unsigned rank,
                               unsigned M, unsigned N_shard, unsigned K, int32_t* C_multicast,
                               int* device_status) {
  if (!A || !rsA || !B_shard || !rsB_shard || !C_ranks || num_ranks == 0 || num_ranks > 8 ||
      rank >= num_ranks)
    return TFCCB200_EINVAL;
  if (M == 0 || N_shard == 0 || K == 0) return TFCCB200_EINVAL;
  const unsigned long long n_total = static_cast<unsigned long long>(N_shard) * num_ranks;
  if (n_total > 0xffffffffull || shape_overflows(M, static_cast<unsigned>(n_total), K, 1))
    return TFCCB200_EOVERFLOW;
  if (!C_ranks[rank]) return TFCCB200_EINVAL;
  QgemmArgs a = {};
  a.stream = static_cast<cudaStream_t>(stream);
  a.A = A; a.B = B_shard; a.rsA = rsA; a.rsB = rsB_shard;
  a.offA = offA; a.offB = offB;
  a.M = M; a.N = N_shard; a.K = K; a.batch = 1;
  a.strideC = 0;
  a.status = device_status;
  for (unsigned d = 0; d < num_ranks; ++d) {
    if (!C_ranks[d]) continue;
    if (reinterpret_cast<uintptr_t>(C_ranks[d]) & 15u) return TFCCB200_EALIGN;
    a.dst[a.num_dst++] = C_ranks[d];
  }
  a.C = C_ranks[rank];
  if (C_multicast && (reinterpret_cast<uintptr_t>(C_multicast) & 15u)) return TFCCB200_EALIGN;
  a.mc_dst = C_multicast;
  a.ldc = n_total;
  a.col_offset = rank * N_shard;
  // the tensor-core kernel is the only one that can store into several matrices
  if (!umma_qgemm_supported(a) || K < 128 || N_shard < 128) return TFCCB200_EALIGN;
  cudaError_t e;
  const DeviceInfo* di = current_device_info(&e);
  if (!di) return static_cast<int>(e);
  return umma_qgemm(a, umma_qgemm_prefers_pair(M, N_shard, K, 1, di->sm_count));
}

int tfccb200_sgemm_skinny_static(void* stream, const float* A, const float* B, float* C,
                                 const float* bias, unsigned M, unsigned N, unsigned K) {
  if (!A || !B || !C || M == 0 || N == 0 || K == 0) return TFCCB200_EINVAL;
  if (M > 8) return TFCCB200_EUNSUPPORTED;
  if (static_cast<unsigned long long>(K) * N > 0xffffffffull) return TFCCB200_EOVERFLOW;
  return skinny_sgemm_static(static_cast<cudaStream_t>(stream), A, B, C, bias, M, N, K);
}

size_t tfccb200_sgemm_skinny_static_capacity(void) { return skinny_sgemm_static_capacity(); }

size_t tfccb200_sgemm_skinny_static_need(unsigned M, unsigned N, unsigned K) {
  if (M == 0 || M > 8 || N == 0 || K == 0) return 0;
  cudaError_t e;
  const DeviceInfo* di = current_device_info(&e);
  return skinny_sgemm_workspace(M, N, K, 1, di ? di->sm_count : 148);
}

int tfccb200_interleave_panels_f32(void* stream, const float* src, float* dst, unsigned M,
                                   unsigned ns, unsigned G) {
  if (!src || !dst || M == 0 || ns == 0 || G == 0) return TFCCB200_EINVAL;
  return interleave_panels_f32(static_cast<cudaStream_t>(stream), src, dst, M, ns, G);
}

int tfccb200_sgemm_host(void* stream, const float* hA, unsigned strideA, const float* hB,
                        unsigned strideB, float* hC, unsigned strideC, const float* hbias,
                        unsigned M, unsigned N, unsigned K, unsigned batch, int precision_mode) {
  if (!hA || !hB || !hC || M == 0 || N == 0 || K == 0 || batch == 0) return TFCCB200_EINVAL;
  if (shape_overflows(M, N, K, batch)) return TFCCB200_EOVERFLOW;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (batch == 1) strideA = strideB = 0, strideC = M * N;
  const size_t nA = strideA ? static_cast<size_t>(strideA) * (batch - 1) + size_t(M) * K
                            : size_t(M) * K;
  const size_t nB = strideB ? static_cast<size_t>(strideB) * (batch - 1) + size_t(K) * N
                            : size_t(K) * N;
  const size_t nC = static_cast<size_t>(strideC) * (batch - 1) + size_t(M) * N;
  const size_t ws = tfccb200_sgemm_workspace(M, N, K, batch, precision_mode);
  DeviceBuffer dA(s), dB(s), dC(s), dBias(s), dW(s), dS(s);
  cudaError_t e;

  // One large product: the transfers dominate, so they are overlapped with the arithmetic.
  // B goes up first; A then goes up in row blocks on a copy stream while the block before it
  // is multiplied on the caller's stream and the block before that comes down on a third
  // stream.  (Pinned host buffers are needed for the copies to really overlap.)
  constexpr unsigned kRowBlock = 512;  // short last block: little is left to do after the last upload
  static const bool pipeline = [] {
    const char* v = std::getenv("TFCCB200_HOST_PIPELINE");
    return !(v && v[0] == '0');
  }();
  if (pipeline && batch == 1 && M >= 2 * kRowBlock &&
      (nA + nB + nC) * 4 >= (size_t(64) << 20)) {
    // Row blocks of kRowBlock; a last block of eight rows or fewer is merged into the one
    // before it, so that every block takes the tensor-core path and one scratch size fits all.
    unsigned blocks = (M + kRowBlock - 1) / kRowBlock;
    if (M - (blocks - 1) * kRowBlock <= 8) --blocks;
    const unsigned last_rows = M - (blocks - 1) * kRowBlock;
    const size_t ws_block = std::max(tfccb200_sgemm_workspace(kRowBlock, N, K, 1, precision_mode),
                                     tfccb200_sgemm_workspace(last_rows, N, K, 1, precision_mode));
    ScopedStream up, down;
    ScopedEvent b_ready, c_done_all, alloc_done;
    if ((e = up.create()) != cudaSuccess || (e = down.create()) != cudaSuccess) return e;
    if ((e = b_ready.create()) != cudaSuccess || (e = c_done_all.create()) != cudaSuccess ||
        (e = alloc_done.create()) != cudaSuccess)
      return e;
    std::vector<ScopedEvent> a_ready(blocks), c_ready(blocks);
    for (unsigned i = 0; i < blocks; ++i)
      if ((e = a_ready[i].create()) != cudaSuccess || (e = c_ready[i].create()) != cudaSuccess)
        return e;
    JoinStreams join;  // from here on an early return waits for all three streams
    join.add(up.s); join.add(down.s); join.add(s);
    if ((e = dA.alloc(nA * 4)) != cudaSuccess) return e;
    if ((e = dB.alloc(nB * 4)) != cudaSuccess) return e;
    if ((e = dC.alloc(nC * 4)) != cudaSuccess) return e;
    if ((e = dW.alloc(ws_block)) != cudaSuccess) return e;
    if ((e = dS.alloc(sizeof(int))) != cudaSuccess) return e;
    if (hbias && (e = dBias.alloc(size_t(N) * 4)) != cudaSuccess) return e;
    if ((e = cudaMemsetAsync(dS.p, 0, sizeof(int), s)) != cudaSuccess) return e;
    // the buffers come from the caller's stream: the side streams start after that point
    if ((e = cudaEventRecord(alloc_done.e, s)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(up.s, alloc_done.e, 0)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(down.s, alloc_done.e, 0)) != cudaSuccess) return e;
    if (hbias && (e = cudaMemcpyAsync(dBias.p, hbias, size_t(N) * 4, cudaMemcpyHostToDevice,
                                      up.s)) != cudaSuccess)
      return e;
    if ((e = cudaMemcpyAsync(dB.p, hB, nB * 4, cudaMemcpyHostToDevice, up.s)) != cudaSuccess)
      return e;
    if ((e = cudaEventRecord(b_ready.e, up.s)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(s, b_ready.e, 0)) != cudaSuccess) return e;
    for (unsigned i = 0; i < blocks; ++i) {
      const unsigned r0 = i * kRowBlock;
      const unsigned rows = (i + 1 == blocks) ? M - r0 : kRowBlock;
      float* dAi = static_cast<float*>(dA.p) + size_t(r0) * K;
      float* dCi = static_cast<float*>(dC.p) + size_t(r0) * N;
      if ((e = cudaMemcpyAsync(dAi, hA + size_t(r0) * K, size_t(rows) * K * 4,
                               cudaMemcpyHostToDevice, up.s)) != cudaSuccess)
        return e;
      if ((e = cudaEventRecord(a_ready[i].e, up.s)) != cudaSuccess) return e;
      if ((e = cudaStreamWaitEvent(s, a_ready[i].e, 0)) != cudaSuccess) return e;
      int st = tfccb200_sgemm(s, dAi, 0, static_cast<float*>(dB.p), 0, dCi, rows * N,
                              hbias ? static_cast<float*>(dBias.p) : nullptr, rows, N, K, 1,
                              precision_mode, dW.p, ws_block, static_cast<int*>(dS.p));
      if (st != TFCCB200_OK) return st;
      if ((e = cudaEventRecord(c_ready[i].e, s)) != cudaSuccess) return e;
      if ((e = cudaStreamWaitEvent(down.s, c_ready[i].e, 0)) != cudaSuccess) return e;
      if ((e = cudaMemcpyAsync(hC + size_t(r0) * N, dCi, size_t(rows) * N * 4,
                               cudaMemcpyDeviceToHost, down.s)) != cudaSuccess)
        return e;
    }
    int dev_status = 0;
    if ((e = cudaMemcpyAsync(&dev_status, dS.p, sizeof(int), cudaMemcpyDeviceToHost, s)) !=
        cudaSuccess)
      return e;
    // rejoin: the caller's stream (which frees the buffers) must follow both side streams
    if ((e = cudaEventRecord(c_done_all.e, down.s)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(s, c_done_all.e, 0)) != cudaSuccess) return e;
    if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
    join.armed = false;  // s has followed both side streams to their end
    return dev_status ? TFCCB200_EDEVICE : TFCCB200_OK;
  }

  JoinStreams join;
  join.add(s);
  if ((e = dA.alloc(nA * 4)) != cudaSuccess) return e;
  if ((e = dB.alloc(nB * 4)) != cudaSuccess) return e;
  if ((e = dC.alloc(nC * 4)) != cudaSuccess) return e;
  if ((e = dW.alloc(ws)) != cudaSuccess) return e;
  if ((e = dS.alloc(sizeof(int))) != cudaSuccess) return e;
  if (hbias && (e = dBias.alloc(size_t(N) * 4)) != cudaSuccess) return e;
  if ((e = cudaMemsetAsync(dS.p, 0, sizeof(int), s)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(dA.p, hA, nA * 4, cudaMemcpyHostToDevice, s)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(dB.p, hB, nB * 4, cudaMemcpyHostToDevice, s)) != cudaSuccess) return e;
  if (hbias &&
      (e = cudaMemcpyAsync(dBias.p, hbias, size_t(N) * 4, cudaMemcpyHostToDevice, s)) !=
          cudaSuccess)
    return e;
  int st = tfccb200_sgemm(s, static_cast<float*>(dA.p), strideA, static_cast<float*>(dB.p),
                          strideB, static_cast<float*>(dC.p), strideC,
                          hbias ? static_cast<float*>(dBias.p) : nullptr, M, N, K, batch,
                          precision_mode, dW.p, ws, static_cast<int*>(dS.p));
  if (st != TFCCB200_OK) return st;
  int dev_status = 0;
  if ((e = cudaMemcpyAsync(hC, dC.p, nC * 4, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(&dev_status, dS.p, sizeof(int), cudaMemcpyDeviceToHost, s)) !=
      cudaSuccess)
    return e;
  if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
  return dev_status ? TFCCB200_EDEVICE : TFCCB200_OK;
}

int tfccb200_qgemm_u8s8s32_host(void* stream, const uint8_t* hA, unsigned strideA,
                                const int8_t* hB, unsigned strideB, float minA, float maxA,
                                float minB, float maxB, int32_t* hC, unsigned strideC,
                                float* minC, float* maxC, unsigned M, unsigned N, unsigned K,
                                unsigned batch) {
  if (!hA || !hB || !hC || !minC || !maxC || M == 0 || N == 0 || K == 0 || batch == 0)
    return TFCCB200_EINVAL;
  if (shape_overflows(M, N, K, batch)) return TFCCB200_EOVERFLOW;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (batch == 1) strideA = strideB = 0, strideC = M * N;
  int32_t offA, offB;
  int st = tfccb200_quantized_matmul_params(minA, maxA, minB, maxB, &offA, &offB, minC, maxC);
  if (st != TFCCB200_OK) return st;
  const unsigned batchA = strideA ? batch : 1, batchB = strideB ? batch : 1;
  const size_t nA = size_t(batchA) * M * K, nB = size_t(batchB) * K * N;
  const size_t nC = static_cast<size_t>(strideC) * (batch - 1) + size_t(M) * N;
  if ((strideA && strideA != M * K) || (strideB && strideB != K * N)) return TFCCB200_EINVAL;
  DeviceBuffer dA(s), dB(s), dC(s), dRa(s), dRb(s), dS(s);
  JoinStreams join;  // an early return waits for the copies already queued
  join.add(s);
  cudaError_t e;
  if ((e = dA.alloc(nA)) != cudaSuccess) return e;
  if ((e = dB.alloc(nB)) != cudaSuccess) return e;
  if ((e = dC.alloc(nC * 4)) != cudaSuccess) return e;
  if ((e = dRa.alloc(size_t(batchA) * M * 4)) != cudaSuccess) return e;
  if ((e = dRb.alloc(size_t(batchB) * N * 4)) != cudaSuccess) return e;
  if ((e = dS.alloc(sizeof(int))) != cudaSuccess) return e;
  if ((e = cudaMemsetAsync(dS.p, 0, sizeof(int), s)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(dA.p, hA, nA, cudaMemcpyHostToDevice, s)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(dB.p, hB, nB, cudaMemcpyHostToDevice, s)) != cudaSuccess) return e;
  // reduce_sum(a, row) and reduce_sum(b, column), then the matmul: the
  // sequence of tfcc/test/quantization.cpp:105-121.
  st = tfccb200_reduce_sum_u8(s, static_cast<uint8_t*>(dA.p), batchA, M, K, 1,
                              static_cast<int32_t*>(dRa.p));
  if (st != TFCCB200_OK) return st;
  st = tfccb200_reduce_sum_s8(s, static_cast<int8_t*>(dB.p), batchB, K, N, 0,
                              static_cast<int32_t*>(dRb.p));
  if (st != TFCCB200_OK) return st;
  st = tfccb200_qgemm_u8s8s32(s, static_cast<uint8_t*>(dA.p), strideA,
                              static_cast<int32_t*>(dRa.p), strideA ? M : 0, offA,
                              static_cast<int8_t*>(dB.p), strideB, static_cast<int32_t*>(dRb.p),
                              strideB ? N : 0, offB, static_cast<int32_t*>(dC.p), strideC, M, N, K,
                              batch, static_cast<int*>(dS.p));
  if (st != TFCCB200_OK) return st;
  int dev_status = 0;
  if ((e = cudaMemcpyAsync(hC, dC.p, nC * 4, cudaMemcpyDeviceToHost, s)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(&dev_status, dS.p, sizeof(int), cudaMemcpyDeviceToHost, s)) !=
      cudaSuccess)
    return e;
  if ((e = cudaStreamSynchronize(s)) != cudaSuccess) return e;
  return dev_status ? TFCCB200_EDEVICE : TFCCB200_OK;
}

}  // extern "C"
