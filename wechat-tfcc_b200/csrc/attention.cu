// One attention head per CTA, start to finish on the tensor cores:
//
//   S = Q . K^T          [seq, seq]   tcgen05.mma, fp32 by three TF32 MMAs (head/tail split)
//   P = softmax(scale S)              in registers, one query row per thread, the reference's
//                                     formula (max, exp, sum, divide: softmaxV2,
//                                     tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:138-155)
//   O = P . V            [seq, dim]   tcgen05.mma again, P written back to shared memory in
//                                     the K-major operand layout
//
// Q, K and V are read where a transformer block's projections leave them -- [batch, seq,
// head, dim] with any row pitch, so a packed [batch, seq, 3*heads*dim] buffer works -- through
// 4-D tensor maps, and O is written as [batch, seq, heads*dim], ready for the output
// projection.  K is consumed as a K-major B operand, so neither the head split / merge
// permutations nor the transposition of K exist as passes over memory.  This replaces, per
// layer of the reference graph: three transposes to [batch, head, seq, dim], one transpose of
// K, a batched matmul, a scale, a softmax, a batched matmul and a transpose back
// (tfcc/cuda/interfaces/tfcc_cudabasicinterface.cu:83-100,
//  tfcc/cuda/interfaces/tfcc_cudaactivationinterface.cu:96-121,
//  tfcc/cuda/interfaces/tfcc_cudablasinterface.cu:201-248).
//
// Limits: seq <= 128 (one score tile holds whole rows), dim 32 or 64.  Everything is sized for
// one CTA per SM; a (batch x heads) grid of 96 fills two thirds of a B200 in one wave.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>

#include "internal.h"
#include "pdl.cuh"
#include "ptx.cuh"

namespace tfccb200 {

namespace {

constexpr int kAttThreads = 256;       // eight warps: warps w and w+4 share TMEM lane quarter w,
                                       // each taking half of a row's columns
constexpr int kAttRows = 128;          // query rows = key rows of a tile
constexpr int kTile = kAttRows * 128;  // bytes of one [128 rows x 32 floats] operand tile

struct AttParams {
  float* out;
  unsigned seq, heads, dim;
  unsigned long long ld_out;
  float scale;
  int* status;
  unsigned long long timeout_ns;
};

// Shared memory (dim = 64: kb = 2 k-blocks of 32):
//   [Q raw kb tiles][Q tail][K raw][K tail]   -> later overwritten by P raw (4 tiles) + P tail
//   [V raw 4 k-blocks x (dim/32) chunks of 4 KB][V tail]
template <int DIM>
struct AttLayout {
  static constexpr int kKb = DIM / 32;              // k-blocks of the first product
  static constexpr int kQBytes = kKb * kTile;       // one copy of Q (or K)
  static constexpr int kVChunk = 32 * 128;          // [32 key rows x 32 floats]
  static constexpr int kVBytes = 4 * kKb * kVChunk; // 128 key rows x DIM floats
  static constexpr int kPBytes = 4 * kTile;         // one copy of P: 4 k-blocks of 32 keys
  static constexpr int kFront = (4 * kQBytes > 2 * kPBytes) ? 4 * kQBytes : 2 * kPBytes;
  static constexpr int kSmem = kFront + 2 * kVBytes + 64 + 2048 + 1024;  // + row max / sum exchange
};

__device__ __forceinline__ bool att_wait(uint32_t bar, uint32_t parity, const AttParams& p,
                                         volatile uint32_t* abort_flag, int bit) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  uint64_t start = 0;
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = ptx::globaltimer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > p.timeout_ns) {
        *abort_flag = 1;
        if (p.status) atomicOr(p.status, bit);
        return false;
      }
    }
  }
}

// tail = round_to_tf32(x - head(x)), head = x with the 13 low mantissa bits cleared; the raw
// value itself serves as the head operand (the tensor core ignores those bits).
__device__ __forceinline__ float tf32_tail(float x) {
  const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  uint32_t t;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(t) : "f"(x - h));
  return __uint_as_float(t);
}

template <int DIM>
__global__ void __launch_bounds__(kAttThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const AttParams p) {
  using L = AttLayout<DIM>;
  extern __shared__ uint8_t smem_raw[];
  pdl_release();
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t q_raw = base, q_lo = base + L::kQBytes;
  const uint32_t k_raw = base + 2 * L::kQBytes, k_lo = base + 3 * L::kQBytes;
  const uint32_t p_raw = base, p_lo = base + L::kPBytes;  // reuse of the Q / K area
  const uint32_t v_raw = base + L::kFront, v_lo = v_raw + L::kVBytes;
  const uint32_t bar_load = v_lo + L::kVBytes, bar_mma = bar_load + 8, tmem_slot = bar_load + 16;
  uint8_t* ctl_gen = gen + L::kFront + 2 * L::kVBytes;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(ctl_gen + 16);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(ctl_gen + 20);

  const unsigned tid = threadIdx.x, warp = tid >> 5;  // 8 warps
  const int head = static_cast<int>(blockIdx.x % p.heads);
  const int b = static_cast<int>(blockIdx.x / p.heads);

  if (tid == 0) {
    ptx::mbar_init(bar_load, 1);
    ptx::mbar_init(bar_mma, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tq);
    ptx::prefetch_tensormap(&tk);
    ptx::prefetch_tensormap(&tv);
  }
  if (warp == 0) {
    ptx::tmem_alloc<1>(tmem_slot, 256);  // scores: 128 columns, output: DIM columns
    ptx::tmem_relinquish<1>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  pdl_wait();  // nothing above touched global memory

  if (tid == 0) {
    ptx::mbar_expect_tx(bar_load, 2u * L::kQBytes + L::kVBytes);
#pragma unroll
    for (int kb = 0; kb < L::kKb; ++kb) {
      ptx::tma_load_4d(q_raw + kb * kTile, &tq, bar_load, kb * 32, head, 0, b);
      ptx::tma_load_4d(k_raw + kb * kTile, &tk, bar_load, kb * 32, head, 0, b);
    }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb)
#pragma unroll
      for (int c = 0; c < L::kKb; ++c)
        ptx::tma_load_4d(v_raw + (kb * L::kKb + c) * L::kVChunk, &tv, bar_load, c * 32, head,
                         kb * 32, b);
  }
  att_wait(bar_load, 0u, p, abort_flag, TFCCB200_DEV_TIMEOUT_TMA);

  // ---- TF32 tails of Q, K and V next to the raw tiles (same swizzled positions) ----
  {
    auto split = [&](uint32_t raw_off, uint32_t lo_off, int bytes) {
      const float4* raw = reinterpret_cast<const float4*>(gen + (raw_off - base));
      float4* lo = reinterpret_cast<float4*>(gen + (lo_off - base));
      for (int i = tid; i < bytes / 16; i += kAttThreads) {
        const float4 x = raw[i];
        lo[i] = make_float4(tf32_tail(x.x), tf32_tail(x.y), tf32_tail(x.z), tf32_tail(x.w));
      }
    };
    split(q_raw, q_lo, L::kQBytes);
    split(k_raw, k_lo, L::kQBytes);
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before_sync();
  __syncthreads();

  // ---- S = Q . K^T: both operands K-major ----
  if (tid == 0) {
    ptx::tc_fence_after_sync();
    constexpr uint32_t idesc = ptx::make_idesc(1u, 2u, 2u, 0u, 0u, 128u, 128u);
#pragma unroll
    for (int kb = 0; kb < L::kKb; ++kb) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t off = kb * kTile + ks * 32;
        const uint64_t a_hi = ptx::smem_desc(q_raw + off, 16, 1024, ptx::kLayoutSw128);
        const uint64_t a_lo = ptx::smem_desc(q_lo + off, 16, 1024, ptx::kLayoutSw128);
        const uint64_t b_hi = ptx::smem_desc(k_raw + off, 16, 1024, ptx::kLayoutSw128);
        const uint64_t b_lo = ptx::smem_desc(k_lo + off, 16, 1024, ptx::kLayoutSw128);
        ptx::umma<ptx::MmaKind::TF32, 1>(tmem_base, a_lo, b_hi, idesc, (kb | ks) ? 1u : 0u);
        ptx::umma<ptx::MmaKind::TF32, 1>(tmem_base, a_hi, b_lo, idesc, 1u);
        ptx::umma<ptx::MmaKind::TF32, 1>(tmem_base, a_hi, b_hi, idesc, 1u);
      }
    }
    ptx::umma_commit<1>(bar_mma, 0);
  }
  // V's tails are made while the tensor core works on the scores
  {
    const float4* raw = reinterpret_cast<const float4*>(gen + (v_raw - base));
    float4* lo = reinterpret_cast<float4*>(gen + (v_lo - base));
    for (int i = tid; i < L::kVBytes / 16; i += kAttThreads) {
      const float4 x = raw[i];
      lo[i] = make_float4(tf32_tail(x.x), tf32_tail(x.y), tf32_tail(x.z), tf32_tail(x.w));
    }
  }
  att_wait(bar_mma, 0u, p, abort_flag, TFCCB200_DEV_TIMEOUT_MMA);
  ptx::tc_fence_after_sync();

  // ---- softmax: a row is shared by two threads (warps w and w+4), 64 columns each; row
  // maximum and row sum are exchanged through shared memory.  Then P (raw and tail) goes into
  // the K-major operand layout over the dead Q / K tiles. ----
  const unsigned row = (warp & 3u) * 32u + (tid & 31u);  // TMEM lane = query row
  const unsigned half = warp >> 2;                       // which 64 columns of the row
  const uint32_t lane_addr = tmem_base + (((warp & 3u) * 32u) << 16);
  float* xch = reinterpret_cast<float*>(ctl_gen + 64);   // [2 halves][128 rows], used twice
  {
    uint32_t u[64];
    ptx::tmem_ld_32x32(lane_addr + half * 64, reinterpret_cast<uint32_t(&)[32]>(u[0]));
    ptx::tmem_ld_32x32(lane_addr + half * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(u[32]));
    ptx::tmem_ld_wait();
    float mx = -3.402823466e+38f;
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const float v = (half * 64 + c < p.seq) ? __uint_as_float(u[c]) * p.scale : -3.402823466e+38f;
      u[c] = __float_as_uint(v);
      mx = fmaxf(mx, v);
    }
    xch[half * 128 + row] = mx;
    __syncthreads();
    mx = fmaxf(mx, xch[(half ^ 1u) * 128 + row]);
    __syncthreads();
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      const float e = (half * 64 + c < p.seq) ? expf(__uint_as_float(u[c]) - mx) : 0.f;
      u[c] = __float_as_uint(e);
      sum += e;
    }
    xch[half * 128 + row] = sum;
    __syncthreads();
    // the two halves in a fixed order, so that both threads of a row divide by the same sum
    sum = xch[row] + xch[128 + row];
    uint8_t* p_raw_gen = gen + (p_raw - base);
    uint8_t* p_lo_gen = gen + (p_lo - base);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const unsigned kb = half * 2 + kk;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v;
        v.x = __uint_as_float(u[kk * 32 + j * 4 + 0]) / sum;
        v.y = __uint_as_float(u[kk * 32 + j * 4 + 1]) / sum;
        v.z = __uint_as_float(u[kk * 32 + j * 4 + 2]) / sum;
        v.w = __uint_as_float(u[kk * 32 + j * 4 + 3]) / sum;
        const unsigned off = kb * kTile + row * 128 + ((j ^ (row & 7u)) << 4);
        *reinterpret_cast<float4*>(p_raw_gen + off) = v;
        *reinterpret_cast<float4*>(p_lo_gen + off) =
            make_float4(tf32_tail(v.x), tf32_tail(v.y), tf32_tail(v.z), tf32_tail(v.w));
      }
    }
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before_sync();
  __syncthreads();

  // ---- O = P . V: A K-major (keys contiguous), B = V as it lies (MN-major) ----
  const uint32_t tmem_o = tmem_base + 128;
  if (tid == 0) {
    ptx::tc_fence_after_sync();
    constexpr uint32_t idesc = ptx::make_idesc(1u, 2u, 2u, 0u, 1u, 128u, static_cast<uint32_t>(DIM));
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t a_off = kb * kTile + ks * 32;
        const uint32_t b_off = kb * L::kKb * L::kVChunk + ks * 1024;
        const uint64_t a_hi = ptx::smem_desc(p_raw + a_off, 16, 1024, ptx::kLayoutSw128);
        const uint64_t a_lo = ptx::smem_desc(p_lo + a_off, 16, 1024, ptx::kLayoutSw128);
        const uint64_t b_hi = ptx::smem_desc(v_raw + b_off, L::kVChunk, 512, ptx::kLayoutSw128Base32);
        const uint64_t b_lo = ptx::smem_desc(v_lo + b_off, L::kVChunk, 512, ptx::kLayoutSw128Base32);
        ptx::umma<ptx::MmaKind::TF32, 1>(tmem_o, a_lo, b_hi, idesc, (kb | ks) ? 1u : 0u);
        ptx::umma<ptx::MmaKind::TF32, 1>(tmem_o, a_hi, b_lo, idesc, 1u);
        ptx::umma<ptx::MmaKind::TF32, 1>(tmem_o, a_hi, b_hi, idesc, 1u);
      }
    }
    ptx::umma_commit<1>(bar_mma, 0);
  }
  att_wait(bar_mma, 1u, p, abort_flag, TFCCB200_DEV_TIMEOUT_MMA);
  ptx::tc_fence_after_sync();

  // ---- output: each thread stores its half of the row's DIM floats (DIM = 32: warps 0-3 only) ----
  {
    constexpr int kColsPerThread = DIM / 2 >= 32 ? DIM / 2 : 32;
    constexpr int kHalves = DIM / kColsPerThread;
    if (static_cast<int>(half) < kHalves) {
      float* dst = p.out + (static_cast<unsigned long long>(b) * p.seq + row) * p.ld_out +
                   static_cast<unsigned long long>(head) * DIM + half * kColsPerThread;
      uint32_t r[32];
      ptx::tmem_ld_32x32(lane_addr + 128 + half * kColsPerThread, r);
      ptx::tmem_ld_wait();
      if (row < p.seq) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {  // a wait was abandoned: give copies and MMAs in flight a bounded moment
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (warp == 0) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<1>(tmem_base, 256);
  }
}

}  // namespace

bool attention_supported(const AttentionArgs& a) {
  if (a.seq == 0 || a.seq > 128 || (a.dim != 32 && a.dim != 64)) return false;
  if (a.batch == 0 || a.heads == 0) return false;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!aligned(a.q) || !aligned(a.k) || !aligned(a.v) || !aligned(a.out)) return false;
  if (a.ld % 4 || a.batch_stride % 4 || a.ld_out % 4) return false;
  if (a.ld < static_cast<unsigned long long>(a.heads) * a.dim) return false;
  if (a.ld_out < static_cast<unsigned long long>(a.heads) * a.dim) return false;
  if (a.batch > 1 && a.batch_stride < a.ld * a.seq) return false;
  if (static_cast<unsigned long long>(a.batch) * a.heads > 0x7fffffffull) return false;
  return true;
}

namespace {

template <int DIM>
int launch_attention(const AttentionArgs& a) {
  using L = AttLayout<DIM>;
  auto kernel = attention_kernel<DIM>;
  static std::atomic<unsigned long long> configured{0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.fetch_or(bit, std::memory_order_release);
  }
  // [batch, seq, head, dim] as a 4-D tensor: dim contiguous, heads dim apart, rows ld apart
  const uint64_t dims[4] = {a.dim, a.heads, a.seq, a.batch};
  const uint64_t strides[3] = {static_cast<uint64_t>(a.dim) * 4, a.ld * 4,
                               (a.batch > 1 ? a.batch_stride : a.ld * a.seq) * 4};
  const uint32_t box_rows[4] = {32, 1, 128, 1};  // Q and K: 128 rows x 32 floats, K-major tiles
  const uint32_t box_v[4] = {32, 1, 32, 1};      // V: 32 key rows x 32 floats, MN-major chunks
  CUtensorMap tq, tk, tv;
  if (!encode_tmap_f32(&tq, a.q, 4, dims, strides, box_rows, 0) ||
      !encode_tmap_f32(&tk, a.k, 4, dims, strides, box_rows, 0) ||
      !encode_tmap_f32(&tv, a.v, 4, dims, strides, box_v, 1))
    return TFCCB200_EINVAL;
  AttParams p = {};
  p.out = a.out;
  p.seq = a.seq; p.heads = a.heads; p.dim = a.dim;
  p.ld_out = a.ld_out;
  p.scale = a.scale;
  p.status = a.status;
  p.timeout_ns = kDefaultTimeoutNs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.batch * a.heads, 1, 1);
  cfg.blockDim = dim3(kAttThreads, 1, 1);
  cfg.dynamicSmemBytes = L::kSmem;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kernel, tq, tk, tv, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

}  // namespace

int attention_f32(const AttentionArgs& a) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  if (di->cc_major != 10) return TFCCB200_EUNSUPPORTED;
  if (!attention_supported(a)) return TFCCB200_EUNSUPPORTED;
  return a.dim == 64 ? launch_attention<64>(a) : launch_attention<32>(a);
}

}  // namespace tfccb200
