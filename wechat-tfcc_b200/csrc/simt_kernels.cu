// CUDA-core kernels: the any-shape fp32 and int8 GEMMs that take whatever the
// tensor-core path cannot (unaligned pitches, tiny problems), the streaming
// kernel for M <= 8, and the integer row / column sums of the quantized path.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "act.cuh"
#include "internal.h"
#include "pdl.cuh"

namespace tfccb200 {

namespace {

// --------------------------------------------------------------------------
// Any-shape tiled GEMM: 64x64 tile, 16-deep k-slab, 256 threads, 4x4 outputs
// per thread.  Scalar guarded loads, so no alignment or divisibility demands.
// fp32 accumulates with FMA in k order; int8 accumulates exactly in int32.
// --------------------------------------------------------------------------
template <class TA, class TB, class TAcc>
struct Widen;
template <>
struct Widen<float, float, float> {
  static __device__ __forceinline__ float a(float v) { return v; }
  static __device__ __forceinline__ float b(float v) { return v; }
};
template <>
struct Widen<uint8_t, int8_t, int32_t> {
  static __device__ __forceinline__ int32_t a(uint8_t v) { return static_cast<int32_t>(v); }
  static __device__ __forceinline__ int32_t b(int8_t v) { return static_cast<int32_t>(v); }
};

struct SimtEpilogue {
  int activation;           // fp32: TFCCB200_ACT_*
  const float* bias;        // fp32
  const int32_t* rsA;       // int8
  const int32_t* rsB;
  unsigned strideRsA, strideRsB;
  int32_t offA, offB, kterm;
  const int32_t* dev_offsets;  // int8: device {offA, offB} replacing the three above
};

template <class TA, class TB, class TAcc>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const TA* __restrict__ A, const TB* __restrict__ B, TAcc* __restrict__ C,
                 unsigned M, unsigned N, unsigned K, unsigned long long strideA,
                 unsigned long long strideB, unsigned long long strideC, SimtEpilogue ep) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ TAcc As[TK][TM + 4];
  __shared__ TAcc Bs[TK][TN + 4];
  using W = Widen<TA, TB, TAcc>;

  const unsigned b = blockIdx.z;
  A += strideA * b;
  B += strideB * b;
  C += strideC * b;
  const unsigned m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const unsigned tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  TAcc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;

  for (unsigned k0 = 0; k0 < K; k0 += TK) {
    // A slab: 64 rows x 16 k, read along k (contiguous), stored k-major
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      unsigned idx = threadIdx.x + i * 256;
      unsigned r = idx >> 4, kk = idx & 15;
      unsigned gr = m0 + r, gk = k0 + kk;
      As[kk][r] = (gr < M && gk < K) ? W::a(A[static_cast<size_t>(gr) * K + gk]) : TAcc(0);
    }
    // B slab: 16 k x 64 columns, read along n (contiguous)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      unsigned idx = threadIdx.x + i * 256;
      unsigned kk = idx >> 6, c = idx & 63;
      unsigned gk = k0 + kk, gc = n0 + c;
      Bs[kk][c] = (gk < K && gc < N) ? W::b(B[static_cast<size_t>(gk) * N + gc]) : TAcc(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      TAcc av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    unsigned r = m0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      unsigned c = n0 + tx * 4 + j;
      if (c >= N) continue;
      TAcc v = acc[i][j];
      if constexpr (sizeof(TA) == 4) {
        if (ep.bias) v += ep.bias[c];
        v = apply_activation(v, ep.activation);
      } else {
        int32_t oa = ep.offA, ob = ep.offB, kt = ep.kterm;
        if (ep.dev_offsets) {
          oa = ep.dev_offsets[0];
          ob = ep.dev_offsets[1];
          kt = static_cast<int32_t>(static_cast<uint32_t>(oa) * static_cast<uint32_t>(ob) * K);
        }
        v = static_cast<int32_t>(
            static_cast<uint32_t>(v) + static_cast<uint32_t>(kt) +
            static_cast<uint32_t>(ep.rsA[static_cast<size_t>(ep.strideRsA) * b + r]) *
                static_cast<uint32_t>(ob) +
            static_cast<uint32_t>(ep.rsB[static_cast<size_t>(ep.strideRsB) * b + c]) *
                static_cast<uint32_t>(oa));
      }
      C[static_cast<size_t>(r) * N + c] = v;
    }
  }
}

// --------------------------------------------------------------------------
// M <= 8 streaming kernel.  y[m,n] = sum_k x[m,k] W[k,n] with W row-major, so
// the contiguous direction of the big operand is n: a thread owns 4 adjacent
// columns (one 128-bit load per row of W), a warp 128 columns, a CTA 1024
// columns = 4 KB of every row it visits.  K is cut into slices so that the
// grid fills every SM several times; a slice's partial sums go to scratch and
// a second tiny kernel adds the slices in a fixed order (deterministic).
// The x slice sits in shared memory as [k][MP] so one broadcast 128-bit read
// yields four rows' multipliers.
// --------------------------------------------------------------------------
constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyCols = kSkinnyThreads * 4;
// rows of W per CTA: bounds the x slice in shared memory to 32 KB
__host__ __device__ constexpr int skinny_max_slice(int mp) { return mp <= 16 ? 512 : 256; }
// weight rows in flight per thread (two batches of U 128-bit loads live at once)
__host__ __device__ constexpr int skinny_unroll(int mp) { return mp <= 16 ? 8 : 4; }

// acc[m] (4 columns as two packed pairs) += x[m] * w, with the packed fp32x2 FMA of sm_100.
template <int MP>
__device__ __forceinline__ void skinny_row_fma(float2 (&acc)[MP][2], const float* __restrict__ xrow,
                                               const float4& w) {
  float xv[MP];
  if constexpr (MP % 4 == 0) {
#pragma unroll
    for (int q = 0; q < MP / 4; ++q) {
      const float4 t = reinterpret_cast<const float4*>(xrow)[q];  // broadcast 128-bit read
      xv[4 * q + 0] = t.x; xv[4 * q + 1] = t.y; xv[4 * q + 2] = t.z; xv[4 * q + 3] = t.w;
    }
  } else if constexpr (MP == 2) {
    const float2 t = *reinterpret_cast<const float2*>(xrow);
    xv[0] = t.x; xv[1] = t.y;
  } else {
    xv[0] = xrow[0];
  }
  const float2 wlo = make_float2(w.x, w.y), whi = make_float2(w.z, w.w);
#pragma unroll
  for (int m = 0; m < MP; ++m) {
    const float2 xx = make_float2(xv[m], xv[m]);
    acc[m][0] = __ffma2_rn(xx, wlo, acc[m][0]);
    acc[m][1] = __ffma2_rn(xx, whi, acc[m][1]);
  }
}

// CTAs of the kernel that fit one SM (register-bound); the grid is planned as one full wave.
constexpr int skinny_resident(int mp) { return mp == 1 ? 3 : (mp <= 8 ? 2 : 1); }

template <int MP>
__global__ void __launch_bounds__(kSkinnyThreads, skinny_resident(MP))
skinny_partial_kernel(const float* __restrict__ X, const float* __restrict__ W,
                      float* __restrict__ part, unsigned M, unsigned N, unsigned K,
                      unsigned slice_rows, unsigned long long strideX, unsigned long long strideW,
                      unsigned kslices) {
  __shared__ __align__(16) float xs[skinny_max_slice(MP) * MP];
  pdl_wait();  // launched to overlap the previous kernel's tail: no global access before this
  const unsigned b = blockIdx.z;
  X += strideX * b;
  W += strideW * b;
  const unsigned k_begin = blockIdx.y * slice_rows;
  const unsigned k_end = min(K, k_begin + slice_rows);
  const unsigned rows = k_end > k_begin ? k_end - k_begin : 0;
  const unsigned col = blockIdx.x * kSkinnyCols + threadIdx.x * 4;
  const bool active = col < N;  // N % 4 == 0 on this path
  const float4* wp =
      reinterpret_cast<const float4*>(W + static_cast<size_t>(k_begin) * N + (active ? col : 0));
  const size_t pitch = N / 4;
  constexpr int U = skinny_unroll(MP);

  // first batch of weight rows is requested before the x slice is staged
  float4 w[U];
#pragma unroll
  for (int u = 0; u < U; ++u)
    w[u] = (active && static_cast<unsigned>(u) < rows) ? __ldcs(wp + u * pitch)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);

  for (unsigned i = threadIdx.x; i < rows * MP; i += kSkinnyThreads) {
    unsigned kk = i / MP, m = i % MP;
    xs[i] = (m < M) ? X[static_cast<size_t>(m) * K + k_begin + kk] : 0.f;
  }
  __syncthreads();

  float2 acc[MP][2];
#pragma unroll
  for (int m = 0; m < MP; ++m) acc[m][0] = acc[m][1] = make_float2(0.f, 0.f);

  // software-pipelined: the next batch of U rows is in flight while this one is multiplied;
  // rows past the slice load nothing and multiply by zero weights
  for (unsigned kk = 0; kk < rows; kk += U) {
    float4 wn[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      wn[u] = (active && kk + U + u < rows) ? __ldcs(wp + (kk + U + u) * pitch)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (kk + u < rows) skinny_row_fma<MP>(acc, xs + (kk + u) * MP, w[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) w[u] = wn[u];
  }

  // let the dependent reduce kernel begin launching; it still waits for this grid's stores
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (active) {
    // part: [batch][kslices][M][N]
    float* pp = part + ((static_cast<size_t>(b) * kslices + blockIdx.y) * M) * N + col;
#pragma unroll
    for (int m = 0; m < MP; ++m)
      if (m < static_cast<int>(M))
        *reinterpret_cast<float4*>(pp + static_cast<size_t>(m) * N) =
            make_float4(acc[m][0].x, acc[m][0].y, acc[m][1].x, acc[m][1].y);
  }
}

// Adds the K slices in a fixed order, then the bias.  Eight lanes share an output quad: lane j
// adds slices j, j + 8, j + 16, ... (all its loads in flight together, two batches at most for
// the slice counts the planner makes), then the eight sums meet in a shuffle tree -- always the
// same order, so a result does not depend on the run.  (One thread per quad walking all the
// slices paid one round of L2 latency per batch of 8 slices: ten rounds for a 4096 x 4096
// weight.)  Launched with programmatic stream serialisation: it may start while the partial
// kernel drains, and waits for that kernel's memory to be visible before it reads the sums.
// LANES = 1 when there are outputs enough to fill the chip with one thread per quad.
template <int LANES>
__global__ void __launch_bounds__(128)
skinny_reduce_kernel(const float* __restrict__ part, const float* __restrict__ bias,
                     float* __restrict__ Y, unsigned MN, unsigned N, unsigned kslices,
                     unsigned long long strideY, int activation) {
  const unsigned b = blockIdx.y;
  const unsigned lane = threadIdx.x % LANES;
  const unsigned i = ((blockIdx.x * 128 + threadIdx.x) / LANES) * 4;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const bool live = i < MN;  // whole groups of eight lanes share i, and every lane shuffles
  const float* pp = part + static_cast<size_t>(b) * kslices * MN + (live ? i : 0);
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr unsigned U = 8;
  unsigned k = lane;
  if (live) {
    for (; k + (U - 1) * LANES < kslices; k += U * LANES) {
      float4 v[U];
#pragma unroll
      for (unsigned u = 0; u < U; ++u)
        v[u] = __ldcg(reinterpret_cast<const float4*>(pp + static_cast<size_t>(k + u * LANES) * MN));
#pragma unroll
      for (unsigned u = 0; u < U; ++u) { s.x += v[u].x; s.y += v[u].y; s.z += v[u].z; s.w += v[u].w; }
    }
    {
      float4 v[U];
#pragma unroll
      for (unsigned u = 0; u < U; ++u)
        v[u] = (k + u * LANES < kslices)
                   ? __ldcg(reinterpret_cast<const float4*>(pp + static_cast<size_t>(k + u * LANES) * MN))
                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (unsigned u = 0; u < U; ++u) { s.x += v[u].x; s.y += v[u].y; s.z += v[u].z; s.w += v[u].w; }
    }
  }
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) {
    s.x += __shfl_xor_sync(0xffffffffu, s.x, o);
    s.y += __shfl_xor_sync(0xffffffffu, s.y, o);
    s.z += __shfl_xor_sync(0xffffffffu, s.z, o);
    s.w += __shfl_xor_sync(0xffffffffu, s.w, o);
  }
  if (!live || lane != 0) return;
  if (bias) {
    const float4 bv = *reinterpret_cast<const float4*>(bias + (i % N));
    s.x += bv.x; s.y += bv.y; s.z += bv.z; s.w += bv.w;
  }
  if (activation != TFCCB200_ACT_NONE) {
    s.x = apply_activation(s.x, activation); s.y = apply_activation(s.y, activation);
    s.z = apply_activation(s.z, activation); s.w = apply_activation(s.w, activation);
  }
  *reinterpret_cast<float4*>(Y + strideY * b + i) = s;
}

// K slices: as many CTAs as are resident at once (one wave), slice length capped by the x
// buffer and rounded to whole batches of 8 rows.
void skinny_plan(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count,
                 unsigned* kslices, unsigned* slice_rows) {
  const unsigned col_blocks = (N + kSkinnyCols - 1) / kSkinnyCols;
  const int mp = M == 1 ? 1 : (M == 2 ? 2 : (M <= 4 ? 4 : (M <= 8 ? 8 : (M <= 16 ? 16 : 32))));
  const unsigned long long want = static_cast<unsigned long long>(skinny_resident(mp)) * sm_count;
  unsigned long long ks = want / (static_cast<unsigned long long>(col_blocks) * batch);
  // beyond 8 rows the partial sums (one M x N slab per slice, written and read once) would
  // outweigh the weights themselves unless the slices stay at least 2 M rows long
  if (M > 8 && ks > K / (2ull * M)) ks = K / (2ull * M);
  if (ks < 1) ks = 1;
  if (ks > K) ks = K;
  unsigned rows = static_cast<unsigned>((K + ks - 1) / ks);
  rows = (rows + 7) / 8 * 8;  // whole batches of 8 rows, no ragged tail inside a slice
  if (rows > static_cast<unsigned>(skinny_max_slice(mp))) rows = skinny_max_slice(mp);
  *slice_rows = rows;
  *kslices = (K + rows - 1) / rows;
}

// --------------------------------------------------------------------------
// Integer sums for the zero-point correction.
// --------------------------------------------------------------------------
template <class T, unsigned V>
__device__ __forceinline__ int32_t sum_vec(const uint4& v) {
  const T* e = reinterpret_cast<const T*>(&v);
  int32_t s = 0;
#pragma unroll
  for (unsigned j = 0; j < V; ++j) s += static_cast<int32_t>(e[j]);
  return s;
}

// Row sums.  TPR threads share a row (32 ... 256, chosen so that a thread issues one to four
// 128-bit loads, all in flight together); a CTA of 256 threads holds 256 / TPR rows.
template <class T, int TPR>
__global__ void __launch_bounds__(256)
reduce_rows_kernel(const T* __restrict__ src, unsigned total_rows, unsigned cols,
                   int32_t* __restrict__ dst) {
  constexpr unsigned V = 16 / sizeof(T);
  constexpr int kRowsPerCta = 256 / TPR;
  __shared__ int32_t warp_sums[8];
  pdl_release();  // the product that follows may run its preamble beside this
  pdl_wait();
  const unsigned row = blockIdx.x * kRowsPerCta + threadIdx.x / TPR;
  const unsigned t = threadIdx.x % TPR;
  int32_t s = 0;
  if (row < total_rows) {
    const T* p = src + static_cast<size_t>(row) * cols;
    if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0 && cols % V == 0) {
      const uint4* p4 = reinterpret_cast<const uint4*>(p);
      const unsigned n4 = cols / V;
      unsigned i = t;
      for (; i + 3 * TPR < n4; i += 4 * TPR) {
        const uint4 v0 = __ldg(p4 + i), v1 = __ldg(p4 + i + TPR), v2 = __ldg(p4 + i + 2 * TPR),
                    v3 = __ldg(p4 + i + 3 * TPR);
        s += sum_vec<T, V>(v0) + sum_vec<T, V>(v1) + sum_vec<T, V>(v2) + sum_vec<T, V>(v3);
      }
      for (; i < n4; i += TPR) s += sum_vec<T, V>(__ldg(p4 + i));
    } else {
      for (unsigned i = t; i < cols; i += TPR) s += static_cast<int32_t>(p[i]);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if constexpr (TPR == 32) {
    if (t == 0 && row < total_rows) dst[row] = s;
  } else {
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
    __syncthreads();
    if (t == 0 && row < total_rows) {
      constexpr int kWarpsPerRow = TPR / 32;
      const int w0 = (threadIdx.x >> 5);
      int32_t total = 0;
#pragma unroll
      for (int w = 0; w < kWarpsPerRow; ++w) total += warp_sums[w0 + w];
      dst[row] = total;
    }
  }
}

// Column sums without atomics or a zeroed destination.  A CTA reads one 128-byte line of
// each row it visits (8 threads x 128 bits = 8 V columns) with 32 rows in flight per pass and
// several passes unrolled; a cluster of 8 CTAs shares the rows of one column block, and the
// eight partial results meet in the first CTA's shared memory (distributed shared memory),
// which adds them and writes the sums.  Needs cols % V == 0 and a 16-byte aligned base.
constexpr int kColsCluster = 8;

// LANES threads share a row segment of LANES x 16 bytes: 8 (a 128-byte line; most CTAs for a
// small operand) or 32 (512 contiguous bytes per row, kinder to DRAM pages, when the operand is
// wide enough to still fill the chip).
template <class T, int LANES>
__global__ void __launch_bounds__(256)
reduce_cols_cluster_kernel(const T* __restrict__ src, unsigned rows, unsigned cols,
                           int32_t* __restrict__ dst) {
  constexpr unsigned V = 16 / sizeof(T);
  constexpr unsigned CW = LANES * V;  // columns per CTA
  constexpr unsigned RL = 256 / LANES;  // rows per pass
  __shared__ int32_t part[RL][CW + 4];
  __shared__ int32_t gather[kColsCluster][CW];
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  // every CTA of the cluster is running before anyone writes into a peer's shared memory
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  pdl_release();
  pdl_wait();
  const unsigned b = blockIdx.z;
  const unsigned lane8 = threadIdx.x % LANES, rlane = threadIdx.x / LANES;
  const unsigned col = blockIdx.y * CW + lane8 * V;
  const bool active = col < cols;
  const unsigned slab = (rows + kColsCluster - 1) / kColsCluster;
  const unsigned r0 = rank * slab;
  const unsigned r1 = min(rows, r0 + slab);
  const uint4* p = reinterpret_cast<const uint4*>(src + static_cast<size_t>(b) * rows * cols +
                                                  (active ? col : 0));
  const size_t pitch = cols / V;  // in 128-bit units
  int32_t acc[V];
#pragma unroll
  for (unsigned v = 0; v < V; ++v) acc[v] = 0;
  if (active) {
    constexpr unsigned U = 8;  // two batches in flight: one round of latency for 512 rows per CTA
    unsigned r = r0 + rlane;
    // full batches of U rows per thread, the next batch requested before this one is added
    // (a slab of more than 512 rows would otherwise pay one round of latency per batch)
    if (r + (U - 1) * RL < r1) {
      uint4 w[U];
#pragma unroll
      for (unsigned u = 0; u < U; ++u) w[u] = __ldcs(p + static_cast<size_t>(r + u * RL) * pitch);
      for (;;) {
        const unsigned rn = r + U * RL;
        const bool more = rn + (U - 1) * RL < r1;
        uint4 nx[U];
        if (more) {
#pragma unroll
          for (unsigned u = 0; u < U; ++u) nx[u] = __ldcs(p + static_cast<size_t>(rn + u * RL) * pitch);
        }
#pragma unroll
        for (unsigned u = 0; u < U; ++u) {
          const T* e = reinterpret_cast<const T*>(&w[u]);
#pragma unroll
          for (unsigned v = 0; v < V; ++v) acc[v] += static_cast<int32_t>(e[v]);
        }
        r = rn;
        if (!more) break;
#pragma unroll
        for (unsigned u = 0; u < U; ++u) w[u] = nx[u];
      }
    }
    for (; r < r1; r += RL) {
      const uint4 w = __ldcs(p + static_cast<size_t>(r) * pitch);
      const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
      for (unsigned v = 0; v < V; ++v) acc[v] += static_cast<int32_t>(e[v]);
    }
  }
#pragma unroll
  for (unsigned v = 0; v < V; ++v) part[rlane][lane8 * V + v] = acc[v];
  __syncthreads();
  constexpr unsigned kPer = (CW + 255) / 256;  // columns per thread in the tree
  int32_t s[kPer];
#pragma unroll
  for (unsigned j = 0; j < kPer; ++j) {
    const unsigned c = threadIdx.x + j * 256;
    s[j] = 0;
    if (c < CW) {
#pragma unroll 8
      for (unsigned r = 0; r < RL; ++r) s[j] += part[r][c];
    }
  }
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
#pragma unroll
  for (unsigned j = 0; j < kPer; ++j) {
    const unsigned c = threadIdx.x + j * 256;
    if (c < CW) {
      const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(&gather[rank][c]));
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0u));
      asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(s[j]) : "memory");
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (rank == 0) {
#pragma unroll
    for (unsigned j = 0; j < kPer; ++j) {
      const unsigned cc = threadIdx.x + j * 256;
      const unsigned c = blockIdx.y * CW + cc;
      if (cc < CW && c < cols) {
        int32_t total = 0;
#pragma unroll
        for (int k = 0; k < kColsCluster; ++k) total += gather[k][cc];
        dst[static_cast<size_t>(b) * cols + c] = total;
      }
    }
  }
}

// Any alignment: one column per thread; dst must be zero on entry (row slabs are combined
// with integer atomics, which is exact and order-independent).
template <class T>
__global__ void __launch_bounds__(256)
reduce_cols_kernel(const T* __restrict__ src, unsigned rows, unsigned cols, unsigned slab,
                   int32_t* __restrict__ dst) {
  const unsigned b = blockIdx.z;
  const unsigned c = blockIdx.x * 256 + threadIdx.x;
  if (c >= cols) return;
  const unsigned r0 = blockIdx.y * slab;
  const unsigned r1 = min(rows, r0 + slab);
  const T* p = src + static_cast<size_t>(b) * rows * cols + c;
  int32_t s = 0;
  for (unsigned r = r0; r < r1; ++r) s += static_cast<int32_t>(p[static_cast<size_t>(r) * cols]);
  atomicAdd(dst + static_cast<size_t>(b) * cols + c, s);
}

// out[m][g*ns + j] = src[g][m][j], 128 bits per thread.
__global__ void __launch_bounds__(256)
interleave_panels_kernel(const float4* __restrict__ src, float4* __restrict__ out, unsigned M,
                         unsigned ns4, unsigned G) {
  const unsigned long long total = static_cast<unsigned long long>(G) * M * ns4;
  for (unsigned long long i = blockIdx.x * 256ull + threadIdx.x; i < total;
       i += static_cast<unsigned long long>(gridDim.x) * 256ull) {
    const unsigned j = static_cast<unsigned>(i % ns4);
    const unsigned long long r = i / ns4;
    const unsigned g = static_cast<unsigned>(r % G);
    const unsigned long long m = r / G;
    out[i] = __ldcs(src + (static_cast<unsigned long long>(g) * M + m) * ns4 + j);
  }
}

// fp32 -> bfloat16 (round to nearest even), 8 elements per thread per step.
__global__ void __launch_bounds__(256)
convert_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t n8 = n / 8;
  for (size_t i = blockIdx.x * 256ull + threadIdx.x; i < n8; i += gridDim.x * 256ull) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i);
    const float4 b = __ldcs(reinterpret_cast<const float4*>(src) + 2 * i + 1);
    __nv_bfloat162 o[4];
    o[0] = __floats2bfloat162_rn(a.x, a.y);
    o[1] = __floats2bfloat162_rn(a.z, a.w);
    o[2] = __floats2bfloat162_rn(b.x, b.y);
    o[3] = __floats2bfloat162_rn(b.z, b.w);
    reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(o);
  }
  for (size_t i = n8 * 8 + blockIdx.x * 256ull + threadIdx.x; i < n; i += gridDim.x * 256ull)
    dst[i] = __float2bfloat16_rn(src[i]);
}

inline cudaError_t launch_status() { return cudaGetLastError(); }

}  // namespace

int simt_sgemm(const SgemmArgs& a) {
  dim3 grid((a.N + 63) / 64, (a.M + 63) / 64, a.batch);
  if (grid.y > 65535 || grid.z > 65535) return TFCCB200_EOVERFLOW;
  SimtEpilogue ep = {};
  ep.bias = a.bias;
  ep.activation = a.activation;
  simt_gemm_kernel<float, float, float><<<grid, 256, 0, a.stream>>>(
      a.A, a.B, a.C, a.M, a.N, a.K, a.strideA, a.strideB, a.strideC, ep);
  cudaError_t e = launch_status();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

int simt_qgemm(const QgemmArgs& a) {
  dim3 grid((a.N + 63) / 64, (a.M + 63) / 64, a.batch);
  if (grid.y > 65535 || grid.z > 65535) return TFCCB200_EOVERFLOW;
  SimtEpilogue ep = {};
  ep.rsA = a.rsA; ep.rsB = a.rsB;
  ep.strideRsA = a.strideRsA; ep.strideRsB = a.strideRsB;
  ep.offA = a.offA; ep.offB = a.offB;
  ep.dev_offsets = a.dev_offsets;
  ep.kterm = static_cast<int32_t>(static_cast<uint32_t>(a.offA) * static_cast<uint32_t>(a.offB) *
                                  a.K);
  simt_gemm_kernel<uint8_t, int8_t, int32_t><<<grid, 256, 0, a.stream>>>(
      a.A, a.B, a.C, a.M, a.N, a.K, a.strideA, a.strideB, a.strideC, ep);
  cudaError_t e = launch_status();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

bool skinny_sgemm_supported(const SgemmArgs& a) {
  if (a.M > 32 || a.N % 4 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.B) & 15u) || (reinterpret_cast<uintptr_t>(a.C) & 15u))
    return false;
  if (a.bias && (reinterpret_cast<uintptr_t>(a.bias) & 15u)) return false;
  if (a.batch > 1 && (a.strideB % 4 != 0 || a.strideC % 4 != 0)) return false;
  if (a.batch > 65535) return false;
  return true;
}

size_t skinny_sgemm_workspace(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count) {
  unsigned ks, rows;
  skinny_plan(M, N, K, batch, sm_count, &ks, &rows);
  return static_cast<size_t>(batch) * ks * M * N * sizeof(float);
}

int skinny_sgemm(const SgemmArgs& a) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  if (!skinny_sgemm_supported(a)) return TFCCB200_EUNSUPPORTED;
  unsigned ks, rows;
  skinny_plan(a.M, a.N, a.K, a.batch, di->sm_count, &ks, &rows);
  const size_t need = static_cast<size_t>(a.batch) * ks * a.M * a.N * sizeof(float);
  if (a.workspace_bytes < need || !a.workspace ||
      (reinterpret_cast<uintptr_t>(a.workspace) & 15u))
    return TFCCB200_EWORKSPACE;
  float* part = static_cast<float*>(a.workspace);
  dim3 grid((a.N + kSkinnyCols - 1) / kSkinnyCols, ks, a.batch);
  if (grid.y > 65535) return TFCCB200_EOVERFLOW;
#define TFCCB200_SKINNY(MP)                                                                  \
  launch_after_previous(skinny_partial_kernel<MP>, grid, dim3(kSkinnyThreads), 0, a.stream, a.A,  \
                        a.B, part, a.M, a.N, a.K, rows, a.strideA, a.strideB, ks)
  if (a.M == 1) TFCCB200_SKINNY(1);
  else if (a.M == 2) TFCCB200_SKINNY(2);
  else if (a.M <= 4) TFCCB200_SKINNY(4);
  else if (a.M <= 8) TFCCB200_SKINNY(8);
  else if (a.M <= 16) TFCCB200_SKINNY(16);
  else TFCCB200_SKINNY(32);
#undef TFCCB200_SKINNY
  cudaError_t e = launch_status();
  if (e != cudaSuccess) return static_cast<int>(e);
  const unsigned MN = a.M * a.N;
  cudaLaunchConfig_t cfg = {};
  // eight lanes per output quad unless one thread per quad already fills the chip
  const bool wide = MN / 4 < 16384u;
  cfg.gridDim = dim3(wide ? (MN / 4 + 15) / 16 : (MN / 4 + 127) / 128, a.batch, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const float* part_c = part;
  const float* bias_c = a.bias;
  float* out_c = a.C;
  unsigned n_c = a.N;
  unsigned long long stride_c = a.strideC;
  int act_c = a.activation;
  e = wide ? cudaLaunchKernelEx(&cfg, skinny_reduce_kernel<8>, part_c, bias_c, out_c, MN, n_c, ks,
                                stride_c, act_c)
           : cudaLaunchKernelEx(&cfg, skinny_reduce_kernel<1>, part_c, bias_c, out_c, MN, n_c, ks,
                                stride_c, act_c);
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch(2);
  return TFCCB200_OK;
}

int convert_f32_to_bf16(cudaStream_t stream, const float* src, void* dst, size_t n) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  size_t blocks = (n / 8 + 255) / 256;
  const size_t cap = static_cast<size_t>(di->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  convert_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      src, static_cast<__nv_bfloat16*>(dst), n);
  cudaError_t e = launch_status();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

int interleave_panels_f32(cudaStream_t stream, const float* src, float* out, unsigned M,
                          unsigned ns, unsigned G) {
  if (ns % 4 != 0 || (reinterpret_cast<uintptr_t>(src) & 15u) ||
      (reinterpret_cast<uintptr_t>(out) & 15u))
    return TFCCB200_EALIGN;
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  const unsigned long long total = static_cast<unsigned long long>(G) * M * (ns / 4);
  unsigned long long blocks = (total + 255) / 256;
  const unsigned long long cap = 16ull * di->sm_count;
  if (blocks > cap) blocks = cap;
  interleave_panels_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(out), M, ns / 4, G);
  cudaError_t e = launch_status();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

// --------------------------------------------------------------------------
// The M <= 8 kernel for callers that cannot give it scratch memory.
//
// Its per-slice partial sums live in a fixed array inside this library's device image
// instead of caller-provided workspace.  Every GPU that loads the library carries the
// array (20 MiB) until the process exits.  All calls on a device share it and it keeps
// whatever the previous call left there; that is harmless because every element a call
// reads was written by the same call first (nothing has to start at zero), but two calls
// that run on the GPU at the same time -- different streams, or different host threads --
// would overwrite each other's partial sums.
// --------------------------------------------------------------------------
constexpr size_t kStaticScratchFloats = size_t(5) << 20;  // 5 Mi floats = 20 MiB
static __device__ __align__(256) float g_skinny_static_scratch[kStaticScratchFloats];

int skinny_sgemm_static(cudaStream_t stream, const float* A, const float* B, float* C,
                        const float* bias, unsigned M, unsigned N, unsigned K) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  int dev = 0;
  if ((ce = cudaGetDevice(&dev)) != cudaSuccess) return static_cast<int>(ce);
  if (dev < 0 || dev >= 64) return TFCCB200_EUNSUPPORTED;

  // In host code the array's name is only a handle; the address the kernels need is looked
  // up once per device, with that device current, and remembered.
  static std::mutex mu;
  static float* device_address[64] = {};
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!device_address[dev]) {
      void* p = nullptr;
      ce = cudaGetSymbolAddress(&p, g_skinny_static_scratch);
      if (ce != cudaSuccess) return static_cast<int>(ce);
      device_address[dev] = static_cast<float*>(p);
    }
    scratch = device_address[dev];
  }

  SgemmArgs a = {};
  a.stream = stream;
  a.A = A; a.B = B; a.C = C; a.bias = bias;
  a.strideA = a.strideB = 0;
  a.strideC = M * N;
  a.M = M; a.N = N; a.K = K; a.batch = 1;
  a.precision = TFCCB200_PRECISION_FP32;
  a.workspace = scratch;
  a.workspace_bytes = kStaticScratchFloats * sizeof(float);
  a.status = nullptr;
  if (!skinny_sgemm_supported(a)) return TFCCB200_EUNSUPPORTED;
  if (skinny_sgemm_workspace(M, N, K, 1, di->sm_count) > a.workspace_bytes)
    return TFCCB200_ESTATICLIMIT;
  return skinny_sgemm(a);
}

size_t skinny_sgemm_static_capacity() { return kStaticScratchFloats * sizeof(float); }

template <class T, int TPR>
cudaError_t launch_reduce_rows(cudaStream_t stream, const T* src, unsigned total_rows,
                               unsigned cols, int32_t* dst) {
  constexpr unsigned kRowsPerCta = 256 / TPR;
  const unsigned blocks = (total_rows + kRowsPerCta - 1) / kRowsPerCta;
  return launch_after_previous(reduce_rows_kernel<T, TPR>, dim3(blocks), dim3(256), 0, stream, src,
                               total_rows, cols, dst);
}

template <class T>
int reduce_sum(cudaStream_t stream, const T* src, unsigned batch, unsigned rows, unsigned cols,
               int row_flag, int32_t* dst) {
  constexpr unsigned V = 16 / sizeof(T);
  if (row_flag) {
    const unsigned long long total = static_cast<unsigned long long>(batch) * rows;
    if (total > 0xffffffffull) return TFCCB200_EOVERFLOW;
    const unsigned n = static_cast<unsigned>(total);
    const unsigned loads = (cols + V - 1) / V;  // 128-bit loads per row
    cudaError_t e;
    if (loads <= 64) e = launch_reduce_rows<T, 32>(stream, src, n, cols, dst);
    else if (loads <= 128) e = launch_reduce_rows<T, 64>(stream, src, n, cols, dst);
    else if (loads <= 512) e = launch_reduce_rows<T, 128>(stream, src, n, cols, dst);
    else e = launch_reduce_rows<T, 256>(stream, src, n, cols, dst);
    if (e != cudaSuccess) return static_cast<int>(e);
    count_launch();
    return TFCCB200_OK;
  }
  if (batch > 65535) return TFCCB200_EOVERFLOW;
  if (cols % V == 0 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0 &&
      (cols + 8 * V - 1) / (8 * V) <= 65535) {
    cudaError_t ce;
    const DeviceInfo* di = current_device_info(&ce);
    if (!di) return static_cast<int>(ce);
    // 512-byte row segments when that still leaves a CTA for every SM
    const unsigned wide_blocks = (cols + 32 * V - 1) / (32 * V);
    const bool wide = static_cast<unsigned long long>(wide_blocks) * kColsCluster * batch >=
                      static_cast<unsigned long long>(di->sm_count);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kColsCluster, wide ? wide_blocks : (cols + 8 * V - 1) / (8 * V), batch);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kColsCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = wide ? cudaLaunchKernelEx(&cfg, reduce_cols_cluster_kernel<T, 32>, src, rows, cols, dst)
                         : cudaLaunchKernelEx(&cfg, reduce_cols_cluster_kernel<T, 8>, src, rows, cols, dst);
    if (e != cudaSuccess) return static_cast<int>(e);
    count_launch();
    return TFCCB200_OK;
  }
  cudaError_t e =
      cudaMemsetAsync(dst, 0, static_cast<size_t>(batch) * cols * sizeof(int32_t), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  unsigned slab = 64;
  while ((rows + slab - 1) / slab > 4096) slab *= 2;
  dim3 grid((cols + 255) / 256, (rows + slab - 1) / slab, batch);
  reduce_cols_kernel<T><<<grid, 256, 0, stream>>>(src, rows, cols, slab, dst);
  e = launch_status();
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

template int reduce_sum<uint8_t>(cudaStream_t, const uint8_t*, unsigned, unsigned, unsigned, int,
                                 int32_t*);
template int reduce_sum<int8_t>(cudaStream_t, const int8_t*, unsigned, unsigned, unsigned, int,
                                int32_t*);
template int reduce_sum<int16_t>(cudaStream_t, const int16_t*, unsigned, unsigned, unsigned, int,
                                 int32_t*);

}  // namespace tfccb200
