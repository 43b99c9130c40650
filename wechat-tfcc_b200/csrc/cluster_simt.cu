// C = A . B (+ bias, activation) for few rows (M <= 32) and a SMALL B, in one launch.
//
// The shapes this serves (config 1 of the benchmarks: 32 x 512 x 2048) are bound by latency,
// not by arithmetic or bandwidth: a few megabytes of B, a few tens of MFLOP.  The tensor-core
// kernel pays its fixed pipeline cost for them and the streaming kernel for few rows
// (simt_kernels.cu) needs a second launch to add its K slices.  Here K is cut into
// ways x cluster slices so that every thread has 8 to 64 rows of B to visit (16 for config 1,
// all requested at once), and the slices are added through distributed shared
// memory inside a thread-block cluster in a fixed order (deterministic).
//
//   grid  (ceil(N / 256), ks, row_groups * batch), cluster (1, ks, 1), block (64, 4)
//   thread (lane, way) of cluster rank r owns columns [256 bx + 4 lane, +4), rows
//   [8 rg, +8) of A and rows [(4 r + way) rows_per_way, +rows_per_way) of B.
//
// B is read once per row group (at most four times for 32 rows), from L2 after the first.
// Replaces, for these shapes, what MKLBlasInterface<float>::matmul / CUDABlasInterface<T>::matmul
// hand to their libraries (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-186,
// tfcc/cuda/interfaces/tfcc_cudablasinterface.cu:201-303).
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>

#include "act.cuh"
#include "internal.h"
#include "pdl.cuh"

namespace cg = cooperative_groups;

namespace tfccb200 {

namespace {

constexpr int kLanes = 64;        // threads across the columns, four columns each
constexpr int kCols = kLanes * 4;
constexpr int kWays = 4;          // K ways inside a CTA
constexpr int kRows = 8;          // rows of A per CTA
constexpr int kSlice = 64;        // most rows of B per way
constexpr int kMaxCluster = 8;    // portable cluster size
constexpr int kInFlight = 8;      // rows of B requested together by a thread (two such batches)

__global__ void __launch_bounds__(kLanes* kWays)
cluster_simt_kernel(const float* __restrict__ X, const float* __restrict__ W,
                    const float* __restrict__ bias, float* __restrict__ Y, unsigned M, unsigned N,
                    unsigned K, unsigned rows_per_way, unsigned row_groups,
                    unsigned long long strideX, unsigned long long strideW,
                    unsigned long long strideY, int activation) {
  __shared__ __align__(16) float xs[kWays][kSlice][kRows];
  __shared__ __align__(16) float4 part[kWays][kRows][kLanes];
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned ks = cluster.dim_blocks().y;
  const unsigned crank = cluster.block_rank();
  const unsigned lane = threadIdx.x, way = threadIdx.y;
  const unsigned rg = blockIdx.z % row_groups, b = blockIdx.z / row_groups;
  const unsigned m0 = rg * kRows;
  const unsigned k_begin = min(K, (blockIdx.y * kWays + way) * rows_per_way);
  const unsigned k_end = min(K, k_begin + rows_per_way);
  const unsigned rows = k_end - k_begin;
  const unsigned col = blockIdx.x * kCols + lane * 4;
  const bool active = col < N;  // N % 4 == 0 on this path

  pdl_wait();  // no global access before this: the launch may overlap the previous kernel's tail
  X += strideX * b;
  W += strideW * b;
  Y += strideY * b;
  const float4* wp =
      reinterpret_cast<const float4*>(W + static_cast<size_t>(k_begin) * N + (active ? col : 0));
  const size_t pitch = N / 4;

  // the first rows of B are requested before this way's slice of A is staged
  float4 w[kInFlight];
#pragma unroll
  for (int u = 0; u < kInFlight; ++u)
    w[u] = (active && static_cast<unsigned>(u) < rows) ? __ldg(wp + u * pitch)
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
  for (unsigned i = lane; i < rows * kRows; i += kLanes) {
    const unsigned m = i / rows, kk = i - m * rows;  // consecutive lanes walk along K
    xs[way][kk][m] = (m0 + m < M) ? X[static_cast<size_t>(m0 + m) * K + k_begin + kk] : 0.f;
  }
  __syncthreads();

  float2 acc[kRows][2];
#pragma unroll
  for (int m = 0; m < kRows; ++m) acc[m][0] = acc[m][1] = make_float2(0.f, 0.f);
  for (unsigned kk = 0; kk < rows; kk += kInFlight) {
    float4 wn[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u)
      wn[u] = (active && kk + kInFlight + u < rows) ? __ldg(wp + (kk + kInFlight + u) * pitch)
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      if (kk + u < rows) {
        const float4 xa = *reinterpret_cast<const float4*>(&xs[way][kk + u][0]);
        const float4 xb = *reinterpret_cast<const float4*>(&xs[way][kk + u][4]);
        const float xv[kRows] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        const float2 wlo = make_float2(w[u].x, w[u].y), whi = make_float2(w[u].z, w[u].w);
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
          const float2 xx = make_float2(xv[m], xv[m]);
          acc[m][0] = __ffma2_rn(xx, wlo, acc[m][0]);
          acc[m][1] = __ffma2_rn(xx, whi, acc[m][1]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) w[u] = wn[u];
  }
  pdl_release();
#pragma unroll
  for (int m = 0; m < kRows; ++m)
    part[way][m][lane] = make_float4(acc[m][0].x, acc[m][0].y, acc[m][1].x, acc[m][1].y);
  __syncthreads();
  // the four ways of this CTA first (way 0 first), in place into way 0's slab ...
  const unsigned t = way * kLanes + lane;
  float4* mine = &part[0][0][0];
  for (unsigned i = t; i < kRows * kLanes; i += kLanes * kWays) {
    float4 v[kWays];
#pragma unroll
    for (int wy = 0; wy < kWays; ++wy) v[wy] = mine[wy * kRows * kLanes + i];
    float4 s = v[0];
#pragma unroll
    for (int wy = 1; wy < kWays; ++wy) { s.x += v[wy].x; s.y += v[wy].y; s.z += v[wy].z; s.w += v[wy].w; }
    mine[i] = s;  // item i of way 0 is read by this thread only
  }
  // ... then cluster rank r adds items [r share, (r+1) share) of the 8 x 64 float4 of the tile
  // over the ranks, rank 0 first, with every rank's value requested before the first is used.
  // (At most two items per thread; their bias is fetched before the cluster meets.)
  const unsigned share = kRows * kLanes / ks;
  constexpr int kItems = kRows * kLanes / (kLanes * kWays);
  float4 bv[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const unsigned i = crank * share + t + j * kLanes * kWays;
    const unsigned c = blockIdx.x * kCols + (i % kLanes) * 4;
    bv[j] = (bias && i < (crank + 1) * share && c < N)
                ? __ldg(reinterpret_cast<const float4*>(bias + c))
                : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  cluster.sync();
  float4 sum[kItems];
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const unsigned i = crank * share + t + j * kLanes * kWays;
    sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < (crank + 1) * share) {
      float4 v[kMaxCluster];
#pragma unroll
      for (int p = 0; p < kMaxCluster; ++p)
        if (static_cast<unsigned>(p) < ks) v[p] = cluster.map_shared_rank(mine, p)[i];
#pragma unroll
      for (int p = 0; p < kMaxCluster; ++p)
        if (static_cast<unsigned>(p) < ks) {
          sum[j].x += v[p].x; sum[j].y += v[p].y; sum[j].z += v[p].z; sum[j].w += v[p].w;
        }
    }
  }
  // this CTA has finished reading its peers' partial sums: say so now, store, and leave once
  // every peer has said the same (nobody exits while its shared memory may still be read)
  cluster.barrier_arrive();
#pragma unroll
  for (int j = 0; j < kItems; ++j) {
    const unsigned i = crank * share + t + j * kLanes * kWays;
    const unsigned m = i / kLanes, l = i % kLanes;
    const unsigned c = blockIdx.x * kCols + l * 4;
    if (i < (crank + 1) * share && m0 + m < M && c < N) {
      float4 s = sum[j];
      s.x += bv[j].x; s.y += bv[j].y; s.z += bv[j].z; s.w += bv[j].w;
      if (activation != TFCCB200_ACT_NONE) {
        s.x = apply_activation(s.x, activation); s.y = apply_activation(s.y, activation);
        s.z = apply_activation(s.z, activation); s.w = apply_activation(s.w, activation);
      }
      *reinterpret_cast<float4*>(Y + static_cast<size_t>(m0 + m) * N + c) = s;
    }
  }
  cluster.barrier_wait();
}

struct Plan {
  unsigned ks, rows_per_way, row_groups;
};

bool make_plan(unsigned M, unsigned K, Plan* p) {
  // Rows of B per thread to aim at: 16 are all requested at once (two batches of kInFlight);
  // a short K is cut finer still (measured 32x256x256: 5.6 us at 32 rows, 4.6 at 16, 3.7 at 8).
  static const unsigned env_aim = [] {
    const char* v = std::getenv("TFCCB200_CS_ROWS");
    const int n = v ? std::atoi(v) : 0;
    return n >= 8 ? static_cast<unsigned>(n) : 0u;
  }();
  const unsigned aim = env_aim ? env_aim : (K <= 256 ? 8u : 16u);
  unsigned ways = (K + aim - 1) / aim;
  unsigned ks = (ways + kWays - 1) / kWays;
  unsigned pow2 = 1;
  while (pow2 < ks) pow2 *= 2;
  ks = std::min<unsigned>(pow2, kMaxCluster);
  unsigned rows = (K + ks * kWays - 1) / (ks * kWays);
  rows = (rows + 7) / 8 * 8;
  if (rows > static_cast<unsigned>(kSlice)) return false;
  p->ks = ks;
  p->rows_per_way = rows;
  p->row_groups = (M + kRows - 1) / kRows;
  return true;
}

}  // namespace

bool cluster_simt_sgemm_supported(const SgemmArgs& a) {
  if (a.M > 32 || a.N % 4 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.B) & 15u) || (reinterpret_cast<uintptr_t>(a.C) & 15u))
    return false;
  if (a.bias && (reinterpret_cast<uintptr_t>(a.bias) & 15u)) return false;
  if (a.batch > 1 && (a.strideB % 4 != 0 || a.strideC % 4 != 0)) return false;
  if (a.num_dst > 1 || a.mc_dst || a.ldc || a.col_offset) return false;
  Plan p;
  if (!make_plan(a.M, a.K, &p)) return false;
  return static_cast<unsigned long long>(p.row_groups) * a.batch <= 65535ull;
}

int cluster_simt_sgemm(const SgemmArgs& a) {
  if (!cluster_simt_sgemm_supported(a)) return TFCCB200_EUNSUPPORTED;
  Plan p;
  make_plan(a.M, a.K, &p);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.N + kCols - 1) / kCols, p.ks, p.row_groups * a.batch);
  cfg.blockDim = dim3(kLanes, kWays, 1);
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = p.ks;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  const float* x = a.A;
  const float* w = a.B;
  const float* bias = a.bias;
  float* y = a.C;
  unsigned M = a.M, N = a.N, K = a.K, rows = p.rows_per_way, groups = p.row_groups;
  unsigned long long sx = a.strideA, sw = a.strideB, sy = a.strideC;
  int act = a.activation;
  cudaError_t e = cudaLaunchKernelEx(&cfg, cluster_simt_kernel, x, w, bias, y, M, N, K, rows, groups,
                                     sx, sw, sy, act);
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

}  // namespace tfccb200
