// Host side of the tcgen05 GEMMs: tensor-map encoding, tile-shape choice and
// launch (plain launch for one CTA per tile, cluster launch for CTA pairs).
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "internal.h"
#include "umma_gemm.cuh"

namespace tfccb200 {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver entry point; it is fetched through the
// runtime so the library links against cudart only.
EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(p);
    }
  });
  return fn;
}

// 3-D map over a batch of row-major matrices: dim0 = contiguous elements of a
// row, dim1 = rows, dim2 = batch entries.  The box is 128 bytes wide with the
// 128-byte swizzle; out-of-range elements read as zero, which is what makes
// ragged M, N and K tails free.
bool make_tmap(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
               uint64_t row_elems, uint64_t rows, uint64_t batch, uint64_t batch_stride_elems,
               uint32_t box_rows, CUtensorMapSwizzle swizzle) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {row_elems, rows, batch};
  uint64_t bstride = batch_stride_elems ? batch_stride_elems : row_elems * rows;
  cuuint64_t strides[2] = {row_elems * elem_bytes, bstride * elem_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / elem_bytes), box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int env_int(const char* name, int fallback);

// Test hook (tfccb200_test_flag_wait): limit and surplus expectation of the waits on scratch
// counters.  0 / 0 = the normal limit and no surplus.
std::atomic<unsigned long long> g_flag_timeout_ns{0};
std::atomic<unsigned> g_flag_expect_extra{0};

// Sharing the last one-to-two waves of tiles out by k-block (UmmaGemmParams::sk_tiles).
// Worth it when the tile count leaves a noticeable part of the last wave idle.
bool stream_k_split(unsigned long long tiles, unsigned groups, unsigned num_kb, unsigned kb_per_chunk,
                    unsigned* sk_tiles, unsigned* sk_kb_per_group) {
  static const int enabled = env_int("TFCCB200_STREAM_K", 1);
  if (!enabled || groups == 0 || tiles <= groups || tiles % groups == 0) return false;
  if (kb_per_chunk == 0 || num_kb % kb_per_chunk != 0) return false;
  const unsigned long long waves = (tiles + groups - 1) / groups;
  if (tiles * 100 >= waves * groups * 96) return false;  // >= 96 % busy already
  const unsigned long long dp_tiles = (tiles / groups - 1) * groups;
  const unsigned long long sk = tiles - dp_tiles;  // groups < sk < 2 * groups
  const unsigned long long chunks = sk * (num_kb / kb_per_chunk);
  const unsigned long long per = (chunks + groups - 1) / groups;
  if (per * kb_per_chunk > 0xffffffffull) return false;
  *sk_tiles = static_cast<unsigned>(sk);
  *sk_kb_per_group = static_cast<unsigned>(per * kb_per_chunk);  // >= num_kb because sk >= groups
  return true;
}

constexpr size_t kStreamKFlagBytes = 4096;  // one counter per CTA of the grid, padded

template <ptx::MmaKind kKind, bool kSplit, int kCtaGroup, int BN, int kStages>
int launch(cudaStream_t stream, const CUtensorMap& ta, const CUtensorMap& tb, UmmaGemmParams p,
           int sm_count) {
  // Tiles leave through a tensor map of C when there is one destination with the dense
  // layout the map describes (the multi-GPU push keeps ordinary stores: several destinations,
  // or a multicast alias).  TFCCB200_TMA_STORE=0 turns it off.
  static const int env_tma_store = env_int("TFCCB200_TMA_STORE", 1);
  CUtensorMap tc = {};
  p.tma_store = 0;
  if (env_tma_store && p.num_dst == 1 && !p.mc_dst && p.ldc % 4 == 0 && p.strideC % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(p.dst[0]) & 15u) == 0 && p.col_offset == 0) {
    const CUtensorMapDataType dt = kKind == ptx::MmaKind::I8 ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    if (make_tmap(&tc, dt, 4, p.dst[0], p.ldc, p.M, p.batch, p.batch > 1 ? p.strideC : 0, 32,
                  CU_TENSOR_MAP_SWIZZLE_128B))
      p.tma_store = 1;
  }
  using Cfg = UmmaGemmConfig<kKind, kSplit, kCtaGroup, BN, kStages>;
  auto kernel = umma_gemm_kernel<kKind, kSplit, kCtaGroup, BN, kStages>;
  // The opt-in shared-memory size is a per-device attribute of the function.
  static std::atomic<unsigned long long> configured{0};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured.fetch_or(bit, std::memory_order_release);
  }
  p.tiles_m = (p.M + Cfg::kTileM - 1) / Cfg::kTileM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const unsigned long long total =
      static_cast<unsigned long long>(p.tiles_m) * p.tiles_n * p.batch;
  if (total == 0 || total > 0x7fffffffull) return TFCCB200_EOVERFLOW;
  unsigned groups = static_cast<unsigned>(sm_count / kCtaGroup);
  if (total < groups) groups = static_cast<unsigned>(total);
  unsigned cluster = kCtaGroup;
  if (p.cluster_k > 1) {
    // K split over a cluster: one tile per cluster, all tiles resident at once
    constexpr bool kCapable = kCtaGroup == 1 && (kSplit || kKind == ptx::MmaKind::I8);
    if (!kCapable || total * p.cluster_k > static_cast<unsigned>(sm_count))
      return TFCCB200_EUNSUPPORTED;
    // fp32: the other ranks' whole partial tiles meet in rank 0's stage buffers; int8: every
    // rank receives the other ranks' BN / cluster_k columns
    const unsigned incoming = kSplit ? (p.cluster_k - 1) * 128u * BN * 4u
                                     : (p.cluster_k - 1) * 128u * (BN / p.cluster_k) * 4u;
    if (incoming > static_cast<unsigned>(Cfg::kRingBytes)) return TFCCB200_EUNSUPPORTED;
    if (!kSplit && (BN % p.cluster_k != 0 || (BN / p.cluster_k) % 32 != 0))
      return TFCCB200_EUNSUPPORTED;
    groups = static_cast<unsigned>(total) * p.cluster_k;
    cluster = p.cluster_k;
  } else {
    p.cluster_k = 1;
  }
  unsigned sk_tiles = 0, sk_per = 0;
  if (kSplit && kCtaGroup == 1 && p.global_k > 1 && p.sk_flags && p.cluster_k == 1 &&
      total * p.global_k <= static_cast<unsigned>(sm_count) &&
      static_cast<size_t>(total) * p.global_k * sizeof(unsigned) <= kStreamKFlagBytes &&
      total * p.global_k * Cfg::kBM * BN * 4ull <= p.sk_capacity) {
    // K shared by global_k consecutive CTAs per tile, partial tiles through the scratch
    groups = static_cast<unsigned>(total) * p.global_k;
    p.sk_tiles = static_cast<unsigned>(total);  // no tile is walked whole
    p.sk_kb_per_group = 0;
    e = cudaMemsetAsync(p.sk_flags, 0, static_cast<size_t>(groups) * sizeof(unsigned), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  } else if (kSplit && p.sk_flags && p.cluster_k == 1 &&
      stream_k_split(total, groups, (p.K + Cfg::kBK - 1) / Cfg::kBK, p.kb_per_chunk, &sk_tiles,
                     &sk_per) &&
      static_cast<size_t>(groups) * kCtaGroup * sizeof(unsigned) <= kStreamKFlagBytes &&
      static_cast<unsigned long long>(groups) * kCtaGroup * Cfg::kBM * BN * 4ull <= p.sk_capacity) {
    p.global_k = 1;
    p.sk_tiles = sk_tiles;
    p.sk_kb_per_group = sk_per;
    e = cudaMemsetAsync(p.sk_flags, 0, static_cast<size_t>(groups) * kCtaGroup * sizeof(unsigned),
                        stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  } else {
    p.global_k = 1;
    p.sk_tiles = 0;
    p.sk_kb_per_group = 0;
    p.sk_flags = nullptr;
    p.sk_partials = nullptr;
  }

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(groups * kCtaGroup, 1, 1);
  cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  count_launch();
  return TFCCB200_OK;
}

// How many clusters of `ks` single CTAs of the fp32 kernel the device holds at once.  The SMs
// of a cluster must share a GPC, so this is not sm_count / ks (a cluster of 3 fits 48 times in
// 148 SMs by count, yet fewer are co-resident and the grid then runs in two waves).
template <ptx::MmaKind kKind, bool kSplit, int BN, int kStages>
int query_active_clusters(unsigned ks) {
  using Cfg = UmmaGemmConfig<kKind, kSplit, 1, BN, kStages>;
  auto kernel = umma_gemm_kernel<kKind, kSplit, 1, BN, kStages>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           Cfg::kSmemBytes) != cudaSuccess)
    return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ks * 64, 1, 1);
  cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

// Cached per device, tile width and cluster size; 0 = not available.
int active_clusters_fp32(int bn, unsigned ks) {
  if (ks < 2 || ks > 4) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  static std::atomic<int> cache[64][3][5];  // value + 1; 0 = not queried yet
  const int w = bn == 256 ? 0 : (bn == 128 ? 1 : 2);
  std::atomic<int>& slot = cache[dev & 63][w][ks];
  int v = slot.load(std::memory_order_acquire);
  if (v == 0) {
    constexpr auto T = ptx::MmaKind::TF32;
    const int n = bn == 256 ? query_active_clusters<T, true, 256, 2>(ks)
                            : (bn == 128 ? query_active_clusters<T, true, 128, 4>(ks)
                                         : query_active_clusters<T, true, 64, 6>(ks));
    v = n + 1;
    slot.store(v, std::memory_order_release);
  }
  return v - 1;
}

// The same for the int8 kernel's single-CTA instantiations.
int active_clusters_i8(int bn, unsigned ks) {
  if (ks < 2 || ks > 4 || (bn != 128 && bn != 256)) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  static std::atomic<int> cache[64][2][5];
  std::atomic<int>& slot = cache[dev & 63][bn == 256 ? 0 : 1][ks];
  int v = slot.load(std::memory_order_acquire);
  if (v == 0) {
    constexpr auto I = ptx::MmaKind::I8;
    const int n = bn == 256 ? query_active_clusters<I, false, 256, 4>(ks)
                            : query_active_clusters<I, false, 128, 6>(ks);
    v = n + 1;
    slot.store(v, std::memory_order_release);
  }
  return v - 1;
}

// Tile shape of the int8 kernel, from a time model fitted to graph-replayed launches over
// rotating operands on B200: a launch costs a fixed part (launch, prologue, first loads,
// epilogue: 8.7 us for 128-wide single-CTA tiles, 12.5 us for 256-wide ones, 8 us for CTA
// pairs) plus its k-blocks times the time to fill one stage (0.25 us for 32 KB when half the
// SMs stream, 0.32 us when nearly all do; 0.62 us for the 48 KB of a 256-wide tile; 0.29 us
// per CTA of a pair).  Filling the stages is what bounds a CTA, so with fewer tiles than SMs the
// K range of a tile is shared by a cluster (reduce-scatter of the int32 partial sums through
// distributed shared memory, exact in any order): measured 256x4096x4096 16.8 -> 13.9 us,
// 128x4096x4096 16.6 -> 12.8 us, 256x1024x8192 24.3 -> 13.0 us.
struct I8Plan {
  bool pair;
  int bn;
  unsigned cluster_k;
};
I8Plan plan_i8(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count, int force_pair) {
  static const int env_bn = env_int("TFCCB200_I8_BN", 0);
  static const int env_ks = env_int("TFCCB200_I8_CLUSTER_K", -1);  // -1: planned; 1: off
  const unsigned num_kb = (K + 127) / 128;
  I8Plan best = {false, 0, 1};
  double best_t = 0;
  for (int pair = 0; pair <= 1; ++pair) {
    if (force_pair >= 0 && pair != force_pair) continue;
    for (int bn : {256, 128}) {
      if (pair && bn != 256) continue;
      if (env_bn && bn != env_bn && !pair) continue;
      if (bn > 128 && static_cast<unsigned>(bn) >= 2 * N) continue;
      const int tile_m = pair ? 256 : 128;
      const int groups = pair ? sm_count / 2 : sm_count;
      const unsigned long long tiles = static_cast<unsigned long long>((M + tile_m - 1) / tile_m) *
                                       ((N + bn - 1) / bn) * batch;
      if (pair && force_pair < 0 && tiles * 5 < static_cast<unsigned long long>(groups) * 3) continue;
      for (unsigned ks = 1; ks <= 4; ks *= 2) {
        if (ks > 1) {
          if (pair || env_ks == 1) break;
          if (tiles > static_cast<unsigned long long>(active_clusters_i8(bn, ks))) continue;
          const unsigned per = (num_kb + ks - 1) / ks;
          if (per < 4 || (num_kb + per - 1) / per != ks) continue;
        }
        if (env_ks > 1 && !pair && ks != static_cast<unsigned>(env_ks)) continue;
        const double waves = static_cast<double>((tiles * ks + groups - 1) / groups);
        const double busy = std::min(1.0, static_cast<double>(tiles * ks) / groups);
        const double fixed = pair ? 8.0 : (bn == 256 ? 12.5 : 8.7);
        const double per_kb = pair ? 0.29 : (bn == 256 ? 0.62 : 0.25 + 0.14 * std::max(0.0, busy - 0.5));
        const double kb = static_cast<double>((num_kb + ks - 1) / ks);
        const double t = waves * (fixed + kb * per_kb) + (ks > 1 ? 0.3 * ks : 0.0);
        if (best.bn == 0 || t < best_t) {
          best_t = t;
          best = {pair != 0, bn, ks};
        }
      }
    }
  }
  if (best.bn == 0) best = {force_pair == 1, force_pair == 1 ? 256 : 128, 1};
  return best;
}

// Time model behind the tile choice, in microseconds, fitted to measurements on B200
// (graph-replayed launches over rotating operands).  A CTA spends a fixed cost (launch,
// prologue, first loads, and an epilogue that grows with the tile width) plus its k-blocks times
// a per-k-block cost that is the larger of the MMA time of the tile and the pipeline round trip
// divided by the stages that fit.  The grid runs in waves.  A K split over a cluster adds the
// hand-off of (ks - 1) partial tiles to rank 0 and their summation.
double per_kblock_us(bool pair, int bn) {
  if (pair) return bn == 256 ? 1.24 : (bn == 128 ? 0.95 : 0.9);
  return bn == 256 ? 1.48 : (bn == 128 ? 0.71 : 0.64);
}
double fixed_us(bool pair, int bn) {
  if (pair) return 11.0;
  return bn == 256 ? 12.5 : (bn == 128 ? 7.2 : 5.5);
}
double cluster_k_us(unsigned ks, int bn) { return ks > 1 ? 0.3 + 1.0 * ks + 0.02 * (bn - 64) : 0.0; }

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::atoi(v) : fallback;
}

}  // namespace

void set_test_flag_wait(unsigned long long timeout_ns, unsigned expect_extra) {
  g_flag_timeout_ns.store(timeout_ns, std::memory_order_relaxed);
  g_flag_expect_extra.store(expect_extra, std::memory_order_relaxed);
}

bool encode_tmap_f32(void* map, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle_mode) {
  EncodeFn fn = encode_fn();
  if (!fn || rank < 1 || rank > 5) return false;
  cuuint64_t d[5];
  cuuint64_t st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) st[i] = strides_bytes[i];
  }
  const CUtensorMapSwizzle sw =
      swizzle_mode == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  return fn(static_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank,
            const_cast<void*>(base), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int umma_sm_budget(int sm_count, unsigned max_ctas) {
  int n = sm_count;
  if (max_ctas && static_cast<int>(max_ctas) < n) n = static_cast<int>(max_ctas);
  n &= ~1;  // whole CTA pairs
  return n < 2 ? 2 : n;
}

bool stream_k_scratch_ok(const SgemmArgs& a, int sm_count) {
  return a.workspace && (reinterpret_cast<uintptr_t>(a.workspace) & 255u) == 0 &&
         a.workspace_bytes >= umma_stream_k_workspace(sm_count);
}

size_t umma_stream_k_workspace(int sm_count) {
  // flags + one 128 x 256 fp32 partial tile per SM: enough for every tile shape
  return kStreamKFlagBytes + static_cast<size_t>(sm_count) * 128 * 256 * 4;
}

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

UmmaPlan umma_plan(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count,
                   int elem_bytes, int force_pair, bool allow_cluster_k, bool allow_stream_k) {
  UmmaPlan best = {false, 0, 1, 1};
  double best_time = 0;
  const unsigned num_kb = (K + 128 / elem_bytes - 1) / (128 / elem_bytes);
  for (int pair = 0; pair <= 1; ++pair) {
    if (force_pair >= 0 && pair != force_pair) continue;
    const int tile_m = pair ? 256 : 128;
    const int groups = pair ? sm_count / 2 : sm_count;
    if (groups < 1) continue;
    for (int bn : {256, 128, 64}) {
      // a CTA stages BN (BN/2 in a pair) columns of B: 128 bytes at least
      if ((pair ? bn / 2 : bn) * elem_bytes < 128) continue;
      if (bn > 64 && static_cast<unsigned>(bn) >= 2 * N) continue;  // mostly padding
      const unsigned long long tiles = static_cast<unsigned long long>((M + tile_m - 1) / tile_m) *
                                       ((N + bn - 1) / bn) * batch;
      if (pair && force_pair < 0) {
        // Measured: CTA pairs only win with full-width tiles and enough of them to occupy
        // most pairs; on smaller problems the extra cluster hops per k-block cost more than
        // the halved B traffic saves (1024x768x768: 32 us in pairs, 23 us single).
        if (bn != 256 || tiles * 5 < static_cast<unsigned long long>(groups) * 3) continue;
      }
      for (unsigned ks = 1; ks <= 4; ++ks) {
        if (ks > 1) {
          // K split over a cluster of single CTAs: one co-resident cluster per tile,
          // >= 4 k-blocks per rank
          if (!allow_cluster_k || pair) break;
          if (tiles > static_cast<unsigned long long>(active_clusters_fp32(bn, ks))) continue;
          const unsigned per = (num_kb + ks - 1) / ks;
          if (per < 4 || (num_kb + per - 1) / per != ks) continue;  // no empty rank
          // the other ranks' partial tiles (128 x bn fp32 each) must fit rank 0's stage buffers
          if ((ks - 1) * 128u * bn * 4u > 192u * 1024u) continue;
        }
        const unsigned long long units = tiles * ks;
        double waves = static_cast<double>((units + groups - 1) / groups);
        double extra = cluster_k_us(ks, bn);
        unsigned sk_tiles, sk_per;
        if (allow_stream_k && ks == 1 &&
            stream_k_split(tiles, static_cast<unsigned>(groups), num_kb, 4, &sk_tiles, &sk_per)) {
          // the ragged last wave is shared by k-block: fractional waves, plus the hand-off
          waves = static_cast<double>(tiles) / groups;
          extra = 4.0;
        }
        const double kb = static_cast<double>((num_kb + ks - 1) / ks);
        const double t =
            waves * (fixed_us(pair != 0, bn) + kb * per_kblock_us(pair != 0, bn)) + extra;
        if (best.bn == 0 || t < best_time) {
          best_time = t;
          best.pair = pair != 0;
          best.bn = bn;
          best.cluster_k = ks;
          best.global_k = 1;
        }
      }
      // K shared by consecutive CTAs through the scratch: any split that fits the SMs, at a
      // higher fixed price than the cluster form (flag reset, partial tiles through L2, the
      // gather; measured 8-11 us) -- pays for long K on few tiles (1024x3072x768: 48 -> 41 us).
      if (allow_stream_k && allow_cluster_k && !pair) {
        for (unsigned gk = 2; gk <= 6; ++gk) {
          if (tiles * gk > static_cast<unsigned long long>(sm_count)) break;
          const unsigned per = (num_kb + gk - 1) / gk;
          if (per < 4) break;
          const double t = fixed_us(false, bn) + per * per_kblock_us(false, bn) +
                           (bn == 64 ? 8.5 : (bn == 128 ? 10.5 : 13.0));
          if (t < best_time) {
            best_time = t;
            best.pair = false;
            best.bn = bn;
            best.cluster_k = 1;
            best.global_k = gk;
          }
        }
      }
    }
  }
  if (best.bn == 0) {  // nothing admissible (e.g. tiny N): widest legal tile
    best.pair = force_pair == 1;
    best.bn = (best.pair ? 256 : 128) / elem_bytes;
    if (best.bn < 64) best.bn = 64;
    best.cluster_k = 1;
    best.global_k = 1;
  }
  return best;
}

size_t bf16_staging_bytes(unsigned M, unsigned N, unsigned K, unsigned batch, unsigned strideA,
                          unsigned strideB) {
  const size_t na = static_cast<size_t>((batch > 1 && strideA) ? batch : 1) * M * K;
  const size_t nb = static_cast<size_t>((batch > 1 && strideB) ? batch : 1) * K * N;
  return ((na * 2 + 255) / 256 + (nb * 2 + 255) / 256) * 256;
}

bool umma_sgemm_supported(const SgemmArgs& a) {
  // TMA wants 16-byte aligned bases and row pitches; the epilogue stores float4.
  if (a.K % 4 != 0 || a.N % 4 != 0) return false;
  if (!aligned16(a.A) || !aligned16(a.B) || !aligned16(a.C)) return false;
  if (a.bias && !aligned16(a.bias)) return false;
  if (a.batch > 1) {
    if (a.strideA % 4 != 0 || a.strideB % 4 != 0 || a.strideC % 4 != 0) return false;
    // A non-zero batch stride must be the dense one: the tensor map describes
    // whole matrices laid end to end.
    if (a.strideA && a.strideA < a.M * a.K) return false;
    if (a.strideB && a.strideB < a.K * a.N) return false;
  }
  return true;
}

int umma_sgemm(const SgemmArgs& a, bool pair) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  if (di->cc_major != 10) return TFCCB200_EUNSUPPORTED;
  if (!umma_sgemm_supported(a)) return TFCCB200_EALIGN;

  const bool a_batched = a.batch > 1 && a.strideA != 0;
  const bool b_batched = a.batch > 1 && a.strideB != 0;
  static const int env_cluster_k = env_int("TFCCB200_CLUSTER_K", -1);  // -1: planned; 1: off
  const bool fp32_split = a.precision == TFCCB200_PRECISION_FP32;
  const int sm_avail = umma_sm_budget(di->sm_count, a.max_ctas);
  const UmmaPlan plan =
      umma_plan(a.M, a.N, a.K, a.batch, sm_avail,
                a.precision == TFCCB200_PRECISION_BF16 ? 2 : 4, pair ? 1 : 0,
                fp32_split && !pair && env_cluster_k != 1,
                fp32_split && stream_k_scratch_ok(a, sm_avail));
  UmmaPlan tuned = plan;
  static const int env_bn = env_int("TFCCB200_FORCE_BN", 0);  // tuning knobs, read once
  if (env_bn == 64 || env_bn == 128 || env_bn == 256) tuned.bn = env_bn;
  if (env_cluster_k > 1) tuned.cluster_k = static_cast<unsigned>(env_cluster_k);
  const int bn = tuned.bn;

  if (a.precision == TFCCB200_PRECISION_BF16) {
    // Opt-in low precision: a pre-pass rounds both operands to bfloat16 in the caller's
    // scratch, then the bfloat16 tensor-core kernel runs on the copies (fp32 accumulate/out).
    if (a.K % 8 != 0 || a.N % 8 != 0) return TFCCB200_EALIGN;
    const size_t na = static_cast<size_t>(a_batched ? a.batch : 1) * a.M * a.K;
    const size_t nb = static_cast<size_t>(b_batched ? a.batch : 1) * a.K * a.N;
    const size_t a_bytes = (na * 2 + 255) / 256 * 256;
    if (!a.workspace || (reinterpret_cast<uintptr_t>(a.workspace) & 255u) ||
        a.workspace_bytes < bf16_staging_bytes(a.M, a.N, a.K, a.batch, a.strideA, a.strideB))
      return TFCCB200_EWORKSPACE;
    void* a16 = a.workspace;
    void* b16 = static_cast<char*>(a.workspace) + a_bytes;
    int st = convert_f32_to_bf16(a.stream, a.A, a16, na);
    if (st != TFCCB200_OK) return st;
    st = convert_f32_to_bf16(a.stream, a.B, b16, nb);
    if (st != TFCCB200_OK) return st;
    CUtensorMap ta16, tb16;
    if (!make_tmap(&ta16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a16, a.K, a.M,
                   a_batched ? a.batch : 1, a.strideA, 128, CU_TENSOR_MAP_SWIZZLE_128B))
      return TFCCB200_EINVAL;
    if (!make_tmap(&tb16, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b16, a.N, a.K,
                   b_batched ? a.batch : 1, a.strideB, 64, CU_TENSOR_MAP_SWIZZLE_128B))
      return TFCCB200_EINVAL;
    UmmaGemmParams q = {};
    q.num_dst = a.num_dst ? a.num_dst : 1;
    if (q.num_dst > kMaxDestinations) return TFCCB200_EINVAL;
    q.dst[0] = a.C;
    for (unsigned d = 0; d < a.num_dst; ++d) q.dst[d] = a.dst[d];
    q.mc_dst = a.mc_dst;
    q.ldc = a.ldc ? a.ldc : a.N;
    q.col_offset = a.col_offset;
    q.bias = a.bias;
    q.activation = a.activation;
    q.M = a.M; q.N = a.N; q.K = a.K; q.batch = a.batch;
    q.strideC = a.strideC;
    q.a_batched = a_batched; q.b_batched = b_batched;
    q.status = a.status;
    q.timeout_ns = kDefaultTimeoutNs;
    q.flag_timeout_ns = kDefaultTimeoutNs;
    constexpr auto H = ptx::MmaKind::BF16;
    const int sms16 = sm_avail;
    if (!pair) {
      if (bn == 256) return launch<H, false, 1, 256, 4>(a.stream, ta16, tb16, q, sms16);
      if (bn == 128) return launch<H, false, 1, 128, 6>(a.stream, ta16, tb16, q, sms16);
      return launch<H, false, 1, 64, 8>(a.stream, ta16, tb16, q, sms16);
    }
    if (bn == 256) return launch<H, false, 2, 256, 6>(a.stream, ta16, tb16, q, sms16);
    return launch<H, false, 2, 128, 8>(a.stream, ta16, tb16, q, sms16);
  }

  CUtensorMap ta, tb;
  if (!make_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.A, a.K, a.M, a_batched ? a.batch : 1,
                 a.strideA, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return TFCCB200_EINVAL;
  // B is the MN-major operand: 32-bit data needs the 32-byte-unit flavour of the swizzle.
  if (!make_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.B, a.N, a.K, b_batched ? a.batch : 1,
                 a.strideB, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B))
    return TFCCB200_EINVAL;

  UmmaGemmParams p = {};
  p.num_dst = a.num_dst ? a.num_dst : 1;
  if (p.num_dst > kMaxDestinations) return TFCCB200_EINVAL;
  p.dst[0] = a.C;
  for (unsigned d = 0; d < a.num_dst; ++d) p.dst[d] = a.dst[d];
  p.mc_dst = a.mc_dst;
  p.ldc = a.ldc ? a.ldc : a.N;
  p.col_offset = a.col_offset;
  p.bias = a.bias;
  p.activation = a.activation;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.strideC = a.strideC;
  p.a_batched = a_batched; p.b_batched = b_batched;
  // Tuning knobs, read once.  TFCCB200_WRITE_HEAD=1 makes the converters store the
  // truncated TF32 head back over the raw tile; by default the raw fp32 tile is the
  // head operand, because the tensor core ignores the 13 low mantissa bits itself
  // (both settings give bit-identical products; the default saves shared-memory
  // stores).  TFCCB200_KB_PER_CHUNK = k-blocks (32 elements of K each) a
  // tensor-memory accumulator sums before its partial is promoted to registers.
  static const int env_write_head = env_int("TFCCB200_WRITE_HEAD", 0);
  static const int env_kb_per_chunk = env_int("TFCCB200_KB_PER_CHUNK", 4);
  p.write_head = env_write_head ? 1 : 0;
  p.kb_per_chunk = env_kb_per_chunk > 0 ? env_kb_per_chunk : 4;
  if (fp32_split && a.workspace && (reinterpret_cast<uintptr_t>(a.workspace) & 255u) == 0 &&
      a.workspace_bytes > kStreamKFlagBytes) {
    p.sk_flags = static_cast<unsigned*>(a.workspace);
    p.sk_partials = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kStreamKFlagBytes);
    p.sk_capacity = a.workspace_bytes - kStreamKFlagBytes;
  }
  p.cluster_k = (fp32_split && !pair) ? tuned.cluster_k : 1;
  static const int env_global_k = env_int("TFCCB200_GLOBAL_K", -1);  // -1: planned; 1: off
  p.global_k = (fp32_split && !pair) ? tuned.global_k : 1;
  if (env_global_k >= 1) p.global_k = (fp32_split && !pair) ? env_global_k : 1;
  if (p.global_k > 1) p.cluster_k = 1;
  p.status = a.status;
  p.timeout_ns = kDefaultTimeoutNs;
  const unsigned long long flag_ns = g_flag_timeout_ns.load(std::memory_order_relaxed);
  p.flag_timeout_ns = flag_ns ? flag_ns : kDefaultTimeoutNs;
  p.flag_expect_extra = g_flag_expect_extra.load(std::memory_order_relaxed);

  constexpr auto T = ptx::MmaKind::TF32;
  const bool split = a.precision == TFCCB200_PRECISION_FP32;
  const int sms = sm_avail;

  // With fewer than two tiles per CTA little or nothing overlaps the epilogue, and an erf per
  // element on the 256 epilogue threads of an SM costs more there (measured +12..15 us on
  // 1024x768x3072) than one more pass over C by a full grid (about 6 us).  The activation is
  // then applied in place by the element-wise kernel; same formula, same bits.
  const unsigned long long tiles = static_cast<unsigned long long>((a.M + (pair ? 256 : 128) - 1) /
                                                                   (pair ? 256 : 128)) *
                                   ((a.N + bn - 1) / bn) * a.batch;
  const bool unfuse = a.activation != TFCCB200_ACT_NONE && a.num_dst <= 1 && a.col_offset == 0 &&
                      (a.ldc == 0 || a.ldc == a.N) &&
                      (a.batch == 1 || a.strideC == static_cast<unsigned long long>(a.M) * a.N) &&
                      tiles < 2ull * static_cast<unsigned long long>(pair ? sms / 2 : sms);
  if (unfuse) p.activation = TFCCB200_ACT_NONE;
  auto finish = [&](int st) {
    if (st != TFCCB200_OK || !unfuse) return st;
    return gelu_f32(a.stream, a.C, static_cast<size_t>(a.batch) * a.M * a.N, a.C);
  };
  if (split) {
    if (!pair) {
      if (bn == 256) return finish(launch<T, true, 1, 256, 2>(a.stream, ta, tb, p, sms));
      if (bn == 128) return finish(launch<T, true, 1, 128, 4>(a.stream, ta, tb, p, sms));
      return finish(launch<T, true, 1, 64, 6>(a.stream, ta, tb, p, sms));
    }
    if (bn == 256) return finish(launch<T, true, 2, 256, 3>(a.stream, ta, tb, p, sms));
    if (bn == 128) return finish(launch<T, true, 2, 128, 5>(a.stream, ta, tb, p, sms));
    return finish(launch<T, true, 2, 64, 6>(a.stream, ta, tb, p, sms));
  }
  if (!pair) {
    if (bn == 256) return finish(launch<T, false, 1, 256, 4>(a.stream, ta, tb, p, sms));
    if (bn == 128) return finish(launch<T, false, 1, 128, 6>(a.stream, ta, tb, p, sms));
    return finish(launch<T, false, 1, 64, 8>(a.stream, ta, tb, p, sms));
  }
  if (bn == 256) return finish(launch<T, false, 2, 256, 6>(a.stream, ta, tb, p, sms));
  if (bn == 128) return finish(launch<T, false, 2, 128, 8>(a.stream, ta, tb, p, sms));
  return finish(launch<T, false, 2, 64, 8>(a.stream, ta, tb, p, sms));
}

bool umma_qgemm_supported(const QgemmArgs& a) {
  if (a.K % 16 != 0 || a.N % 16 != 0) return false;
  if (!aligned16(a.A) || !aligned16(a.B) || !aligned16(a.C) || !aligned16(a.rsB)) return false;
  if (a.batch > 1) {
    if (a.strideA % 16 != 0 || a.strideB % 16 != 0 || a.strideC % 4 != 0 ||
        a.strideRsB % 4 != 0)
      return false;
    if (a.strideA && a.strideA < a.M * a.K) return false;
    if (a.strideB && a.strideB < a.K * a.N) return false;
  }
  return true;
}

bool umma_qgemm_prefers_pair(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count) {
  return plan_i8(M, N, K, batch, sm_count, -1).pair;
}

int umma_qgemm(const QgemmArgs& a, bool pair) {
  cudaError_t ce;
  const DeviceInfo* di = current_device_info(&ce);
  if (!di) return static_cast<int>(ce);
  if (di->cc_major != 10) return TFCCB200_EUNSUPPORTED;
  if (!umma_qgemm_supported(a)) return TFCCB200_EALIGN;

  const bool a_batched = a.batch > 1 && a.strideA != 0;
  const bool b_batched = a.batch > 1 && a.strideB != 0;
  const I8Plan plan = plan_i8(a.M, a.N, a.K, a.batch, di->sm_count, pair ? 1 : 0);
  const int bn = plan.bn;

  CUtensorMap ta, tb;
  if (!make_tmap(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.A, a.K, a.M, a_batched ? a.batch : 1,
                 a.strideA, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return TFCCB200_EINVAL;
  if (!make_tmap(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.B, a.N, a.K, b_batched ? a.batch : 1,
                 a.strideB, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return TFCCB200_EINVAL;

  UmmaGemmParams p = {};
  p.num_dst = a.num_dst ? a.num_dst : 1;
  if (p.num_dst > kMaxDestinations) return TFCCB200_EINVAL;
  p.dst[0] = a.C;
  for (unsigned d = 0; d < a.num_dst; ++d) p.dst[d] = a.dst[d];
  p.mc_dst = a.mc_dst;
  p.ldc = a.ldc ? a.ldc : a.N;
  p.col_offset = a.col_offset;
  p.rsA = a.rsA; p.rsB = a.rsB;
  p.offA = a.offA; p.offB = a.offB;
  p.kterm = static_cast<int32_t>(static_cast<uint32_t>(a.offA) * static_cast<uint32_t>(a.offB) *
                                 a.K);
  p.q_offsets = a.dev_offsets;
  // the K split over a cluster stores from registers into one matrix only
  p.cluster_k = (!pair && a.num_dst <= 1 && !a.mc_dst) ? plan.cluster_k : 1;
  p.strideRsA = a.strideRsA; p.strideRsB = a.strideRsB;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.strideC = a.strideC;
  p.a_batched = a_batched; p.b_batched = b_batched;
  p.status = a.status;
  p.timeout_ns = kDefaultTimeoutNs;
  p.flag_timeout_ns = kDefaultTimeoutNs;

  constexpr auto I = ptx::MmaKind::I8;
  const int sms = di->sm_count;
  if (!pair) {
    if (bn == 256) return launch<I, false, 1, 256, 4>(a.stream, ta, tb, p, sms);
    return launch<I, false, 1, 128, 6>(a.stream, ta, tb, p, sms);
  }
  return launch<I, false, 2, 256, 6>(a.stream, ta, tb, p, sms);
}

}  // namespace tfccb200
