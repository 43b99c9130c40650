// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[b] = A[b] . B[b]       A: [M,K] row-major (K-major operand)
//                            B: [K,N] row-major (MN-major operand, no transpose pass)
//
// Two element kinds share the kernel:
//   * TF32 on fp32 data.  With kSplit the fp32 product is rebuilt from three
//     MMAs per k-step: every raw fp32 tile that TMA brings in is split in
//     shared memory into a TF32 head (top 19 bits, truncation) and a TF32 tail
//     (x - head, rounded to TF32); head*head + head*tail + tail*head is
//     accumulated in fp32 in tensor memory.  HBM traffic stays that of one
//     fp32 GEMM.
//   * I8: u8 x s8 -> s32, exact, with the zero-point correction applied while
//     the accumulator leaves tensor memory.
//   * BF16 on operands that a pre-pass rounded from fp32 to bfloat16 (opt-in
//     low-precision mode); fp32 accumulation and fp32 output.
//
// Work layout per CTA (kCtaGroup == 1) or per CTA pair (kCtaGroup == 2):
//   tile        128*kCtaGroup rows x BN columns, accumulator in TMEM, two
//               accumulator buffers so the epilogue of tile i overlaps the
//               mainloop of tile i+1
//   k-block     128 bytes of K per A row (32 fp32 / 128 int8) = 4 MMA k-steps
//   stage       A: 128 rows x 128 B, 128B-swizzled (K-major canonical layout)
//               B: (BN_local*elem/128) boxes of [k-block rows x 128 B], MN-major
//                  canonical layout: 128B swizzle of 16-byte units for int8, of
//                  32-byte units for fp32 (the TMA mode SWIZZLE_128B_ATOM_32B)
//               (+ tail tiles of the same shape for the TF32 tails when kSplit:
//                one per stage for CTA pairs, a ring of two of their own for single
//                CTAs, which leaves room for a deeper ring of raw stages)
// Warps without kSplit: 0 = TMA producer, 1 = MMA issuer and TMEM owner,
// 2..5 = epilogue (one TMEM lane quarter each).
//
// With kSplit the tensor core's fp32 accumulator is not trusted over a long K:
// it narrows every partial sum without round-to-nearest, which biases the
// result by an amount that grows linearly with K (measured 7e-9 * K normwise).
// So K is cut into chunks of `kb_per_chunk` k-blocks; each chunk is accumulated
// in one of the two TMEM buffers starting from zero, and eight epilogue warps
// add the finished chunk into fp32 registers with round-to-nearest adds while
// the MMA issuer fills the other buffer.  The register budget is rebalanced
// with setmaxnreg: warpgroup 0 = {TMA, MMA, 2 idle warps}, warpgroups 1-2 =
// epilogue (hold a 128 x BN fp32 running sum), warpgroup 3 = converters.
//
// How the tiles of a problem reach the CTAs (kSplit; see UmmaGemmParams):
//   * by default every CTA / pair walks whole tiles with a stride of the grid;
//   * cluster_k > 1: fewer tiles than SMs -- a thread-block cluster shares one tile's
//     k-blocks and reduces through distributed shared memory;
//   * global_k > 1: the same without a cluster, partial tiles through scratch in L2;
//   * sk_tiles > 0: more tiles than the grid but a ragged last wave -- the last one to two
//     waves are cut into equal k-block ranges, a cut tile being started by one group and
//     finished (same summation order, same bits) by the next.
// The kernel is launched with programmatic stream serialisation: everything up to
// pdl_wait() (barriers, tensor memory, descriptor prefetch) may overlap the previous
// kernel's tail.
//
// Every wait on an mbarrier is bounded: after `timeout_ns` the waiter raises a
// CTA-wide abort flag, ORs a bit into *status and carries on without the data,
// so the kernel always runs to its end, frees its tensor memory and returns.
#pragma once

#include "../../include/tfcc_b200.h"
#include "act.cuh"
#include "pdl.cuh"
#include "ptx.cuh"

namespace tfccb200 {

constexpr int kMaxDestinations = 8;

struct UmmaGemmParams {
  // Result destinations: the same tile is stored into each of them (one in the plain case;
  // one per GPU when column shards of C are pushed straight into every peer's full matrix).
  // float* (TF32) or int32_t* (I8); element (b, i, j) goes to
  // dst[d] + b*strideC + i*ldc + col_offset + j.
  void* dst[kMaxDestinations];
  unsigned num_dst;
  // When set, the tile goes out through this NVLink multicast address instead (one store
  // reaches the same offset of every GPU bound to it) and dst[] is not written
  void* mc_dst;
  unsigned long long ldc;  // row pitch of the destinations, in elements
  unsigned col_offset;     // first destination column of this problem's column 0
  const float* bias;       // [N] or nullptr (float kinds only)
  int activation;          // TFCCB200_ACT_*, applied after the bias (float kinds only)
  const int32_t* rsA;      // I8: row sums of A, [batch?][M]
  const int32_t* rsB;      // I8: column sums of B, [batch?][N]
  int32_t offA, offB;      // I8 zero-point offsets
  int32_t kterm;           // I8: offA*offB*K (wrapped)
  const int32_t* q_offsets;  // I8: when set, {offA, offB} are read from device memory instead
                             // (written by a prologue kernel from device-resident ranges)
  unsigned strideRsA, strideRsB;
  unsigned M, N, K, batch;
  unsigned long long strideC;  // elements between batch entries of C
  unsigned a_batched, b_batched;  // 0: operand shared by the whole batch
  unsigned tma_store;      // 1: the kernel's C tensor map is valid and tiles are stored through it
  unsigned tiles_m, tiles_n;      // tile grid of one batch entry
  unsigned write_head;     // kSplit: 1 = store the truncated head back (independent of how
                           // the tensor core narrows fp32), 0 = feed the raw fp32 as head
  unsigned kb_per_chunk;   // kSplit: k-blocks accumulated inside tensor memory before the
                           // partial sum is promoted to registers (>= 1)
  unsigned cluster_k;      // kSplit or I8, one CTA per tile only: >= 1.  With k > 1 a cluster of k
                           // CTAs shares one tile, each CTA taking a contiguous range of k-blocks.
                           // fp32: ranks 1.. hand their partial sums to rank 0 through its
                           // shared memory and rank 0 adds them in rank order (deterministic)
                           // before the store.  int8: every rank owns BN / k columns of the
                           // tile, receives the other ranks' int32 partial sums for them
                           // through its shared memory, adds (exact in any order) and stores.
                           // The grid must hold every tile at once.
  // kSplit only, sk_tiles > 0: the first sk_tiles tiles (between one and two per CTA / pair)
  // are shared out by k-block rather than by tile, so that a tile count that is not a
  // multiple of the grid leaves no SM idle in the last wave.  Group g takes k-blocks
  // [g, g+1) * sk_kb_per_group of those tiles laid end to end; a tile cut between groups g-1
  // and g is begun by g-1, whose fp32 partial sums travel through sk_partials (one tile slot
  // per CTA) guarded by sk_flags, and finished and stored by g.  The remaining tiles are
  // walked tile by tile as usual.  Cuts fall on chunk boundaries and the finisher continues
  // the running sum, so results are bit-identical to the unsplit order.
  unsigned sk_tiles;
  unsigned sk_kb_per_group;  // multiple of kb_per_chunk, >= k-blocks of one tile
  // kSplit, single CTAs, global_k > 1 (instead of the above): fewer tiles than SMs, so
  // global_k consecutive CTAs share one tile's k-blocks.  Ranks 1.. publish their sums like a
  // head piece; rank 0 adds them to its own in rank order (deterministic) and stores the tile.
  // Unlike cluster_k this needs no co-scheduled cluster, so any global_k that fits the SM
  // count works; the partial tiles cross L2 instead of distributed shared memory.
  unsigned global_k;
  float* sk_partials;        // [grid CTAs][128 x BN] fp32
  unsigned* sk_flags;        // [grid CTAs], zero before the launch
  unsigned long long sk_capacity;  // host only: bytes available behind sk_partials
  int* status;             // device int or nullptr
  unsigned long long timeout_ns;
  // Waits on the scratch counters above have their own limit and may be told to expect more
  // arrivals than any launch delivers: the test hook tfccb200_test_flag_wait() uses the two to
  // make such a wait run out at once, which drives the give-up path (status word, abort flag,
  // orderly teardown) without anything hanging.  Normal launches: timeout_ns and 0.
  unsigned long long flag_timeout_ns;
  unsigned flag_expect_extra;
};

// One stretch of k-blocks of one tile, as every role of a CTA walks them.
struct UmmaSegment {
  unsigned tile, kb_lo, kb_hi;
  unsigned mode;  // 0: whole tile (or this rank's share of it); kSegHead; kSegTail
};
constexpr unsigned kSegHead = 1;  // k-blocks [0, kb_hi): partial sums go to the next group
constexpr unsigned kSegTail = 2;  // k-blocks [kb_lo, end): continues the previous group's sums
constexpr unsigned kSegGather = 3;  // rank 0 of a global K split: adds the other ranks' sums
constexpr int kMaxSkSegments = 4;

template <ptx::MmaKind kKind, bool kSplit, int kCtaGroup, int BN, int kStages>
struct UmmaGemmConfig {
  static constexpr int kElemBytes =
      (kKind == ptx::MmaKind::TF32) ? 4 : (kKind == ptx::MmaKind::BF16 ? 2 : 1);
  static constexpr int kBM = 128;                      // rows per CTA
  static constexpr int kTileM = kBM * kCtaGroup;       // rows per MMA
  static constexpr int kBK = 128 / kElemBytes;         // elements of K per k-block
  static constexpr int kUmmaK = 32 / kElemBytes;       // elements of K per MMA
  static constexpr int kKSteps = 4;
  static constexpr int kBNLocal = BN / kCtaGroup;      // B columns staged by one CTA
  static constexpr int kBChunks = kBNLocal * kElemBytes / 128;  // 128-byte-wide boxes of B
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBChunkBytes = kBK * 128;
  static constexpr int kBBytes = kBChunks * kBChunkBytes;
  static constexpr int kRawBytes = kABytes + kBBytes;
  static constexpr int kStageBytes = kRawBytes;  // one slot of the ring TMA fills
  // kSplit: the low-order (tail) copies live in a ring of their own.  A raw tile is in flight
  // from the moment its TMA is issued, a tail tile only from its conversion to the end of
  // its MMAs, so a few tail slots serve any number of raw slots and the bytes saved buy a
  // deeper load pipeline.  A tail slot frees when its MMAs retire and the next use needs a
  // conversion plus two barrier hops before its MMAs can be queued: with CTA pairs (32 KB to
  // convert per k-block, MMAs of about a microsecond) two slots left the tensor pipe waiting
  // (measured 6 % slower than three), single CTAs do well with two.
  static constexpr int kTailStages = kSplit ? (kCtaGroup == 2 ? 3 : 2) : 0;
  static constexpr int kRingBytes = (kStages + kTailStages) * kRawBytes;
  static constexpr int kBKStepBytes = kUmmaK * 128;    // B advance per MMA k-step
  // MN-major B: 8-bit data uses the plain 128-byte swizzle (atoms of 8 k-rows, 1024 B apart);
  // 32-bit data must use the 128-byte swizzle with 32-byte units (atoms of 4 k-rows, 512 B).
  static constexpr uint32_t kBLayout =
      (kKind == ptx::MmaKind::TF32) ? ptx::kLayoutSw128Base32 : ptx::kLayoutSw128;
  static constexpr uint32_t kBSbo = (kKind == ptx::MmaKind::TF32) ? 512 : 1024;
  static constexpr int kNumConvertWarps = kSplit ? 4 : 0;
  static constexpr int kNumEpilogueWarps = kSplit ? 8 : 4;
  static constexpr int kFirstEpilogueWarp = kSplit ? 4 : 2;  // kSplit: warps 2,3 idle (warpgroup fill)
  static constexpr int kFirstConvertWarp = kFirstEpilogueWarp + kNumEpilogueWarps;
  static constexpr int kThreads = 32 * (kFirstConvertWarp + kNumConvertWarps);
  static constexpr int kEpiCols = kSplit ? BN / 2 : BN;  // accumulator columns owned by one thread
  // setmaxnreg targets (kSplit): 128*48 + 256*208 + 128*48 = 65536 registers
  static constexpr int kRegsControl = 48, kRegsEpilogue = 208, kRegsConvert = 48;
  static constexpr int kTmemCols = (2 * BN <= 32) ? 32 : 2 * BN;  // power of two by construction
  // Each epilogue warp transposes 32x32 blocks through 4 KB of shared memory so that its
  // global stores cover whole 128-byte lines (and peers' memory is written in full lines).
  static constexpr int kEpiStageBytes = 4096;
  static constexpr int kEpiStagingBytes = kNumEpilogueWarps * kEpiStageBytes;
  static constexpr int kBarrierBytes =
      256 + 16 * kMaxSkSegments + 16 + 128;  // + segment table, store target
  static constexpr int kSmemBytes =
      kRingBytes + kEpiStagingBytes + kBarrierBytes + 1024;  // +align slack
  static constexpr uint32_t kIdesc =
      (kKind == ptx::MmaKind::TF32)
          ? ptx::make_idesc(1u, 2u, 2u, 0u, 1u, static_cast<uint32_t>(kTileM), BN)
          : (kKind == ptx::MmaKind::BF16)
                ? ptx::make_idesc(1u, 1u, 1u, 0u, 1u, static_cast<uint32_t>(kTileM), BN)
                : ptx::make_idesc(2u, 0u, 1u, 0u, 1u, static_cast<uint32_t>(kTileM), BN);
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "MMA N out of range");
  static_assert((BN & (BN - 1)) == 0, "BN must be a power of two (TMEM allocation)");
  static_assert(kBNLocal * kElemBytes % 128 == 0, "B tile must be whole 128-byte boxes");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  static_assert(!kSplit || kEpiCols % 16 == 0, "epilogue reads 16 columns at a time");
  static_assert(!kSplit || (kFirstEpilogueWarp == 4 && kFirstConvertWarp == 12 && kThreads == 512),
                "setmaxnreg assumes warpgroups {control, epilogue, epilogue, convert}");
};

struct UmmaCtl {
  volatile uint32_t* abort_flag;  // shared
  int* status;                    // global or nullptr
  unsigned long long timeout_ns;
  unsigned long long flag_timeout_ns;  // limit of bounded_flag_wait
};

template <bool kClusterAcquire>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, int bit,
                                             const UmmaCtl& ctl) {
  auto probe = [&]() {
    if constexpr (kClusterAcquire) return ptx::mbar_try_wait_cluster(bar, parity);
    else return ptx::mbar_try_wait(bar, parity);
  };
  if (probe()) return true;
  if (*ctl.abort_flag) return false;
  uint64_t start = 0;
  uint32_t spins = 0;
  while (true) {
    if (probe()) return true;
    if ((++spins & 0xFF) == 0) {
      if (*ctl.abort_flag) return false;
      uint64_t now = ptx::globaltimer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > ctl.timeout_ns) {
        *ctl.abort_flag = 1;
        if (ctl.status) atomicOr(ctl.status, bit);
        return false;
      }
    }
  }
}

// Wait (bounded like the barrier waits) until a counter in global memory that other CTAs of
// the same grid increment reaches `expect`; an acquire on success.
__device__ __forceinline__ bool bounded_flag_wait(const unsigned* flag, unsigned expect, int bit,
                                                  const UmmaCtl& ctl) {
  uint64_t start = 0;
  uint32_t spins = 0;
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= expect) return true;
    if ((++spins & 0x3F) == 0) {
      if (*ctl.abort_flag) return false;
      uint64_t now = ptx::globaltimer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > ctl.flag_timeout_ns) {
        *ctl.abort_flag = 1;
        if (ctl.status) atomicOr(ctl.status, bit);
        return false;
      }
    }
    __nanosleep(64);
  }
}

// A thread's share of a partial-sum tile: kCount float4, 512 bytes apart (one base register,
// immediate offsets, L2 only).
template <int kCount, int V = 0>
__device__ __forceinline__ void sk_load_partial(float* sum, const float4* src) {
  if constexpr (V < kCount) {
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4 + %5];"
                 : "=f"(sum[4 * V]), "=f"(sum[4 * V + 1]), "=f"(sum[4 * V + 2]), "=f"(sum[4 * V + 3])
                 : "l"(src), "n"(V * 512)
                 : "memory");
    sk_load_partial<kCount, V + 1>(sum, src);
  }
}
template <int kCount, int V = 0>
__device__ __forceinline__ void sk_add_partial(float* sum, const float4* src) {
  if constexpr (V < kCount) {
    float a, b, c, d;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4 + %5];"
                 : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
                 : "l"(src), "n"(V * 512)
                 : "memory");
    sum[4 * V] += a; sum[4 * V + 1] += b; sum[4 * V + 2] += c; sum[4 * V + 3] += d;
    sk_add_partial<kCount, V + 1>(sum, src);
  }
}
template <int kCount, int V = 0>
__device__ __forceinline__ void sk_store_partial(const float* sum, float4* dst) {
  if constexpr (V < kCount) {
    asm volatile("st.global.cg.v4.f32 [%0 + %1], {%2, %3, %4, %5};"
                 :
                 : "l"(dst), "n"(V * 512), "f"(sum[4 * V]), "f"(sum[4 * V + 1]),
                   "f"(sum[4 * V + 2]), "f"(sum[4 * V + 3])
                 : "memory");
    sk_store_partial<kCount, V + 1>(sum, dst);
  }
}

// ---- epilogue: 32x32 block of 32-bit results, one row per lane -> coalesced line stores ----
// Chunk q (4 values) of the lane's row goes to 16-byte slot q ^ (row & 7) of that row: both
// the row-wise writes and the transposed reads below are then free of bank conflicts.
__device__ __forceinline__ void epi_stage_chunk(uint32_t* stage, uint32_t lane, int q, uint4 v) {
  *reinterpret_cast<uint4*>(stage + lane * 32 + ((q ^ (lane & 7)) << 2)) = v;
}

// Where a tile's rows go.  The kernel parameters live in constant memory; read through a
// reference inside a loop that also stores to global memory they are reloaded after every store
// (the compiler cannot rule out that the store changed them) at global-load latency each time --
// measured 0.24 us per store instruction, 4 us per tile.  So thread 0 copies what the store
// loops need into shared memory once per launch; reloads from there cost a few cycles and no
// registers are tied up while the running sums fill the register file.
struct EpiTarget {
  uint32_t* dst[kMaxDestinations];
  uint32_t* mc;  // multicast alias or nullptr
  unsigned long long ldc;
  unsigned num_dst;
  unsigned col_offset;
  unsigned M, N;
  int activation;
  const float* bias;
  unsigned tma_store;  // tiles leave through the C tensor map (single destination)
};

__device__ __forceinline__ void fill_epi_target(EpiTarget* t, const UmmaGemmParams& p) {
  for (unsigned d = 0; d < kMaxDestinations; ++d)
    t->dst[d] = d < p.num_dst ? static_cast<uint32_t*>(p.dst[d]) : nullptr;
  t->mc = static_cast<uint32_t*>(p.mc_dst);
  t->ldc = p.ldc;
  t->num_dst = p.num_dst;
  t->col_offset = p.col_offset;
  t->M = p.M;
  t->N = p.N;
  t->activation = p.activation;
  t->bias = p.bias;
  t->tma_store = p.tma_store;
}

// After all 8 chunks of every lane are staged: lane l takes column chunk l%8 of rows
// i*4 + l/8, adds the per-column term, and stores to every destination.  A warp instruction
// writes 4 rows x 128 contiguous bytes.
template <bool kIsFloat>
__device__ __forceinline__ void epi_flush_block(uint32_t* stage, uint32_t lane, unsigned row0,
                                                unsigned col_blk, const EpiTarget& t,
                                                unsigned long long batch_off, uint4 col_term) {
  __syncwarp();
  const unsigned cq = lane & 7u;
  const unsigned col = col_blk + cq * 4;
  const bool col_ok = col < t.N;  // N is a multiple of 4 on this path: a chunk is all in or out
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const unsigned r = i * 4 + (lane >> 3);
    uint4 v = *reinterpret_cast<const uint4*>(stage + r * 32 + ((cq ^ (r & 7u)) << 2));
    if constexpr (kIsFloat) {
      v.x = __float_as_uint(__uint_as_float(v.x) + __uint_as_float(col_term.x));
      v.y = __float_as_uint(__uint_as_float(v.y) + __uint_as_float(col_term.y));
      v.z = __float_as_uint(__uint_as_float(v.z) + __uint_as_float(col_term.z));
      v.w = __float_as_uint(__uint_as_float(v.w) + __uint_as_float(col_term.w));
      if (t.activation != TFCCB200_ACT_NONE) {
        v.x = __float_as_uint(apply_activation(__uint_as_float(v.x), t.activation));
        v.y = __float_as_uint(apply_activation(__uint_as_float(v.y), t.activation));
        v.z = __float_as_uint(apply_activation(__uint_as_float(v.z), t.activation));
        v.w = __float_as_uint(apply_activation(__uint_as_float(v.w), t.activation));
      }
    } else {
      v.x += col_term.x; v.y += col_term.y; v.z += col_term.z; v.w += col_term.w;
    }
    const unsigned grow = row0 + r;
    if (grow < t.M && col_ok) {
      const unsigned long long off =
          batch_off + static_cast<unsigned long long>(grow) * t.ldc + t.col_offset + col;
      if (t.mc) {
        ptx::multimem_st_v4(t.mc + off, v);
      } else {
        for (unsigned d = 0; d < t.num_dst; ++d) *reinterpret_cast<uint4*>(t.dst[d] + off) = v;
      }
    }
  }
  __syncwarp();
}

// The same 32x32 block leaving through the tensor map of C instead: the staged block (already
// complete: bias, activation or zero-point terms applied in registers) is handed to the TMA
// unit by one lane as a [32 rows x 128 bytes] box; the unit clips rows and columns outside C.
// Plain st.global from the eight epilogue warps of a CTA proved to be latency-bound (about
// 0.24 us per store instruction per warp, 4 us for a 128-wide tile), which in the
// latency-bound shapes sits entirely on the critical path of the launch.
__device__ __forceinline__ void epi_tma_store_block(uint32_t* stage, uint32_t lane,
                                                    const CUtensorMap* tmap, unsigned col,
                                                    unsigned row0, unsigned batch) {
  ptx::fence_proxy_async_smem();  // the staged values -> visible to the async proxy
  __syncwarp();
  if (lane == 0) {
    ptx::tma_store_3d(tmap, ptx::smem_u32(stage), static_cast<int32_t>(col),
                      static_cast<int32_t>(row0), static_cast<int32_t>(batch));
    ptx::bulk_commit_group();
  }
}
// Before the stage is written again (and before the CTA leaves).
__device__ __forceinline__ void epi_tma_stage_free(uint32_t lane) {
  if (lane == 0) ptx::bulk_wait_read_all();
  __syncwarp();
}

// Tile order: groups of 8 tile-rows are walked column by column so that CTAs
// running at the same time share B panels and a small set of A panels in L2.
__device__ __forceinline__ void tile_coords(unsigned t, unsigned tiles_m, unsigned tiles_n,
                                            unsigned& b, unsigned& tm, unsigned& tn) {
  const unsigned per_batch = tiles_m * tiles_n;
  b = t / per_batch;
  unsigned r = t - b * per_batch;
  constexpr unsigned G = 8;
  unsigned group = r / (G * tiles_n);
  unsigned first_m = group * G;
  unsigned gsz = min(tiles_m - first_m, G);
  unsigned in_group = r - group * G * tiles_n;
  tm = first_m + in_group % gsz;
  tn = in_group / gsz;
}

template <ptx::MmaKind kKind, bool kSplit, int kCtaGroup, int BN, int kStages>
__global__ void __launch_bounds__(UmmaGemmConfig<kKind, kSplit, kCtaGroup, BN, kStages>::kThreads,
                                  1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                 const __grid_constant__ CUtensorMap tmapC, const UmmaGemmParams p) {
  using Cfg = UmmaGemmConfig<kKind, kSplit, kCtaGroup, BN, kStages>;
  extern __shared__ uint8_t smem_raw[];
  pdl_release();  // the next kernel in the stream may begin its preamble

  // ---- carve shared memory (stage buffers need 1024-byte alignment for the swizzle) ----
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  uint8_t* epi_stage_gen = smem_gen + Cfg::kRingBytes;
  const uint32_t bar_base = smem_base + Cfg::kRingBytes + Cfg::kEpiStagingBytes;
  uint8_t* bar_gen = smem_gen + Cfg::kRingBytes + Cfg::kEpiStagingBytes;
  // Where raw stage s and tail slot t live.  With fewer tail slots than raw stages the tail
  // ring follows the raw ring; with equally many, every raw stage is followed by its own tail
  // tile (one combined stage).
  constexpr bool kTailPerStage = Cfg::kTailStages == kStages;
  constexpr uint32_t kRawPitch = kTailPerStage ? 2u * Cfg::kRawBytes : 1u * Cfg::kRawBytes;
  constexpr uint32_t kTailBase = kTailPerStage ? 1u * Cfg::kRawBytes : kStages * Cfg::kRawBytes;
  constexpr uint32_t kTailPitch = kRawPitch;
  // barrier slots (8 bytes each)
  auto full_raw = [&](int s) { return bar_base + 8u * s; };                 // TMA -> converter / MMA
  auto full_cvt = [&](int s) { return bar_base + 8u * (kStages + s); };     // converter -> MMA
  auto empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };  // MMA -> TMA
  auto tmem_full = [&](int a) { return bar_base + 8u * (3 * kStages + a); };
  auto tmem_empty = [&](int a) { return bar_base + 8u * (3 * kStages + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (3 * kStages + 4);
  volatile uint32_t* tmem_slot_gen =
      reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (3 * kStages + 4));
  volatile uint32_t* abort_flag =
      reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (3 * kStages + 4) + 4);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCtaGroup == 2) ? ptx::cluster_ctarank() : 0u;
  const bool is_leader = (cta_rank == 0);
  // K split over a cluster (see UmmaGemmParams::cluster_k): the fp32 split kernel and the int8
  // kernel, single CTAs only
  constexpr bool kClusterKCapable = kCtaGroup == 1 && (kSplit || kKind == ptx::MmaKind::I8);
  const unsigned ksplit = (kClusterKCapable && p.cluster_k > 1) ? p.cluster_k : 1u;
  const unsigned krank = ksplit > 1 ? ptx::cluster_ctarank() : 0u;
  const bool in_cluster = (kCtaGroup == 2) || ksplit > 1;
  const unsigned num_groups = gridDim.x / (kCtaGroup * ksplit);  // CTAs / pairs / clusters walking the tiles
  const unsigned group_id = blockIdx.x / (kCtaGroup * ksplit);
  const unsigned total_tiles = p.batch * p.tiles_m * p.tiles_n;
  const unsigned num_kb = (p.K + Cfg::kBK - 1) / Cfg::kBK;
  const unsigned kb_per_rank = (num_kb + ksplit - 1) / ksplit;
  const unsigned kb_lo = krank * kb_per_rank;                  // this CTA's k-blocks: [kb_lo, kb_hi)
  const unsigned kb_hi = min(num_kb, kb_lo + kb_per_rank);
  const uint32_t red_free = bar_base + 8u * (3 * kStages + 5);   // rank 0 -> others: buffer usable
  const uint32_t red_ready = bar_base + 8u * (3 * kStages + 6);  // others -> rank 0: partials written
  static_assert(8 * (3 * kStages + 7) <= 256, "barrier slots overrun their area");
  static_assert(Cfg::kTailStages <= kStages, "a tail slot is released by the raw-stage barrier");

  // segment table of the k-shared tiles (see UmmaGemmParams::sk_tiles), filled by thread 0
  uint4* seg_table = reinterpret_cast<uint4*>(bar_gen + 256);
  volatile uint32_t* sk_count_gen =
      reinterpret_cast<volatile uint32_t*>(bar_gen + 256 + 16 * kMaxSkSegments);

  // where the tiles go, read from shared memory by the store loops (see EpiTarget)
  static_assert(sizeof(EpiTarget) <= 128, "store target overruns its area");
  EpiTarget* tgt_smem = reinterpret_cast<EpiTarget*>(bar_gen + 256 + 16 * kMaxSkSegments + 16);

  UmmaCtl ctl{abort_flag, p.status, p.timeout_ns, p.flag_timeout_ns};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_raw(s), 1);
      ptx::mbar_init(full_cvt(s), kSplit ? Cfg::kNumConvertWarps * kCtaGroup : 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full(a), 1);
      ptx::mbar_init(tmem_empty(a), Cfg::kNumEpilogueWarps * kCtaGroup);
    }
    // fp32: rank 0 alone tells the others that its stage buffers are free; int8: every rank
    // hears from all the others
    ptx::mbar_init(red_free, (kSplit || ksplit < 2) ? 1 : ksplit - 1);
    ptx::mbar_init(red_ready, ksplit > 1 ? (ksplit - 1) * Cfg::kNumEpilogueWarps * 32 : 1);
    *abort_flag = 0;
    fill_epi_target(tgt_smem, p);
    unsigned nseg = 0;
    if (kSplit && p.global_k > 1) {
      const unsigned tile = group_id / p.global_k, r = group_id % p.global_k;
      const unsigned per = (num_kb + p.global_k - 1) / p.global_k;
      const unsigned lo = min(num_kb, r * per), hi = min(num_kb, lo + per);
      if (tile < total_tiles) seg_table[nseg++] = make_uint4(tile, lo, hi, r == 0 ? kSegGather : kSegHead);
    } else if (kSplit && p.sk_tiles) {
      const unsigned long long total_kb = static_cast<unsigned long long>(p.sk_tiles) * num_kb;
      const unsigned long long s0 = static_cast<unsigned long long>(group_id) * p.sk_kb_per_group;
      const unsigned long long e0 = min(total_kb, s0 + p.sk_kb_per_group);
      if (s0 < e0) {
        const unsigned t_first = static_cast<unsigned>(s0 / num_kb);
        const unsigned s_off = static_cast<unsigned>(s0 - static_cast<unsigned long long>(t_first) * num_kb);
        const unsigned t_last = static_cast<unsigned>((e0 - 1) / num_kb);
        const unsigned e_off = static_cast<unsigned>(e0 - static_cast<unsigned long long>(t_last) * num_kb);
        const bool has_tail = s_off != 0, has_head = e_off != num_kb;
        // The head goes first and the tail last: the previous group has then long published
        // the sums this group's tail continues, and nobody waits on anybody in practice.
        if (has_head) seg_table[nseg++] = make_uint4(t_last, 0u, e_off, kSegHead);
        for (unsigned t = t_first + (has_tail ? 1u : 0u);
             t + (has_head ? 1u : 0u) <= t_last && nseg < kMaxSkSegments - 1; ++t)
          seg_table[nseg++] = make_uint4(t, 0u, num_kb, 0u);
        if (has_tail) seg_table[nseg++] = make_uint4(t_first, s_off, num_kb, kSegTail);
      }
    }
    *sk_count_gen = nseg;
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmapA);
    ptx::prefetch_tensormap(&tmapB);
    if (p.tma_store) ptx::prefetch_tensormap(&tmapC);
  }
  if (warp == 1) {
    ptx::tmem_alloc<kCtaGroup>(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish<kCtaGroup>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (in_cluster) {  // peer barriers must exist before anyone signals them
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;
  // Everything above touched only shared and tensor memory and may have overlapped the tail of
  // the previous kernel in the stream; operands, bias, scratch and results come after this.
  pdl_wait();

  // The walk of this CTA: first its segments of the k-shared tiles, then whole tiles with a
  // stride of the grid.  Every role iterates the same list.
  const unsigned sk_count = kSplit ? *sk_count_gen : 0u;
  const unsigned dp_first = (kSplit ? p.sk_tiles : 0u) + group_id;
  const unsigned num_segments =
      sk_count + (dp_first < total_tiles ? (total_tiles - dp_first + num_groups - 1) / num_groups : 0u);
  auto segment = [&](unsigned i) {
    UmmaSegment sg;
    if (kSplit && i < sk_count) {
      const uint4 v = seg_table[i];
      sg.tile = v.x; sg.kb_lo = v.y; sg.kb_hi = v.z; sg.mode = v.w;
    } else {
      sg.tile = dp_first + (i - sk_count) * num_groups;
      sg.kb_lo = kb_lo; sg.kb_hi = kb_hi; sg.mode = 0u;
    }
    return sg;
  };

  // number of k-blocks per accumulator hand-off: the whole K unless partial sums are promoted
  const unsigned kb_per_chunk = kSplit ? max(1u, p.kb_per_chunk) : max(1u, num_kb);

  // Roles are split by warpgroup first, so that (kSplit) each warpgroup executes exactly
  // one setmaxnreg at the top of the code it alone runs.
  if (warp < Cfg::kFirstEpilogueWarp) {
  if constexpr (kSplit) ptx::setmaxnreg_dec<Cfg::kRegsControl>();
  // =========================== TMA producer ===========================
  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool live = true;  // cleared when a wait is abandoned: nothing more is loaded
      for (unsigned si = 0; si < num_segments && live; ++si) {
        const UmmaSegment sg = segment(si);
        unsigned b, tm, tn;
        tile_coords(sg.tile, p.tiles_m, p.tiles_n, b, tm, tn);
        const int m0 = static_cast<int>(tm * Cfg::kTileM + cta_rank * Cfg::kBM);
        const int n0 = static_cast<int>(tn * BN + cta_rank * Cfg::kBNLocal);
        const int ba = p.a_batched ? static_cast<int>(b) : 0;
        const int bb = p.b_batched ? static_cast<int>(b) : 0;
        for (unsigned kb = sg.kb_lo; kb < sg.kb_hi; ++kb) {
          if (!bounded_wait<false>(empty_bar(s), ph ^ 1u, TFCCB200_DEV_TIMEOUT_TMA, ctl)) {
            live = false;
            break;
          }
          const uint32_t stage = smem_base + s * kRawPitch;
          const int k0 = static_cast<int>(kb * Cfg::kBK);
          if constexpr (kCtaGroup == 2 && !kSplit) {
            // Both CTAs' bytes are counted on the leader's barrier; the MMA
            // issuer in the leader is the only consumer.
            const uint32_t bar = full_raw(s) & 0xFEFFFFFFu;
            if (is_leader) ptx::mbar_expect_tx(full_raw(s), 2u * Cfg::kRawBytes);
            ptx::tma_load_3d_pair(stage, &tmapA, bar, k0, m0, ba);
#pragma unroll
            for (int c = 0; c < Cfg::kBChunks; ++c)
              ptx::tma_load_3d_pair(stage + Cfg::kABytes + c * Cfg::kBChunkBytes, &tmapB, bar,
                                    n0 + c * (128 / Cfg::kElemBytes), k0, bb);
          } else {
            ptx::mbar_expect_tx(full_raw(s), Cfg::kRawBytes);
            ptx::tma_load_3d(stage, &tmapA, full_raw(s), k0, m0, ba);
#pragma unroll
            for (int c = 0; c < Cfg::kBChunks; ++c)
              ptx::tma_load_3d(stage + Cfg::kABytes + c * Cfg::kBChunkBytes, &tmapB, full_raw(s),
                               n0 + c * (128 / Cfg::kElemBytes), k0, bb);
          }
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
    }
  }
  // =========================== MMA issuer ===========================
  else if (warp == 1) {
    if (lane == 0 && is_leader) {
      int s = 0;
      uint32_t ph = 0;
      int ts = 0;       // slot of the tail ring (kSplit)
      unsigned it = 0;  // accumulator hand-offs so far (tiles, or chunks when kSplit)
      const uint16_t pair_mask = 0x3;
      bool live = true;  // cleared when a wait is abandoned: no further MMA is issued
      for (unsigned si = 0; si < num_segments && live; ++si) {
        const UmmaSegment sg = segment(si);
        for (unsigned kb0 = sg.kb_lo; kb0 < sg.kb_hi && live; kb0 += kb_per_chunk, ++it) {
          const unsigned acc = it & 1u;
          const uint32_t acc_ph = (it >> 1) & 1u;
          if (!bounded_wait<(kCtaGroup == 2)>(tmem_empty(acc), acc_ph ^ 1u,
                                              TFCCB200_DEV_TIMEOUT_MMA, ctl)) {
            live = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * BN;
          const unsigned kb_end = min(sg.kb_hi, kb0 + kb_per_chunk);
          for (unsigned kb = kb0; kb < kb_end; ++kb) {
            bool ready;
            if constexpr (kSplit) {
              ready = bounded_wait<(kCtaGroup == 2)>(full_cvt(s), ph, TFCCB200_DEV_TIMEOUT_MMA, ctl);
            } else {
              ready = bounded_wait<false>(full_raw(s), ph, TFCCB200_DEV_TIMEOUT_MMA, ctl);
            }
            if (!ready) {
              live = false;
              break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t a_hi = smem_base + s * kRawPitch;
            const uint32_t b_hi = a_hi + Cfg::kABytes;
            const uint32_t a_lo = smem_base + kTailBase + ts * kTailPitch;
            const uint32_t b_lo = a_lo + Cfg::kABytes;
#pragma unroll
            for (int ks = 0; ks < Cfg::kKSteps; ++ks) {
              const uint64_t da_hi = ptx::smem_desc(a_hi + ks * 32, 16, 1024, ptx::kLayoutSw128);
              const uint64_t db_hi = ptx::smem_desc(b_hi + ks * Cfg::kBKStepBytes,
                                                    Cfg::kBChunkBytes, Cfg::kBSbo, Cfg::kBLayout);
              const uint32_t accum = (kb > kb0 || ks > 0) ? 1u : 0u;
              if constexpr (kSplit) {
                const uint64_t da_lo = ptx::smem_desc(a_lo + ks * 32, 16, 1024, ptx::kLayoutSw128);
                const uint64_t db_lo = ptx::smem_desc(b_lo + ks * Cfg::kBKStepBytes,
                                                      Cfg::kBChunkBytes, Cfg::kBSbo, Cfg::kBLayout);
                ptx::umma<kKind, kCtaGroup>(d_tmem, da_lo, db_hi, Cfg::kIdesc, accum);
                ptx::umma<kKind, kCtaGroup>(d_tmem, da_hi, db_lo, Cfg::kIdesc, 1u);
                ptx::umma<kKind, kCtaGroup>(d_tmem, da_hi, db_hi, Cfg::kIdesc, 1u);
              } else {
                ptx::umma<kKind, kCtaGroup>(d_tmem, da_hi, db_hi, Cfg::kIdesc, accum);
              }
            }
            ptx::umma_commit<kCtaGroup>(empty_bar(s), pair_mask);  // stage free when MMAs retire
            if constexpr (kSplit) {
              if (++ts == Cfg::kTailStages) ts = 0;
            }
            if (++s == kStages) { s = 0; ph ^= 1u; }
          }
          if (!live) break;
          ptx::umma_commit<kCtaGroup>(tmem_full(acc), pair_mask);  // this accumulator is complete
        }
      }
    }
  }
  // (kSplit: warps 2 and 3 only fill the control warpgroup)
  }
  // =========================== epilogue ===========================
  else if (warp < Cfg::kFirstConvertWarp) {
    if constexpr (kSplit) ptx::setmaxnreg_inc<Cfg::kRegsEpilogue>();
    const uint32_t q = warp & 3u;  // TMEM lane quarter this warp may read
    // kSplit: warps 4..7 own the left half of the columns, 8..11 the right half
    const uint32_t col_half = kSplit ? (warp - Cfg::kFirstEpilogueWarp) >> 2 : 0u;
    unsigned it = 0;
    const uint32_t leader_tmem_empty0 =
        (kCtaGroup == 2) ? ptx::mapa(tmem_empty(0), 0) : tmem_empty(0);
    auto release_acc = [&](unsigned acc) {
      // the accumulator buffer may now be overwritten by the MMA issuer
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtaGroup == 2) ptx::mbar_arrive_cluster(leader_tmem_empty0 + 8u * acc);
        else ptx::mbar_arrive(tmem_empty(acc));
      }
    };
    for (unsigned si = 0; si < num_segments; ++si) {
      const UmmaSegment sg = segment(si);
      // Where the tile goes.  (kSplit computes this only after the accumulation, when the
      // registers holding the running sums are the only other long-lived values.)
      unsigned b, row0, col0;
      unsigned long long batch_off;
      auto locate_tile = [&]() {
        unsigned tm, tn;
        tile_coords(sg.tile, p.tiles_m, p.tiles_n, b, tm, tn);
        row0 = tm * Cfg::kTileM + cta_rank * Cfg::kBM + q * 32;  // lane 0's row
        col0 = tn * BN + col_half * Cfg::kEpiCols;
        batch_off = p.strideC * b;
      };
      if constexpr (!kSplit) locate_tile();
      const uint32_t lane_addr = tmem_base + ((q * 32u) << 16) + col_half * Cfg::kEpiCols;
      uint32_t* stage = reinterpret_cast<uint32_t*>(
          epi_stage_gen + (warp - Cfg::kFirstEpilogueWarp) * Cfg::kEpiStageBytes);
      uint32_t* const stage_one = stage;
      auto bias_term = [&](unsigned col_blk, const float* bias, unsigned n) {
        uint4 t = make_uint4(0u, 0u, 0u, 0u);  // +0.0f
        const unsigned col = col_blk + (lane & 7u) * 4;
        if (bias && col < n) t = __ldg(reinterpret_cast<const uint4*>(bias + col));
        return t;
      };
      // The per-column terms of this tile (bias; int8: column sums of B, row sums of A) are
      // asked for now, while the mainloop runs, so that the loads after the accumulation hit
      // the cache instead of adding a trip to DRAM to every launch's tail.
      if (sg.mode != kSegHead) {
        unsigned pb, ptm, ptn;
        tile_coords(sg.tile, p.tiles_m, p.tiles_n, pb, ptm, ptn);
        const unsigned pcol = ptn * BN + lane * 8;  // 32 lanes x 32 bytes cover 256 columns
        if constexpr (kKind == ptx::MmaKind::I8) {
          if (pcol < p.N && lane * 8 < BN)
            ptx::prefetch_l2(p.rsB + static_cast<size_t>(p.strideRsB) * pb + pcol);
          const unsigned prow = ptm * Cfg::kTileM + cta_rank * Cfg::kBM + q * 32 + (lane & 3u) * 8;
          if (lane < 4 && prow < p.M)
            ptx::prefetch_l2(p.rsA + static_cast<size_t>(p.strideRsA) * pb + prow);
        } else {
          if (p.bias && pcol < p.N && lane * 8 < BN) ptx::prefetch_l2(p.bias + pcol);
        }
        // The CTA's last tile stages its results in the dead ring (see the store loops), which
        // leaves this warp's 4 KB block free: the warp's per-column terms go there now, so that
        // the store phase reads them from shared memory.  (Loaded one by one after the
        // accumulation they cost about 0.12 us each, a microsecond per 32 columns.)
        if (si + 1 == num_segments) {
          constexpr int kWarpCols = kSplit ? Cfg::kEpiCols : BN;
          const unsigned wcol0 = ptn * BN + col_half * Cfg::kEpiCols;
          if constexpr (kKind == ptx::MmaKind::I8) {
            const int32_t* rsb = p.rsB + static_cast<size_t>(p.strideRsB) * pb;
#pragma unroll
            for (int i = 0; i < kWarpCols / 32; ++i) {
              const unsigned col = wcol0 + i * 32 + lane;
              stage_one[i * 32 + lane] = col < p.N ? static_cast<uint32_t>(__ldg(rsb + col)) : 0u;
            }
          } else {
#pragma unroll
            for (int i = 0; i < kWarpCols / 32; ++i) {
              const unsigned col = wcol0 + i * 32 + lane;
              stage_one[i * 32 + lane] =
                  (p.bias && col < p.N) ? __float_as_uint(__ldg(p.bias + col)) : 0u;
            }
          }
          __syncwarp();
        }
      }

      if constexpr (kSplit) {
        // ---- promote every chunk's partial sum into registers (round-to-nearest adds) ----
        float sum[Cfg::kEpiCols];
        constexpr int kSkVec = Cfg::kEpiCols / 4;
        // this thread's float4 slots in a partial-sum tile: [warp][4-column group][lane]
        const unsigned sk_slot = ((warp - Cfg::kFirstEpilogueWarp) * kSkVec) * 32 + lane;
        constexpr unsigned kSkTileVecs = Cfg::kNumEpilogueWarps * kSkVec * 32;  // float4 per CTA tile
        if (sg.mode == kSegTail) {
          // continue the sums the previous group published for the same rows of this tile
          const unsigned src_cta = (group_id - 1) * kCtaGroup + cta_rank;
          if (lane == 0)
            bounded_flag_wait(p.sk_flags + src_cta,
                              Cfg::kNumEpilogueWarps * 32u + p.flag_expect_extra,
                              TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
          __syncwarp();
          const float4* src = reinterpret_cast<const float4*>(p.sk_partials) +
                              static_cast<size_t>(src_cta) * kSkTileVecs + sk_slot;
          sk_load_partial<kSkVec>(sum, src);
        } else {
#pragma unroll
          for (int j = 0; j < Cfg::kEpiCols; ++j) sum[j] = 0.f;
        }
        for (unsigned kb0 = sg.kb_lo; kb0 < sg.kb_hi; kb0 += kb_per_chunk, ++it) {
          const unsigned acc = it & 1u;
          const uint32_t acc_ph = (it >> 1) & 1u;
          bounded_wait<false>(tmem_full(acc), acc_ph, TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
          ptx::tc_fence_after_sync();
          const uint32_t taddr = lane_addr + acc * BN;
#pragma unroll
          for (int c = 0; c < Cfg::kEpiCols / 16; ++c) {
            uint32_t r[16];
            ptx::tmem_ld_32x16(taddr + c * 16, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) sum[c * 16 + j] += __uint_as_float(r[j]);
          }
          release_acc(acc);
        }
        if (sg.mode == kSegHead) {
          // publish the partial sums for the group that finishes this tile
          const unsigned my_cta = group_id * kCtaGroup + cta_rank;
          float4* out = reinterpret_cast<float4*>(p.sk_partials) +
                        static_cast<size_t>(my_cta) * kSkTileVecs + sk_slot;
          sk_store_partial<kSkVec>(sum, out);
          __threadfence();
          atomicAdd(p.sk_flags + my_cta, 1u);
          continue;
        }
        if (sg.mode == kSegGather) {
          // rank 0 of a global K split: the other ranks' sums, in rank order
          for (unsigned r = 1; r < p.global_k; ++r) {
            const unsigned src_cta = group_id + r;
            if (lane == 0)
              bounded_flag_wait(p.sk_flags + src_cta,
                                Cfg::kNumEpilogueWarps * 32u + p.flag_expect_extra,
                                TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
            __syncwarp();
            sk_add_partial<kSkVec>(sum, reinterpret_cast<const float4*>(p.sk_partials) +
                                            static_cast<size_t>(src_cta) * kSkTileVecs + sk_slot);
          }
        }
        if (ksplit > 1) {
          // ---- K split over the cluster: partial sums meet in rank 0's (now idle) stage
          // buffers, laid out [rank-1][warp][4-column group][lane] so that every access is a
          // conflict-free 128-bit one.  Rank 0's last tmem_full above means all its MMAs have
          // retired, so its stages are dead and may be overwritten.
          const unsigned ew = warp - Cfg::kFirstEpilogueWarp;
          constexpr int kVec = Cfg::kEpiCols / 4;
          if (krank == 0) {
            if (ew == 0 && lane == 0)
              for (unsigned r = 1; r < ksplit; ++r) ptx::mbar_arrive_cluster(ptx::mapa(red_free, r));
            bounded_wait<true>(red_ready, 0u, TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
            const float4* red = reinterpret_cast<const float4*>(smem_gen);
            for (unsigned r = 1; r < ksplit; ++r) {  // fixed order: rank 1, 2, ...
#pragma unroll
              for (int v = 0; v < kVec; ++v) {
                const float4 t = red[(((r - 1) * Cfg::kNumEpilogueWarps + ew) * kVec + v) * 32 + lane];
                sum[4 * v + 0] += t.x; sum[4 * v + 1] += t.y;
                sum[4 * v + 2] += t.z; sum[4 * v + 3] += t.w;
              }
            }
          } else {
            bounded_wait<true>(red_free, 0u, TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
            const uint32_t remote = ptx::mapa(smem_base, 0);
#pragma unroll
            for (int v = 0; v < kVec; ++v)
              ptx::st_shared_cluster_v4(
                  remote + 16u * ((((krank - 1) * Cfg::kNumEpilogueWarps + ew) * kVec + v) * 32 + lane),
                  make_float4(sum[4 * v], sum[4 * v + 1], sum[4 * v + 2], sum[4 * v + 3]));
            ptx::mbar_arrive_cluster(ptx::mapa(red_ready, 0));  // every lane: releases its own stores
            continue;  // rank 0 stores the tile
          }
        }
        locate_tile();
        const EpiTarget& tgt = *tgt_smem;
        const float* const pbias = tgt.bias;
        if (tgt.tma_store) {
          const unsigned n_lim = tgt.N;
          const int act = tgt.activation;
          // The CTA's last tile: every MMA has retired and every load has been consumed, so
          // the stage ring is dead and each warp stages ALL its blocks there (its own slot of
          // the partial-sum area, which only it read), fires the stores back to back and waits
          // once.  Earlier tiles reuse the warp's 4 KB block, their waits hide behind the next
          // tile's mainloop.
          const bool last_tile = si + 1 == num_segments;
          uint32_t* const wide = reinterpret_cast<uint32_t*>(
              smem_gen + (warp - Cfg::kFirstEpilogueWarp) * (Cfg::kEpiCols / 32) * Cfg::kEpiStageBytes);
#pragma unroll
          for (int c = 0; c < Cfg::kEpiCols / 32; ++c) {
            if (col0 + c * 32 >= n_lim) break;  // warp-uniform
            uint32_t* const stage = last_tile ? wide + c * (Cfg::kEpiStageBytes / 4) : stage_one;
            if (!last_tile) epi_tma_stage_free(lane);
#pragma unroll
            for (int qq = 0; qq < 8; ++qq) {
              const unsigned col = col0 + c * 32 + 4 * qq;
              float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
              if (last_tile) bv = *reinterpret_cast<const float4*>(stage_one + c * 32 + 4 * qq);
              else if (pbias && col < n_lim) bv = __ldg(reinterpret_cast<const float4*>(pbias + col));
              float4 v = make_float4(sum[c * 32 + 4 * qq + 0] + bv.x, sum[c * 32 + 4 * qq + 1] + bv.y,
                                     sum[c * 32 + 4 * qq + 2] + bv.z, sum[c * 32 + 4 * qq + 3] + bv.w);
              if (act != TFCCB200_ACT_NONE) {
                v.x = apply_activation(v.x, act); v.y = apply_activation(v.y, act);
                v.z = apply_activation(v.z, act); v.w = apply_activation(v.w, act);
              }
              epi_stage_chunk(stage, lane, qq,
                              make_uint4(__float_as_uint(v.x), __float_as_uint(v.y),
                                         __float_as_uint(v.z), __float_as_uint(v.w)));
            }
            epi_tma_store_block(stage, lane, &tmapC, col0 + c * 32, row0, b);
          }
          epi_tma_stage_free(lane);
          continue;
        }
#pragma unroll
        for (int c = 0; c < Cfg::kEpiCols / 32; ++c) {
          if (col0 + c * 32 >= tgt.N) break;  // warp-uniform
#pragma unroll
          for (int qq = 0; qq < 8; ++qq)
            epi_stage_chunk(stage, lane, qq,
                            make_uint4(__float_as_uint(sum[c * 32 + 4 * qq + 0]),
                                       __float_as_uint(sum[c * 32 + 4 * qq + 1]),
                                       __float_as_uint(sum[c * 32 + 4 * qq + 2]),
                                       __float_as_uint(sum[c * 32 + 4 * qq + 3])));
          epi_flush_block<true>(stage, lane, row0, col0 + c * 32, tgt, batch_off,
                                bias_term(col0 + c * 32, pbias, tgt.N));
        }
      } else {
        const unsigned acc = it & 1u;
        const uint32_t acc_ph = (it >> 1) & 1u;
        ++it;
        const unsigned pN = tgt_smem->N, pM = tgt_smem->M;
        const float* const pbias = tgt_smem->bias;
        // int8: the zero-point scalars of this lane's row, fetched before the accumulator is
        // waited for so that their latency hides behind the mainloop
        const int32_t* rsB = nullptr;
        const unsigned row = row0 + lane;
        const bool row_ok = row < pM;
        uint32_t oa = 0, ob = 0, row_term = 0;
        if constexpr (kKind == ptx::MmaKind::I8) {
          rsB = p.rsB + static_cast<size_t>(p.strideRsB) * b;
          oa = static_cast<uint32_t>(p.offA);
          ob = static_cast<uint32_t>(p.offB);
          row_term = static_cast<uint32_t>(p.kterm);
          if (p.q_offsets) {
            oa = static_cast<uint32_t>(__ldg(p.q_offsets));
            ob = static_cast<uint32_t>(__ldg(p.q_offsets + 1));
            row_term = oa * ob * p.K;
          }
          if (row_ok)
            row_term += static_cast<uint32_t>(__ldg(p.rsA + static_cast<size_t>(p.strideRsA) * b + row)) * ob;
        }
        bounded_wait<false>(tmem_full(acc), acc_ph, TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
        ptx::tc_fence_after_sync();
        const uint32_t taddr = lane_addr + acc * BN;
        const EpiTarget& tgt = *tgt_smem;
        if constexpr (kKind != ptx::MmaKind::I8) {
          if (tgt.tma_store) {
            const int act = tgt.activation;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              if (col0 + c * 32 >= pN) break;  // warp-uniform
              uint32_t r[32];
              ptx::tmem_ld_32x32(taddr + c * 32, r);
              ptx::tmem_ld_wait();
              epi_tma_stage_free(lane);
#pragma unroll
              for (int qq = 0; qq < 8; ++qq) {
                const unsigned col = col0 + c * 32 + 4 * qq;
                float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (pbias && col < pN) bv = __ldg(reinterpret_cast<const float4*>(pbias + col));
                float4 v = make_float4(__uint_as_float(r[4 * qq]) + bv.x, __uint_as_float(r[4 * qq + 1]) + bv.y,
                                       __uint_as_float(r[4 * qq + 2]) + bv.z, __uint_as_float(r[4 * qq + 3]) + bv.w);
                if (act != TFCCB200_ACT_NONE) {
                  v.x = apply_activation(v.x, act); v.y = apply_activation(v.y, act);
                  v.z = apply_activation(v.z, act); v.w = apply_activation(v.w, act);
                }
                epi_stage_chunk(stage, lane, qq,
                                make_uint4(__float_as_uint(v.x), __float_as_uint(v.y),
                                           __float_as_uint(v.z), __float_as_uint(v.w)));
              }
              epi_tma_store_block(stage, lane, &tmapC, col0 + c * 32, row0, b);
            }
            epi_tma_stage_free(lane);
          } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            if (col0 + c * 32 >= pN) break;  // warp-uniform
            const uint4 bt = bias_term(col0 + c * 32, pbias, pN);
            uint32_t r[32];
            ptx::tmem_ld_32x32(taddr + c * 32, r);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int qq = 0; qq < 8; ++qq)
              epi_stage_chunk(stage, lane, qq,
                              make_uint4(r[4 * qq], r[4 * qq + 1], r[4 * qq + 2], r[4 * qq + 3]));
            epi_flush_block<true>(stage, lane, row0, col0 + c * 32, tgt, batch_off, bt);
          }
          }
        } else {
          // zero-point correction.  The int8 mainloop already saturates shared-memory
          // bandwidth (TMA fill + MMA operand reads), so this epilogue stays out of shared
          // memory: every lane stores its own row's columns straight from registers.
          if (ksplit > 1) {
            // ---- K split over the cluster: reduce-scatter of the int32 accumulators.  Rank r
            // owns columns [r, r+1) * BN / ksplit of the tile.  The tmem_full wait above means
            // this CTA's MMAs have retired, so its stage buffers are dead; once every rank has
            // said so, each sends the others their slices of its accumulator straight into
            // their stage buffers, laid out [source][warp][4-column group][lane] (conflict-free
            // 128-bit accesses), and then adds what it received to its own slice.
            const unsigned ew = warp - Cfg::kFirstEpilogueWarp;
            const unsigned slice = BN / ksplit;  // multiple of 32 (checked on the host)
            const unsigned qper = slice / 4;     // 128-bit groups per row of a slice
            if (ew == 0 && lane == 0)
              for (unsigned r = 0; r < ksplit; ++r)
                if (r != krank) ptx::mbar_arrive_cluster(ptx::mapa(red_free, r));
            bounded_wait<true>(red_free, 0u, TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
            for (unsigned d = 0; d < ksplit; ++d) {
              if (d == krank) continue;
              const unsigned si = krank < d ? krank : krank - 1;  // this rank among d's sources
              const uint32_t remote = ptx::mapa(smem_base, d);
              for (unsigned c = 0; c < slice / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(taddr + d * slice + c * 32, r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int v = 0; v < 8; ++v)
                  ptx::st_shared_cluster_v4_b32(
                      remote + 16u * (((si * Cfg::kNumEpilogueWarps + ew) * qper + c * 8 + v) * 32 + lane),
                      r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
              }
              ptx::mbar_arrive_cluster(ptx::mapa(red_ready, d));  // every lane: releases its stores
            }
            bounded_wait<true>(red_ready, 0u, TFCCB200_DEV_TIMEOUT_EPILOGUE, ctl);
            const uint4* red = reinterpret_cast<const uint4*>(smem_gen);
            const unsigned colbase = col0 + krank * slice;
            uint32_t* crow = tgt.dst[0] + batch_off + static_cast<unsigned long long>(row) * tgt.ldc +
                             tgt.col_offset + colbase;
            for (unsigned c = 0; c < slice / 32; ++c) {
              if (colbase + c * 32 >= pN) break;
              uint32_t r[32];
              ptx::tmem_ld_32x32(taddr + krank * slice + c * 32, r);
              ptx::tmem_ld_wait();
              for (unsigned s2 = 0; s2 + 1 < ksplit; ++s2) {
#pragma unroll
                for (int v = 0; v < 8; ++v) {
                  const uint4 t = red[((s2 * Cfg::kNumEpilogueWarps + ew) * qper + c * 8 + v) * 32 + lane];
                  r[4 * v] += t.x; r[4 * v + 1] += t.y; r[4 * v + 2] += t.z; r[4 * v + 3] += t.w;
                }
              }
              if (tgt.tma_store) {
                // the ring is dead (one tile per cluster): all blocks staged side by side in
                // this warp's own incoming slot, stores fired back to back, one wait at the end
                uint32_t* const stage = reinterpret_cast<uint32_t*>(smem_gen) +
                                        (ew * (slice / 32) + c) * (Cfg::kEpiStageBytes / 4);
#pragma unroll
                for (int qq = 0; qq < 8; ++qq) {
                  const uint4 sb = *reinterpret_cast<const uint4*>(stage_one + krank * slice + c * 32 + 4 * qq);
                  epi_stage_chunk(stage, lane, qq,
                                  make_uint4(r[4 * qq] + row_term + sb.x * oa, r[4 * qq + 1] + row_term + sb.y * oa,
                                             r[4 * qq + 2] + row_term + sb.z * oa, r[4 * qq + 3] + row_term + sb.w * oa));
                }
                epi_tma_store_block(stage, lane, &tmapC, colbase + c * 32, row0, b);
              } else if (row_ok) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  const unsigned col = colbase + c * 32 + j;
                  if (col < pN) {
                    const uint4 sb = __ldg(reinterpret_cast<const uint4*>(rsB + col));
                    uint4 v;
                    v.x = r[j + 0] + row_term + sb.x * oa;
                    v.y = r[j + 1] + row_term + sb.y * oa;
                    v.z = r[j + 2] + row_term + sb.z * oa;
                    v.w = r[j + 3] + row_term + sb.w * oa;
                    *reinterpret_cast<uint4*>(crow + c * 32 + j) = v;
                  }
                }
              }
            }
            if (tgt.tma_store) epi_tma_stage_free(lane);
          } else if (tgt.num_dst > 1 || tgt.mc) {
            // column shards pushed to several GPUs: go through the transposing stage so that
            // every store instruction covers whole 128-byte lines of the peers' memory
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              if (col0 + c * 32 >= pN) break;
              uint32_t r[32];
              ptx::tmem_ld_32x32(taddr + c * 32, r);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int qq = 0; qq < 8; ++qq)
                epi_stage_chunk(stage, lane, qq,
                                make_uint4(r[4 * qq] + row_term, r[4 * qq + 1] + row_term,
                                           r[4 * qq + 2] + row_term, r[4 * qq + 3] + row_term));
              uint4 ct = make_uint4(0u, 0u, 0u, 0u);
              const unsigned col = col0 + c * 32 + (lane & 7u) * 4;
              if (col < pN) {
                ct = __ldg(reinterpret_cast<const uint4*>(rsB + col));
                ct.x *= oa; ct.y *= oa; ct.z *= oa; ct.w *= oa;
              }
              epi_flush_block<false>(stage, lane, row0, col0 + c * 32, tgt, batch_off, ct);
            }
          } else {
          uint32_t* crow = tgt.dst[0] + batch_off + static_cast<unsigned long long>(row) * tgt.ldc +
                           tgt.col_offset + col0;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            if (col0 + c * 32 >= pN) break;
            uint32_t r[32];
            ptx::tmem_ld_32x32(taddr + c * 32, r);
            ptx::tmem_ld_wait();
            if (tgt.tma_store) {
              const bool last_tile = si + 1 == num_segments;  // ring dead: stage side by side
              uint32_t* const stage =
                  last_tile ? reinterpret_cast<uint32_t*>(smem_gen) +
                                  ((warp - Cfg::kFirstEpilogueWarp) * (BN / 32) + c) * (Cfg::kEpiStageBytes / 4)
                            : stage_one;
              if (!last_tile) epi_tma_stage_free(lane);
#pragma unroll
              for (int qq = 0; qq < 8; ++qq) {
                const unsigned col = col0 + c * 32 + 4 * qq;
                uint4 sb = make_uint4(0u, 0u, 0u, 0u);
                if (last_tile) sb = *reinterpret_cast<const uint4*>(stage_one + c * 32 + 4 * qq);
                else if (col < pN) sb = __ldg(reinterpret_cast<const uint4*>(rsB + col));
                epi_stage_chunk(stage, lane, qq,
                                make_uint4(r[4 * qq] + row_term + sb.x * oa, r[4 * qq + 1] + row_term + sb.y * oa,
                                           r[4 * qq + 2] + row_term + sb.z * oa, r[4 * qq + 3] + row_term + sb.w * oa));
              }
              epi_tma_store_block(stage, lane, &tmapC, col0 + c * 32, row0, b);
            } else if (row_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const unsigned col = col0 + c * 32 + j;
                if (col < pN) {  // N % 16 == 0 on this path
                  const uint4 sb = __ldg(reinterpret_cast<const uint4*>(rsB + col));
                  uint4 v;
                  v.x = r[j + 0] + row_term + sb.x * oa;
                  v.y = r[j + 1] + row_term + sb.y * oa;
                  v.z = r[j + 2] + row_term + sb.z * oa;
                  v.w = r[j + 3] + row_term + sb.w * oa;
                  *reinterpret_cast<uint4*>(crow + c * 32 + j) = v;
                }
              }
            }
          }
          if (tgt.tma_store) epi_tma_stage_free(lane);
          }
        }
        release_acc(acc);
      }
    }
  }
  // =========================== converters (kSplit) ===========================
  else {
    if constexpr (kSplit) {
      ptx::setmaxnreg_dec<Cfg::kRegsConvert>();
      const unsigned cthread = threadIdx.x - 32 * Cfg::kFirstConvertWarp;
      constexpr unsigned kCThreads = 32 * Cfg::kNumConvertWarps;
      constexpr unsigned kVecs = Cfg::kRawBytes / 16;
      static_assert(kVecs % kCThreads == 0, "converter loop must divide evenly");
      const uint32_t leader_full_cvt0 = (kCtaGroup == 2) ? ptx::mapa(full_cvt(0), 0) : full_cvt(0);
      int s = 0;
      uint32_t ph = 0;
      int ts = 0;  // tail ring slot
      // A tail slot is free again when the MMAs of the k-block that used it kTailStages
      // k-blocks ago have retired, which is what that k-block's raw-stage barrier (empty_bar)
      // reports: the converter follows the raw ring with that lag.
      unsigned done = 0;  // k-blocks converted so far
      int ls = 0;         // raw stage of the k-block kTailStages back, and its phase
      uint32_t lph = 0;
      bool live = true;  // cleared when a wait is abandoned: nothing more is converted
      for (unsigned si = 0; si < num_segments && live; ++si) {
        const UmmaSegment sg = segment(si);
        for (unsigned kb = sg.kb_lo; kb < sg.kb_hi; ++kb) {
          if constexpr (Cfg::kTailStages < kStages) {
            // (with as many tail slots as raw stages the raw tile's arrival implies it)
            if (done >= static_cast<unsigned>(Cfg::kTailStages)) {
              if (!bounded_wait<false>(empty_bar(ls), lph, TFCCB200_DEV_TIMEOUT_CONVERT, ctl)) {
                live = false;
                break;
              }
              if (++ls == kStages) { ls = 0; lph ^= 1u; }
            }
            ++done;
          }
          if (!bounded_wait<false>(full_raw(s), ph, TFCCB200_DEV_TIMEOUT_CONVERT, ctl)) {
            live = false;
            break;
          }
          float4* raw = reinterpret_cast<float4*>(smem_gen + s * kRawPitch);
          float4* tail = reinterpret_cast<float4*>(smem_gen + kTailBase + ts * kTailPitch);
          constexpr int kIter = kVecs / kCThreads;
          constexpr int kUnroll = (kIter % 4 == 0) ? 4 : (kIter % 2 == 0 ? 2 : 1);
#pragma unroll 1
          for (int i0 = 0; i0 < kIter; i0 += kUnroll) {
            float4 x[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) x[u] = raw[cthread + (i0 + u) * kCThreads];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
              float4 h, l;
              h.x = __uint_as_float(__float_as_uint(x[u].x) & 0xFFFFE000u);
              h.y = __uint_as_float(__float_as_uint(x[u].y) & 0xFFFFE000u);
              h.z = __uint_as_float(__float_as_uint(x[u].z) & 0xFFFFE000u);
              h.w = __uint_as_float(__float_as_uint(x[u].w) & 0xFFFFE000u);
              uint32_t lx, ly, lz, lw;
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lx) : "f"(x[u].x - h.x));
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(ly) : "f"(x[u].y - h.y));
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lz) : "f"(x[u].z - h.z));
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lw) : "f"(x[u].w - h.w));
              l.x = __uint_as_float(lx); l.y = __uint_as_float(ly);
              l.z = __uint_as_float(lz); l.w = __uint_as_float(lw);
              tail[cthread + (i0 + u) * kCThreads] = l;
              if (p.write_head) raw[cthread + (i0 + u) * kCThreads] = h;
            }
          }
          ptx::fence_proxy_async_smem();  // generic-proxy stores -> visible to tcgen05.mma
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtaGroup == 2) ptx::mbar_arrive_cluster(leader_full_cvt0 + 8u * s);
            else ptx::mbar_arrive(full_cvt(s));
          }
          if (++s == kStages) { s = 0; ph ^= 1u; }
          if (++ts == Cfg::kTailStages) ts = 0;
        }
      }
    }
  }

  // ---- teardown: nobody leaves while a peer may still signal it; TMEM goes back ----
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // A wait was abandoned: loads and MMAs may still be in flight.  Give them a
    // bounded moment to land before shared and tensor memory are released.
    const uint64_t t0 = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (in_cluster) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<kCtaGroup>(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace tfccb200
