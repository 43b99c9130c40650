// Internal declarations shared by the translation units of libtfcc_b200.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/tfcc_b200.h"

namespace tfccb200 {

// Immutable facts about one CUDA device, looked up once.
struct DeviceInfo {
  int sm_count;
  int cc_major, cc_minor;
  size_t l2_bytes;
};
// Info for the current device; nullptr when the runtime reports an error (*err is set).
const DeviceInfo* current_device_info(cudaError_t* err);

void count_launch(unsigned n = 1);

// Default bound of every device-side wait (nanoseconds).
constexpr unsigned long long kDefaultTimeoutNs = 2000000000ull;

struct SgemmArgs {
  cudaStream_t stream;
  const float* A;
  const float* B;
  float* C;
  const float* bias;
  unsigned strideA, strideB, strideC;
  unsigned M, N, K, batch;
  int precision;
  void* workspace;
  size_t workspace_bytes;
  int* status;
  // Tensor-core path only: store the result into `num_dst` matrices of row pitch `ldc`
  // starting at column `col_offset` (num_dst == 0: the plain case, C with pitch N).
  float* dst[8];
  unsigned num_dst;
  float* mc_dst;  // NVLink multicast alias of the destinations, or nullptr
  unsigned long long ldc;
  unsigned col_offset;
  int activation;  // TFCCB200_ACT_*: applied to A.B + bias before the store
  unsigned max_ctas;  // tensor-core path: use at most this many SMs (0 = all); lets two
                      // products run side by side on disjoint parts of the chip
};

struct QgemmArgs {
  cudaStream_t stream;
  const uint8_t* A;
  const int8_t* B;
  int32_t* C;
  const int32_t* rsA;
  const int32_t* rsB;
  unsigned strideA, strideB, strideC, strideRsA, strideRsB;
  int32_t offA, offB;
  const int32_t* dev_offsets;  // device {offA, offB}; when set, offA / offB above are ignored
  unsigned M, N, K, batch;
  int* status;
  // Tensor-core path only (as in SgemmArgs): several destinations / a multicast alias, row
  // pitch ldc, first column col_offset; num_dst == 0 is the plain case.
  int32_t* dst[8];
  unsigned num_dst;
  int32_t* mc_dst;
  unsigned long long ldc;
  unsigned col_offset;
};

// ---- tcgen05 paths (umma_launch.cu) ----
// pair == true runs cta_group::2 (a CTA pair per 256-row tile).
// Tile shape for a problem: CTA pairs or single CTAs, and the tile width.
// force_pair: -1 = choose, 0 = single CTAs, 1 = pairs.
struct UmmaPlan {
  bool pair;
  int bn;
  unsigned cluster_k;  // > 1: K of one tile is shared by a cluster of that many single CTAs
  unsigned global_k;   // > 1: ... by that many consecutive CTAs, partial tiles through scratch
};
UmmaPlan umma_plan(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count,
                   int elem_bytes, int force_pair, bool allow_cluster_k, bool allow_stream_k);
// Tiled fp32 tensor map of `rank` dimensions (dims[0] contiguous; strides_bytes[i] = pitch of
// dimension i+1) into *map, a CUtensorMap; swizzle_mode 0 = 128-byte swizzle of 16-byte units,
// 1 = of 32-byte units (MN-major 32-bit MMA operands).
bool encode_tmap_f32(void* map, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, int swizzle_mode);
int umma_sm_budget(int sm_count, unsigned max_ctas);  // SMs a launch may use (whole pairs)
bool stream_k_scratch_ok(const SgemmArgs& a, int sm_count);  // scratch lent for the k-shared wave
size_t umma_stream_k_workspace(int sm_count);  // scratch that lets umma_sgemm share tiles by k-block
void set_test_flag_wait(unsigned long long timeout_ns, unsigned expect_extra);
bool umma_sgemm_supported(const SgemmArgs& a);
int umma_sgemm(const SgemmArgs& a, bool pair);
bool umma_qgemm_supported(const QgemmArgs& a);
bool umma_qgemm_prefers_pair(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count);
int umma_qgemm(const QgemmArgs& a, bool pair);

// ---- CUDA-core paths (simt_kernels.cu) ----
int simt_sgemm(const SgemmArgs& a);
bool skinny_sgemm_supported(const SgemmArgs& a);
size_t skinny_sgemm_workspace(unsigned M, unsigned N, unsigned K, unsigned batch, int sm_count);
int skinny_sgemm(const SgemmArgs& a);
bool cluster_simt_sgemm_supported(const SgemmArgs& a);  // cluster_simt.cu: M <= 32, K <= 2048
int cluster_simt_sgemm(const SgemmArgs& a);
int skinny_sgemm_static(cudaStream_t stream, const float* A, const float* B, float* C,
                        const float* bias, unsigned M, unsigned N, unsigned K);
size_t skinny_sgemm_static_capacity();
int simt_qgemm(const QgemmArgs& a);
int convert_f32_to_bf16(cudaStream_t stream, const float* src, void* dst, size_t n);
// Scratch bytes of the bfloat16 mode: both operands rounded to bfloat16, each 256-byte aligned.
size_t bf16_staging_bytes(unsigned M, unsigned N, unsigned K, unsigned batch, unsigned strideA,
                          unsigned strideB);
int interleave_panels_f32(cudaStream_t stream, const float* src, float* out, unsigned M,
                          unsigned ns, unsigned G);
template <class T>
int reduce_sum(cudaStream_t stream, const T* src, unsigned batch, unsigned rows, unsigned cols,
               int row_flag, int32_t* dst);

// ---- multi-GPU shim (group.cu) ----
// One rank's view of an N-split product whose operands start in host memory.
// Side streams and events of one rank of the host-buffer N split: uploads, the exchange of A rows
// and downloads each run on a stream of their own beside the stream of the products.
constexpr unsigned kMaxHostBlocks = 16;
struct HostLanes {
  cudaStream_t up = nullptr, xch = nullptr, down = nullptr;
  cudaEvent_t start = nullptr;  // everything queued on the product stream before the call
  cudaEvent_t b_up = nullptr;   // the B shard is on the device
  cudaEvent_t tail = nullptr;   // the last download has finished
  cudaEvent_t a_up[kMaxHostBlocks] = {};     // row block p of A is on this device
  cudaEvent_t a_sent[kMaxHostBlocks] = {};   // ... and stored into every peer
  cudaEvent_t c_whole[kMaxHostBlocks] = {};  // row block p of C is whole on this device
  cudaError_t create();  // on the current device
  void join();           // waits for the three streams
  void destroy();
};

struct NsplitHostRank {
  cudaStream_t stream;
  HostLanes* lanes;
  const float* hA_rows;    // host: this rank's M / num_ranks rows of A
  const float* hB_shard;   // host: first element of this rank's column shard of B
  unsigned ldb_host;       // row pitch of hB_shard in elements
  float* hC_rows;          // host: this rank's M / num_ranks rows of the full-width C
  float* const* A_ranks;   // device: every rank's [M,K] staging (peers may be NULL = not written)
  float* A_multicast;      // NVLink multicast alias of the A buffers, or nullptr
  float* B_shard_dev;      // device: [K, N_shard]
  float* const* C_ranks;   // device: every rank's [M, N_shard * num_ranks] staging
  float* C_multicast;
  unsigned num_ranks, rank;
  unsigned M, N_shard, K;
  int precision;
  void* workspace;
  size_t workspace_bytes;
  int* status;
};
// The call runs in nsplit_host_blocks() row blocks; a caller drives all its ranks through
//   start(r);  for p in 0..blocks: { if p < blocks: before_barrier(r, p);  BARRIER;
//   after_barrier(r, p); }  finish(r)
// where BARRIER orders the ranks' product streams.
int nsplit_host_check(const NsplitHostRank& r);
unsigned nsplit_host_blocks(const NsplitHostRank& r);
int nsplit_host_start(const NsplitHostRank& r, unsigned blocks);
int nsplit_host_before_barrier(const NsplitHostRank& r, unsigned blocks, unsigned p);
int nsplit_host_after_barrier(const NsplitHostRank& r, unsigned blocks, unsigned p);

// ---- fused attention (attention.cu) ----
struct AttentionArgs {
  cudaStream_t stream;
  const float* q;  // element (b, s, h, d) at q + b*batch_stride + s*ld + h*dim + d; same for k, v
  const float* k;
  const float* v;
  float* out;      // element (b, s, h, d) at out + (b*seq + s)*ld_out + h*dim + d
  unsigned batch, seq, heads, dim;
  unsigned long long ld, batch_stride, ld_out;
  float scale;
  int* status;
};
bool attention_supported(const AttentionArgs& a);
int attention_f32(const AttentionArgs& a);

// ---- attention / FFN glue (nn_kernels.cu) ----
int softmax_f32(cudaStream_t stream, const float* src, unsigned rows, unsigned cols, float scale,
                float* dst);
int layer_norm_f32(cudaStream_t stream, const float* x, const float* residual, const float* gamma,
                   const float* beta, float eps, unsigned rows, unsigned cols, float* dst);
int gelu_f32(cudaStream_t stream, const float* src, size_t n, float* dst);
int permute_0213_f32(cudaStream_t stream, const float* src, unsigned d0, unsigned d1, unsigned d2,
                     unsigned d3, float* dst);
int transpose_last2_f32(cudaStream_t stream, const float* src, unsigned batch, unsigned r,
                        unsigned c, float* dst);

// ---- quantize / dequantize / requantize (quantize_kernels.cu) ----
int minmax_f32(cudaStream_t stream, const float* src, size_t n, float* out);
int quantize_f32(cudaStream_t stream, const float* src, size_t n, const float* pmin,
                 const float* pmax, void* dst, int dst_type);
int quantized_matmul_params_dev(cudaStream_t stream, const float* minA, const float* maxA,
                                const float* minB, const float* maxB, int32_t* offsets,
                                float* minC, float* maxC);
int quantize_rows_f32(cudaStream_t stream, const float* src, unsigned rows, unsigned cols,
                      const float* pmin, const float* pmax, void* dst, int dst_type,
                      int32_t* row_sums);
int dequantize_f32(cudaStream_t stream, const void* src, int src_type, size_t n, const float* pmin,
                   const float* pmax, float* dst);
int requantize(cudaStream_t stream, const void* src, int src_type, size_t n, const float* pmin_in,
               const float* pmax_in, const float* pmin_out, const float* pmax_out, void* dst,
               int dst_type);

}  // namespace tfccb200
