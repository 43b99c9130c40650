/*
 * tfcc_b200.h -- C ABI of the B200 (sm_100a) matmul kernel library for TFCC.
 *
 * Every entry point is `extern "C"`, never throws, never exits the process and
 * returns an int status: 0 on success, a negative TFCCB200_E* code for an
 * argument problem detected on the host, or a positive cudaError_t value for a
 * CUDA runtime failure.  Device buffers are plain pointers; all matrices are
 * contiguous row-major, exactly as TFCC tensors are
 * (tfcc/core/framework/tfcc_tensor.h:26-56).  Strides between consecutive
 * batch entries are counted in ELEMENTS and a stride of 0 broadcasts a single
 * matrix over the batch, which is how the reference backends receive a rank-2
 * operand next to a batched one
 * (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-151,
 *  tfcc/cuda/interfaces/tfcc_cudablasinterface.cu:201-217).
 *
 * Launches are asynchronous on the given stream; nothing here synchronises
 * unless the comment of the function says so.  Entry points are re-entrant
 * across host threads and streams.  State the library keeps per process:
 * per-device caches of immutable facts (SM count, driver entry point for
 * tensor-map encoding, occupancy of cluster launches); a stream-ordered memory
 * pool of its own per device, used only by the *_host entry points for their
 * staging buffers (the device's default pool is never touched); the 20 MiB
 * device array behind tfccb200_sgemm_skinny_static, shared by all calls of that
 * one entry point; the launch counter; the device groups created by
 * tfccb200_group_create.
 *
 * Scratch memory ("workspace") passed to an entry point belongs to that call
 * until the call's kernels have finished: two calls that can run on the GPU at
 * the same time (different streams) must be given different workspaces.
 */
#ifndef TFCC_B200_H_
#define TFCC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported from the shared library even when it is built with hidden default visibility. */
#define TFCCB200_API __attribute__((visibility("default")))

/* ---- status codes ------------------------------------------------------- */
#define TFCCB200_OK 0
#define TFCCB200_EINVAL -1      /* NULL pointer, zero extent, bad enum value          */
#define TFCCB200_EALIGN -2      /* a forced kernel path needs an alignment not met     */
#define TFCCB200_EWORKSPACE -3  /* workspace too small for the chosen kernel           */
#define TFCCB200_EOVERFLOW -4   /* an element count does not fit the 32-bit TFCC Shape */
#define TFCCB200_EUNSUPPORTED -5/* forced kernel path cannot run this problem          */
#define TFCCB200_EDEVICE -6     /* a kernel gave up a bounded wait (see device_status) */
#define TFCCB200_ESTATICLIMIT -7 /* tfccb200_sgemm_skinny_static: built-in scratch too small  */

/* ---- precision modes of the fp32 GEMM ----------------------------------- */
/* FP32:  fp32 result.  Tensor-core tiles split every operand into a TF32 head
 *        and a TF32 tail and issue three MMAs (head*head, head*tail,
 *        tail*head); CUDA-core paths use fp32 FMA.  Normwise relative error
 *        against an fp64 product stays below 1e-5.
 * TF32:  one MMA per tile on the TF32 heads only (about 1e-3 relative).
 * BF16:  operands rounded to bfloat16 by a pre-pass into the caller's workspace, bfloat16
 *        tensor-core products, fp32 accumulation (about 4e-3 relative).  Needs K % 8 == 0
 *        and N % 8 == 0; other shapes are computed as FP32.
 * All modes read and write fp32 buffers. */
#define TFCCB200_PRECISION_FP32 0
#define TFCCB200_PRECISION_TF32 1
#define TFCCB200_PRECISION_BF16 2

/* ---- kernel paths (for tests and benchmarks; AUTO is what TFCC uses) ----- */
#define TFCCB200_PATH_AUTO 0
#define TFCCB200_PATH_SIMT 1    /* CUDA-core tiled kernel, any shape / alignment          */
#define TFCCB200_PATH_SKINNY 2  /* streaming kernel for few rows (M <= 32; AUTO: M <= 16 and a B too large for path 5) */
#define TFCCB200_PATH_UMMA 3    /* tcgen05 + TMEM + TMA, one CTA per tile                  */
#define TFCCB200_PATH_UMMA2 4   /* tcgen05 cta_group::2, a pair of CTAs per 256-row tile    */
#define TFCCB200_PATH_CLUSTER_SIMT 5 /* M <= 32, K <= 2048: CUDA cores, one launch, K split over a cluster (AUTO: B up to 16 MB) */

/* Bits a kernel ORs into *device_status when it abandons a bounded wait.     */
#define TFCCB200_DEV_TIMEOUT_TMA 0x1
#define TFCCB200_DEV_TIMEOUT_MMA 0x2
#define TFCCB200_DEV_TIMEOUT_CONVERT 0x4
#define TFCCB200_DEV_TIMEOUT_EPILOGUE 0x8

TFCCB200_API const char* tfccb200_strerror(int status);

/* Library version as major*10000 + minor*100 + patch. */
TFCCB200_API int tfccb200_version(void);

/*
 * C[b] = A[b] . B[b] (+ bias), fp32, b in [0, batch).
 *   A: [M,K], B: [K,N], C: [M,N], bias: [N] or NULL.
 * Replaces CUDABlasInterface<float>::matmul(a,b) and matmul(a,b,c)
 * (tfcc/cuda/interfaces/tfcc_cudablasinterface.cu:201-248, :251-303) and the
 * oneDNN calls of MKLBlasInterface<float>
 * (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:41-67, :87-118).  The bias is
 * added in the epilogue, so C is written once instead of being pre-filled and
 * accumulated into.
 *
 * Non-finite inputs: NaN propagates as NaN on every path.  On the tensor-core paths an
 * infinite element makes its whole output row (column) NaN where IEEE arithmetic would give
 * +-inf, because the fp32 product is rebuilt from head and tail parts and inf has no tail
 * (inf - inf); the CUDA-core paths (few rows: M <= 16, or M <= 32 against a small B; unaligned
 * shapes) follow IEEE.  The reference's own tests feed finite values only.
 *
 * workspace / workspace_bytes: scratch in device memory of at least
 * tfccb200_sgemm_workspace() bytes (may be NULL when that returns 0).
 * device_status: optional int in device memory; kernels OR a TFCCB200_DEV_*
 * bit into it if a bounded wait runs out.  May be NULL.
 */
TFCCB200_API int tfccb200_sgemm(void* stream, const float* A, unsigned strideA, const float* B,
                   unsigned strideB, float* C, unsigned strideC, const float* bias, unsigned M,
                   unsigned N, unsigned K, unsigned batch, int precision_mode, void* workspace,
                   size_t workspace_bytes, int* device_status);

/* Same, with the kernel path forced (TFCCB200_PATH_*).  Used by the parity
 * tests to exercise every kernel on every shape it accepts. */
TFCCB200_API int tfccb200_sgemm_ex(void* stream, const float* A, unsigned strideA, const float* B,
                      unsigned strideB, float* C, unsigned strideC, const float* bias, unsigned M,
                      unsigned N, unsigned K, unsigned batch, int precision_mode, int path,
                      void* workspace, size_t workspace_bytes, int* device_status);

/* Scratch bytes tfccb200_sgemm wants for this problem on the current device.  The few-row
 * streaming kernel (M <= 16) and the bf16 mode cannot run without theirs; the fp32 tensor-core kernel
 * runs without but uses its share (partial tiles of a ragged last wave) when given. */
TFCCB200_API size_t tfccb200_sgemm_workspace(unsigned M, unsigned N, unsigned K, unsigned batch,
                                int precision_mode);

/* Which TFCCB200_PATH_* tfccb200_sgemm would take (pointers assumed 16-byte
 * aligned, as TFCC's allocators guarantee). */
TFCCB200_API int tfccb200_sgemm_path(unsigned M, unsigned N, unsigned K, unsigned batch, unsigned strideA,
                        unsigned strideB, int precision_mode);

/*
 * Quantized matmul, u8 x s8 -> s32 with the zero-point correction fused into
 * the epilogue:
 *   C[b][i][j] = sum_k A[b][i][k]*B[b][k][j]
 *              + offA*offB*K + rsA[b][i]*offB + rsB[b][j]*offA      (int32, wraps)
 * which equals sum_k (A+offA)(B+offB) when rsA / rsB are the row sums of A and
 * column sums of B.  Replaces the two queued tasks of
 * tfcc::mkl::quantization::matmul -- _mkl_create_offset_matrix followed by the
 * accumulating AVX2 GEMM (tfcc/mkl/operations/tfcc_mklquantization.cpp:33-69,
 * :176-201) -- and its N==1 fast path (:151-174).
 * strideRsA / strideRsB are 0 when the sums are shared by the whole batch.
 */
TFCCB200_API int tfccb200_qgemm_u8s8s32(void* stream, const uint8_t* A, unsigned strideA, const int32_t* rsA,
                           unsigned strideRsA, int32_t offA, const int8_t* B, unsigned strideB,
                           const int32_t* rsB, unsigned strideRsB, int32_t offB, int32_t* C,
                           unsigned strideC, unsigned M, unsigned N, unsigned K, unsigned batch,
                           int* device_status);

TFCCB200_API int tfccb200_qgemm_u8s8s32_ex(void* stream, const uint8_t* A, unsigned strideA,
                              const int32_t* rsA, unsigned strideRsA, int32_t offA,
                              const int8_t* B, unsigned strideB, const int32_t* rsB,
                              unsigned strideRsB, int32_t offB, int32_t* C, unsigned strideC,
                              unsigned M, unsigned N, unsigned K, unsigned batch, int path,
                              int* device_status);

/*
 * The quantized matmul with the operand ranges in DEVICE memory, which is where TFCC keeps them
 * (Tensor<float> of one element each, tfcc/mkl/operations/tfcc_mklquantization.h:39-45): a
 * one-thread prologue kernel derives the zero-point offsets and the float range of the result
 * with the reference's double / float formulas (tfcc/mkl/operations/tfcc_mklquantization.cpp:
 * 181-193) and the GEMM reads the offsets from device memory, so nothing returns to the host and
 * nothing synchronises.  minA .. maxB: one float each (read); minC, maxC: one float each
 * (written); offsets: two int32 of scratch that receive {offA, offB}.  `path` is a
 * TFCCB200_PATH_* (AUTO for normal use).  Results equal tfccb200_qgemm_u8s8s32 fed by
 * tfccb200_quantized_matmul_params.
 */
TFCCB200_API int tfccb200_qgemm_u8s8s32_dev(void* stream, const uint8_t* A, unsigned strideA,
                                            const int32_t* rsA, unsigned strideRsA,
                                            const float* minA, const float* maxA, const int8_t* B,
                                            unsigned strideB, const int32_t* rsB,
                                            unsigned strideRsB, const float* minB,
                                            const float* maxB, int32_t* C, unsigned strideC,
                                            float* minC, float* maxC, int32_t* offsets, unsigned M,
                                            unsigned N, unsigned K, unsigned batch, int path,
                                            int* device_status);

/*
 * Host-side scalar math of the quantized matmul: zero-point offsets and the
 * float range of the int32 result, from the (min,max) float ranges of the
 * operands.  Restates get_quantized_scale_info<uint8_t/int8_t> minus
 * numeric_limits::lowest() and get_quantization_range_for_multiplication
 * (tfcc/core/utils/tfcc_quantizationutils.h:23-56,
 *  tfcc/mkl/operations/tfcc_mklquantization.cpp:181-193).
 */
TFCCB200_API int tfccb200_quantized_matmul_params(float minA, float maxA, float minB, float maxB,
                                     int32_t* offA, int32_t* offB, float* minC, float* maxC);

/*
 * dst = sum of src over its last dimension (row_flag != 0, dst is
 * [batch,rows]) or over its second-to-last dimension (row_flag == 0, dst is
 * [batch,cols]); src is [batch,rows,cols].  int32 accumulation.  Replaces
 * tfcc::mkl::quantization::reduce_sum<T>
 * (tfcc/mkl/operations/tfcc_mklquantization.cpp:205-318).
 */
TFCCB200_API int tfccb200_reduce_sum_u8(void* stream, const uint8_t* src, unsigned batch, unsigned rows,
                           unsigned cols, int row_flag, int32_t* dst);
TFCCB200_API int tfccb200_reduce_sum_s8(void* stream, const int8_t* src, unsigned batch, unsigned rows,
                           unsigned cols, int row_flag, int32_t* dst);
TFCCB200_API int tfccb200_reduce_sum_s16(void* stream, const int16_t* src, unsigned batch, unsigned rows,
                            unsigned cols, int row_flag, int32_t* dst);

/* ---- activations that the fp32 GEMM can apply in its epilogue ----------------- */
#define TFCCB200_ACT_NONE 0
#define TFCCB200_ACT_GELU_ERF 1 /* 0.5 x (1 + erf(x / sqrt 2)), the reference's gelu_accurate */

/*
 * tfccb200_sgemm_ex with an activation applied to A.B + bias while the result leaves the
 * accumulator: MatmulWithBias followed by Gelu (the FFN of a transformer block) in one pass
 * over C.  The reference runs them as two operators
 * (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:154-186 then
 *  _MKLActivationKernel::geluAccurate, tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:214-220).
 */
TFCCB200_API int tfccb200_sgemm_act(void* stream, const float* A, unsigned strideA,
                                    const float* B, unsigned strideB, float* C, unsigned strideC,
                                    const float* bias, unsigned M, unsigned N, unsigned K,
                                    unsigned batch, int precision_mode, int path, int activation,
                                    void* workspace, size_t workspace_bytes, int* device_status);

/*
 * dst[r][:] = softmax(scale * src[r][:]) over the last dimension (max subtraction, exp, sum,
 * divide: _MKLActivationKernel::softmaxV2, tfcc/mkl/kernel/tfcc_mklactivationkernel.hpp:138-155;
 * cf. _cuda_softmax_v1_small, tfcc/cuda/interfaces/tfcc_cudaactivationinterface.cu:96-121).
 * The pre-scale folds the separate "x / sqrt(d)" operator of an attention block into the pass.
 */
TFCCB200_API int tfccb200_softmax_f32(void* stream, const float* src, unsigned rows,
                                      unsigned cols, float scale, float* dst);

/*
 * Scaled dot-product attention of one transformer block in one kernel, one CTA per
 * (batch, head):  out = softmax(scale * Q . K^T) . V  with fp32 results (tensor-core products
 * by three TF32 MMAs, softmax as tfccb200_softmax_f32).
 *   q, k, v: element (b, s, h, d) at  base + (b*seq + s)*ld_qkv + h*dim + d  -- the layout the
 *            Q/K/V projections produce ([batch, seq, heads*dim] matrices, or slices of one packed
 *            [batch, seq, 3*heads*dim] matrix: pass the three slice bases and ld_qkv = 3*heads*dim);
 *   out:     element (b, s, h, d) at  out + (b*seq + s)*ld_out + h*dim + d.
 * It stands for this sequence of reference operators: transpose of q, k, v to
 * [batch, head, seq, dim], transpose of k's last two axes, batched matmul, scale, softmax,
 * batched matmul, transpose back (tfcc/cuda/interfaces/tfcc_cudabasicinterface.cu:83-100,
 * tfcc/cuda/interfaces/tfcc_cudaactivationinterface.cu:96-121,
 * tfcc/cuda/interfaces/tfcc_cudablasinterface.cu:201-248); none of the permutations is a pass
 * over memory here, K is read as a K-major operand.
 * Limits: seq <= 128, dim 32 or 64, 16-byte aligned bases, ld % 4 == 0; anything else returns
 * TFCCB200_EUNSUPPORTED and the caller composes the separate operators.
 */
TFCCB200_API int tfccb200_attention_f32(void* stream, const float* q, const float* k,
                                        const float* v, float* out, unsigned batch, unsigned seq,
                                        unsigned heads, unsigned dim, unsigned ld_qkv,
                                        unsigned ld_out, float scale, int* device_status);

/*
 * dst = (t - mean(t)) / sqrt(var(t) + eps) * gamma + beta with t = x (+ residual when not
 * NULL), row by row, two-pass mean and variance (_mkl_layer_normalize,
 * tfcc/mkl/interfaces/tfcc_mklnormalizationinterface.cpp:29-62).  Rows of up to 1024 columns
 * are held in registers by one warp; longer rows take one CTA each and three passes (cf.
 * _cuda_layer_normalize_large, tfcc/cuda/interfaces/tfcc_cudanormalizationinterface.cu:85).
 */
TFCCB200_API int tfccb200_layer_norm_f32(void* stream, const float* x, const float* residual,
                                         const float* gamma, const float* beta, float eps,
                                         unsigned rows, unsigned cols, float* dst);

/* dst[i] = gelu_accurate(src[i]) (erf form). */
TFCCB200_API int tfccb200_gelu_f32(void* stream, const float* src, size_t n, float* dst);

/* [d0,d1,d2,d3] -> [d0,d2,d1,d3] (split / merge attention heads) and [batch,r,c] ->
 * [batch,c,r] (K transposed); the index maps of _cuda_transpose_4d / _3d
 * (tfcc/cuda/interfaces/tfcc_cudabasicinterface.cu:66-100) for these two permutations. */
TFCCB200_API int tfccb200_permute_0213_f32(void* stream, const float* src, unsigned d0,
                                           unsigned d1, unsigned d2, unsigned d3, float* dst);
TFCCB200_API int tfccb200_transpose_last2_f32(void* stream, const float* src, unsigned batch,
                                              unsigned r, unsigned c, float* dst);

/* ---- element types of the quantization entry points ------------------------ */
#define TFCCB200_TYPE_S8 0
#define TFCCB200_TYPE_U8 1
#define TFCCB200_TYPE_S16 2
#define TFCCB200_TYPE_U16 3
#define TFCCB200_TYPE_S32 4
#define TFCCB200_TYPE_U32 5

/*
 * minmax[0] = min(src), minmax[1] = max(src) over n floats; minmax is DEVICE memory (two
 * floats, 8-byte aligned).  The range reduction of MKLQuantizationInterface<T>::quantize(a)
 * (tfcc/mkl/interfaces/tfcc_mklquantizationinterface.cpp:47-57).
 */
TFCCB200_API int tfccb200_minmax_f32(void* stream, const float* src, size_t n, float* minmax);

/*
 * dst[i] = clamp(round(src[i] * scale) - offset + lowest(T)), scale and offset derived in
 * double precision from the DEVICE scalars *min_value, *max_value; everything becomes
 * lowest(T) when *min_value >= *max_value.  dst_type is a TFCCB200_TYPE_*.  Replaces
 * MKLQuantizationInterface<T>::quantize (tfcc_mklquantizationinterface.cpp:150-240) and
 * _MKLQuantizationKernel<T>::quantize (tfcc/mkl/kernel/tfcc_mklquantizationkernel.hpp:23-33).
 */
TFCCB200_API int tfccb200_quantize_f32(void* stream, const float* src, size_t n,
                                       const float* min_value, const float* max_value, void* dst,
                                       int dst_type);

/*
 * tfccb200_quantize_f32 on a [rows, cols] matrix together with reduce_sum(dst, row): row_sums[r]
 * receives the int32 sum of the quantized values of row r, produced in the same pass, so that
 * the sequence quantize -> reduce_sum -> matmul of a quantized dense layer
 * (tfcc/test/quantization.cpp:105-121;
 *  tfcc/mkl/interfaces/tfcc_mklquantizationinterface.cpp:150-189 then
 *  tfcc/mkl/operations/tfcc_mklquantization.cpp:205-237) reads the activations once.
 * dst_type is TFCCB200_TYPE_S8, _U8 or _S16 (the types reduce_sum exists for).  Results are
 * identical to the two separate calls.
 */
TFCCB200_API int tfccb200_quantize_rowsum_f32(void* stream, const float* src, unsigned rows,
                                              unsigned cols, const float* min_value,
                                              const float* max_value, void* dst, int dst_type,
                                              int32_t* row_sums);

/*
 * dst[i] = float(min + (src[i] - lowest(T)) * scale); *min_value when the range is empty.
 * Replaces MKLQuantizationInterface<T>::dequantize (tfcc_mklquantizationinterface.cpp:284-333).
 */
TFCCB200_API int tfccb200_dequantize_f32(void* stream, const void* src, int src_type, size_t n,
                                         const float* min_value, const float* max_value,
                                         float* dst);

/*
 * Re-express quantized values of one type and range in another type and range.  Replaces
 * _requantize_helper<TO,TI> (tfcc_mklquantizationinterface.cpp:71-147).
 */
TFCCB200_API int tfccb200_requantize(void* stream, const void* src, int src_type, size_t n,
                                     const float* min_input, const float* max_input,
                                     const float* min_output, const float* max_output, void* dst,
                                     int dst_type);

/*
 * C = A . B (+ bias) for M <= 8, single matrices, fp32 -- the decode / GEMV shape -- for
 * callers that have no device memory to lend.  This entry point has no counterpart in the
 * reference.
 *
 * Who needs it: an embedder that hands all of HBM to its own arena at start-up and runs with
 * device allocation switched off afterwards, or a serving thread on which cudaMalloc is banned
 * because it stalls every stream of the device.  Such a caller cannot allocate the workspace
 * that tfccb200_sgemm wants for this shape and cannot let the library allocate it either.
 * Here the per-slice partial sums go to a 20 MiB array that is part of the library's device
 * image, so the call allocates nothing: no cudaMalloc, no cudaFree, no pool.
 *
 * Limits and rules:
 *  - the problem's scratch need -- tfccb200_sgemm_skinny_static_need(M, N, K) bytes: one
 *    M x N fp32 partial result per K slice, the slice count chosen for the current device --
 *    must fit tfccb200_sgemm_skinny_static_capacity() bytes, else TFCCB200_ESTATICLIMIT; M = 8,
 *    K = 4096, N = 16384 needs 9 MiB on a 148-SM part.  (tfccb200_sgemm_workspace may report
 *    more for the same shape: it also covers what other kernel paths would like to borrow.)
 *    N % 4 == 0 and 16-byte aligned B, C, bias are required as for the workspace form
 *    (TFCCB200_EUNSUPPORTED otherwise);
 *  - the first call on each device looks up the array's device address (a one-time host-side
 *    set-up); make that first call before starting any stream capture;
 *  - the array is shared by every call on the device and is never cleared -- no call reads
 *    what it has not written itself -- so calls must not overlap on the GPU: issue them on
 *    one stream, or order the streams yourself.  Overlapping calls race on the array;
 *  - every process that loads the library holds the 20 MiB on each GPU it uses, until exit.
 * The result is bit-identical to tfccb200_sgemm on the same problem.
 */
TFCCB200_API int tfccb200_sgemm_skinny_static(void* stream, const float* A, const float* B,
                                              float* C, const float* bias, unsigned M,
                                              unsigned N, unsigned K);
TFCCB200_API size_t tfccb200_sgemm_skinny_static_capacity(void);
/* Scratch bytes the call above would use for this problem on the current device (0 for
 * M > 8 or an empty problem). */
TFCCB200_API size_t tfccb200_sgemm_skinny_static_need(unsigned M, unsigned N, unsigned K);

/*
 * N-split GEMM with the all-gather fused into the epilogue.  Rank `rank` of `num_ranks`
 * GPUs holds A [M,K] and the column shard B_shard [K, N_shard] of B; it computes
 * A . B_shard (+ bias_shard) on the tensor-core path and stores the tile results directly
 * into columns [rank*N_shard, (rank+1)*N_shard) of EVERY rank's row-major
 * C [M, num_ranks*N_shard]: C_ranks is a HOST array of num_ranks device pointers, entry r
 * being rank r's C mapped into this process (peer access / symmetric memory).  Remote rows
 * are written with ordinary 128-byte-line stores over NVLink while the remaining tiles are
 * still being multiplied; no TMA or multicast instruction touches peer memory.  When the
 * kernel has finished on every rank (the caller runs a cross-rank barrier after it), each
 * rank holds the complete C.  Needs K % 4 == 0, N_shard % 4 == 0, 16-byte aligned bases.
 * `C_multicast` (may be NULL) is the address of the same C through an NVLink multicast object
 * that every rank's C is bound to (NVLS; torch symmetric memory's multicast_ptr): when given,
 * each line is stored once with multimem.st and the switch replicates it to all ranks, so a
 * GPU sends its shard once instead of num_ranks - 1 times; C_ranks is then only checked.
 * `workspace` (256-byte aligned, tfccb200_sgemm_workspace(M, N_shard, K, 1, mode) bytes, may be
 * NULL) lets the kernel share the tiles of a ragged last wave by k-block; the result is
 * the same bit for bit with or without it.
 * No counterpart in the reference, which has no multi-device operator.
 */
TFCCB200_API int tfccb200_sgemm_nsplit_push(void* stream, const float* A, const float* B_shard,
                                            float* const* C_ranks, unsigned num_ranks,
                                            unsigned rank, const float* bias_shard, unsigned M,
                                            unsigned N_shard, unsigned K, int precision_mode,
                                            float* C_multicast, void* workspace,
                                            size_t workspace_bytes, int* device_status);

/* Same, with two more controls.  An entry of C_ranks other than C_ranks[rank] may be NULL: that
 * rank's copy is then not written by this call.  max_ctas > 0 limits the launch to that many
 * SMs (rounded down to whole CTA pairs), so that two products -- for instance two steps of a
 * pipeline, each with its own C and workspace, on two streams -- can run side by side on
 * disjoint parts of the chip: the pushes of one then overlap the arithmetic of the other. */
TFCCB200_API int tfccb200_sgemm_nsplit_push_ex(void* stream, const float* A, const float* B_shard,
                                               float* const* C_ranks, unsigned num_ranks,
                                               unsigned rank, const float* bias_shard, unsigned M,
                                               unsigned N_shard, unsigned K, int precision_mode,
                                               float* C_multicast, void* workspace,
                                               size_t workspace_bytes, unsigned max_ctas,
                                               int* device_status);

/*
 * The quantized matmul of tfccb200_qgemm_u8s8s32 (single matrices) with the same fused gather:
 * rank `rank` holds A [M,K] with its row sums, the column shard B_shard [K,N_shard] with that
 * shard's column sums, and stores its int32 tiles, zero-point correction applied, into columns
 * [rank*N_shard, (rank+1)*N_shard) of every non-NULL C_ranks[r] ([M, num_ranks*N_shard]
 * row-major), or once through C_multicast.  Integer results do not depend on the split, so the
 * assembled C equals the single-GPU result bit for bit.  Needs K % 16 == 0, N_shard % 16 == 0,
 * K >= 128, N_shard >= 128 (tensor-core path only).  No counterpart in the reference.
 */
TFCCB200_API int tfccb200_qgemm_nsplit_push(void* stream, const uint8_t* A, const int32_t* rsA,
                                            int32_t offA, const int8_t* B_shard,
                                            const int32_t* rsB_shard, int32_t offB,
                                            int32_t* const* C_ranks, unsigned num_ranks,
                                            unsigned rank, unsigned M, unsigned N_shard,
                                            unsigned K, int32_t* C_multicast, int* device_status);

/*
 * Cross-rank barrier supplied by a one-process-per-GPU caller: must enqueue on `stream` a
 * barrier behind which everything the other ranks enqueued before their own matching call has
 * completed (e.g. a symmetric-memory barrier kernel, or a tiny NCCL all-reduce).  Returns 0 or
 * a status that the entry point hands back unchanged.
 */
typedef int (*tfccb200_barrier_fn)(void* ctx, void* stream);

/*
 * One rank's share of an N-split product whose operands start in HOST memory and whose result
 * returns to host memory -- the data::set -> matmul -> data::get round trip
 * (tfcc/cuda/interfaces/tfcc_cudadatainterface.cu:62-90) spread over num_ranks GPUs so that the
 * job's host traffic crosses num_ranks PCIe links once instead of every link carrying all of it:
 *   1. rank r uploads rows [r*M/G, (r+1)*M/G) of A (hA_rows) into its own A staging and stores
 *      them on into every peer's A staging over NVLink, and uploads its column shard of B
 *      (hB_shard, row pitch ldb_host elements) into B_shard_dev;
 *   2. barrier; tfccb200_sgemm_nsplit_push; barrier;
 *   3. rank r downloads rows [r*M/G, (r+1)*M/G) of the assembled C into hC_rows
 *      ([M/G, num_ranks*N_shard]).
 * The three run as a pipeline over row blocks of about 256 rows per rank (at most 16 blocks;
 * TFCCB200_HOST_BLOCKS in the environment overrides the count): step p multiplies block p of
 * every rank while later blocks are still being uploaded and exchanged and earlier ones are
 * being downloaded, on three side streams that the calling thread keeps per device; `barrier`
 * is called blocks + 1 times, always on `stream`.
 * Per rank 4 (M K / G + K N_shard) bytes go up and 4 M N / G come down.  A_ranks / C_ranks are
 * every rank's device staging buffers mapped into this process ([M,K] and
 * [M, num_ranks*N_shard] floats; the call orders rows inside them block by block, so their
 * content afterwards is not the row-major A or C); A_multicast / C_multicast their NVLink
 * multicast aliases or NULL.  M % num_ranks == 0, K % 4 == 0, N_shard % 4 == 0.  Host buffers
 * should be pinned.  Every rank must make the call with the same shapes.  Synchronises `stream`
 * and the side streams before returning, also on an error; *device_status is left for the
 * caller to read.  `barrier` may be NULL when num_ranks == 1.  No counterpart in the reference.
 */
TFCCB200_API int tfccb200_sgemm_nsplit_host(void* stream, const float* hA_rows,
                                            const float* hB_shard, unsigned ldb_host,
                                            float* hC_rows, float* const* A_ranks,
                                            float* A_multicast, float* B_shard_dev,
                                            float* const* C_ranks, float* C_multicast,
                                            unsigned num_ranks, unsigned rank, unsigned M,
                                            unsigned N_shard, unsigned K, int precision_mode,
                                            void* workspace, size_t workspace_bytes,
                                            tfccb200_barrier_fn barrier, void* barrier_ctx,
                                            int* device_status);

/*
 * Device group for a process that drives several GPUs itself -- the shape of a TFCC program
 * with one Device per GPU (tfcc/core/utils/tfcc_initializer.cpp:50-66,
 * tfcc/cuda/utils/tfcc_cudautils.cpp:23-50).  Creating a group enables peer access between
 * every pair of its devices and gives each member a stream, a device status word and scratch
 * for the tensor-core kernel; members are ordered against each other with CUDA events, never
 * by blocking the host.  The calls below may be made from any one host thread at a time and
 * restore the caller's current device.  `devices` may name the same GPU more than once (the
 * members then share it; useful for exercising the multi-rank logic on one GPU).
 */
typedef struct tfccb200_group tfccb200_group;
TFCCB200_API int tfccb200_group_create(int ndev, const int* devices, tfccb200_group** out);
TFCCB200_API int tfccb200_group_destroy(tfccb200_group* group);
TFCCB200_API int tfccb200_group_size(const tfccb200_group* group);
TFCCB200_API int tfccb200_group_device(const tfccb200_group* group, int member);
TFCCB200_API void* tfccb200_group_stream(const tfccb200_group* group, int member);
/* Waits for every member's stream; TFCCB200_EDEVICE if a kernel abandoned a bounded wait. */
TFCCB200_API int tfccb200_group_sync(tfccb200_group* group);

/*
 * N-split product on device-resident operands: arrays of one pointer per member, A[i] [M,K] and
 * B_shards[i] [K,N_shard] on member i's device, C[i] that member's full [M, G*N_shard].  Each
 * member's kernel is queued on its group stream; when the call returns nothing has been waited
 * for, and work queued later on any member's group stream sees the complete C.
 */
TFCCB200_API int tfccb200_group_sgemm_nsplit(tfccb200_group* group, const float* const* A,
                                             const float* const* B_shards, float* const* C,
                                             const float* const* bias_shards, unsigned M,
                                             unsigned N_shard, unsigned K, int precision_mode);
TFCCB200_API int tfccb200_group_qgemm_nsplit(tfccb200_group* group, const uint8_t* const* A,
                                             const int32_t* const* rsA, int32_t offA,
                                             const int8_t* const* B_shards,
                                             const int32_t* const* rsB_shards, int32_t offB,
                                             int32_t* const* C, unsigned M, unsigned N_shard,
                                             unsigned K);
/*
 * C = A . B with all three matrices in host memory (row-major [M,K], [K,N], [M,N]; pinned for
 * the copies to overlap), N split over the group: every member uploads M/G rows of A and its
 * column shard of B, the rows are exchanged over NVLink, and every member downloads M/G rows of
 * the assembled C.  M and N must be multiples of the group size, K and N/G of 4.  Staging
 * buffers belong to the group and are kept between calls.  Synchronous.
 */
TFCCB200_API int tfccb200_group_sgemm_nsplit_host(tfccb200_group* group, const float* hA,
                                                  const float* hB, float* hC, unsigned M,
                                                  unsigned N, unsigned K, int precision_mode);

/*
 * dst[m][g*ns + j] = src[g][m][j] for g < G, m < M, j < ns (fp32, ns % 4 == 0).
 * Turns the rank-major result of an all-gather of column shards of C into the
 * row-major [M, G*ns] matrix.  No counterpart in the reference, which has no
 * multi-device operator; used by the N-split multi-GPU shim.
 */
TFCCB200_API int tfccb200_interleave_panels_f32(void* stream, const float* src, float* dst,
                                                unsigned M, unsigned ns, unsigned G);

/*
 * Host-buffer forms: the caller passes HOST pointers; the call stages the
 * operands in device memory, runs the device entry point above on `stream`,
 * copies the result back and synchronises the stream before returning.  This
 * is the data::set -> matmul -> data::get round trip of a TFCC user
 * (tfcc/cuda/interfaces/tfcc_cudadatainterface.cu:62-90) in one call.
 * Device staging buffers come from the stream-ordered CUDA allocator.
 */
TFCCB200_API int tfccb200_sgemm_host(void* stream, const float* hA, unsigned strideA, const float* hB,
                        unsigned strideB, float* hC, unsigned strideC, const float* hbias,
                        unsigned M, unsigned N, unsigned K, unsigned batch, int precision_mode);

TFCCB200_API int tfccb200_qgemm_u8s8s32_host(void* stream, const uint8_t* hA, unsigned strideA,
                                const int8_t* hB, unsigned strideB, float minA, float maxA,
                                float minB, float maxB, int32_t* hC, unsigned strideC,
                                float* minC, float* maxC, unsigned M, unsigned N, unsigned K,
                                unsigned batch);

/*
 * Test hook for the give-up path of the fp32 tensor-core kernel.  CTAs that share a tile's
 * k-blocks through scratch wait, with a time limit, on counters that other CTAs of the same
 * launch raise; when a wait runs out the kernel ORs TFCCB200_DEV_TIMEOUT_EPILOGUE into
 * *device_status, every role of the CTA stops waiting, and the kernel runs to its normal end
 * (tensor memory freed, context intact) with an undefined C.  This call changes, for every later
 * launch of the process, the limit of those waits (nanoseconds; 0 = the normal 2 s) and makes
 * them expect `expect_extra` more arrivals than a launch ever delivers (0 = normal), so that a
 * test can see the status word and the orderly return without anything having to hang:
 * tfccb200_test_flag_wait(1000000, 1) before the launch, tfccb200_test_flag_wait(0, 0) after.
 * Not for production use.  No counterpart in the reference.
 */
TFCCB200_API void tfccb200_test_flag_wait(unsigned long long timeout_ns, unsigned expect_extra);

/* Number of kernels this library has launched in the calling process since it
 * was loaded (monotonic; for benchmarks that must report their launch count). */
TFCCB200_API unsigned long long tfccb200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TFCC_B200_H_ */
