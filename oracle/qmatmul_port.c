/*
 * TEST INFRASTRUCTURE -- CPU restatement of the reference's quantized matmul
 * path in plain C.  It exists to check the CUDA library and to serve as the
 * timed CPU baseline; nothing shipped links or calls it.
 *
 * Each function names the reference code it follows (paths relative to the
 * reference tree).  The arithmetic is all-integer with int32 wrap-around, so
 * any correct evaluation order gives bit-identical results.
 *
 * Parity pin: checked against the reference's own golden expectations
 * (tfcc/test/quantization.cpp:105-218 with data from
 * tfcc/test/python/testcase/quantization/mklquantizationmatmul.py) and against
 * the reference's AVX2 kernel compiled from its sources (oracle/_ref).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

/* get_quantized_scale_info<T> for an 8-bit T
 * (tfcc/core/utils/tfcc_quantizationutils.h:45-56): scale and offset in double. */
static void scale_info_8bit(float min_value, float max_value, double* scale, int64_t* offset) {
  const int64_t step_cnt = (int64_t)1 << 8;
  double range_adjust = step_cnt / (step_cnt - 1.0);
  double range = (max_value - min_value) * range_adjust;
  double range_scale = step_cnt / range;
  *scale = range_scale;
  *offset = (int64_t)round(min_value * range_scale);
}

/* Offsets and result range as the matmul task computes them
 * (tfcc/mkl/operations/tfcc_mklquantization.cpp:181-193;
 *  get_quantization_range_for_multiplication, tfcc_quantizationutils.h:23-43). */
EXPORT void oracle_matmul_params(float min_a, float max_a, float min_b, float max_b,
                                 int32_t* off_a, int32_t* off_b, float* min_c, float* max_c) {
  double scale;
  int64_t oa, ob;
  scale_info_8bit(min_a, max_a, &scale, &oa);
  scale_info_8bit(min_b, max_b, &scale, &ob);
  oa -= 0;      /* numeric_limits<uint8_t>::lowest() */
  ob -= -128;   /* numeric_limits<int8_t>::lowest()  */
  *off_a = (int32_t)oa;
  *off_b = (int32_t)ob;
  float a_level = (max_a - min_a) / (float)(255 - 0);
  float b_level = (max_b - min_b) / (float)(127 - (-128));
  float c_level = a_level * b_level;
  *min_c = c_level * (float)(int64_t)INT32_MIN;
  *max_c = c_level * (float)(int64_t)INT32_MAX;
}

/* _mkl_create_offset_matrix (tfcc_mklquantization.cpp:33-69):
 * c[b][i][j] = offA*offB*k + rsA[b][i]*offB + rsB[b][j]*offA, int32. */
EXPORT void oracle_create_offset_matrix(unsigned batch, const int32_t* a, unsigned total_a,
                                        unsigned stride_a, const int32_t* b, unsigned total_b,
                                        unsigned stride_b, int32_t offset_a, int32_t offset_b,
                                        int32_t k, int32_t* c, unsigned stride_c) {
  int32_t global_offset = (int32_t)((uint32_t)offset_a * (uint32_t)offset_b * (uint32_t)k);
  for (unsigned i = 0; i < batch; ++i) {
    const int32_t* ra = a + (size_t)i * stride_a;
    const int32_t* rb = b + (size_t)i * stride_b;
    int32_t* rc = c + (size_t)i * stride_c;
#pragma omp parallel for
    for (unsigned j = 0; j < total_a; ++j) {
      int32_t* pc = rc + (size_t)j * total_b;
      int32_t oa = (int32_t)((uint32_t)ra[j] * (uint32_t)offset_b);
      for (unsigned kk = 0; kk < total_b; ++kk) {
        int32_t ob = (int32_t)((uint32_t)rb[kk] * (uint32_t)offset_a);
        pc[kk] = (int32_t)((uint32_t)global_offset + (uint32_t)oa + (uint32_t)ob);
      }
    }
  }
}

/* The accumulating GEMM, c += a.b with a u8 [m,k], b s8 [k,n], c s32 [m,n] row-major.
 * The reference runs it as quantizedMatmulColMajor on the swapped operands
 * (tfcc_mklquantization.cpp:199-201; kernel/tfcc_mklquantizationmatmul.avx256.cpp:90-165),
 * widening to 16 bits, multiplying pairs with vpmaddwd and adding in int32
 * (gemm/tfcc_mklmatmulkernel.h:142-260).  Products of u8 and s8 fit 16 bits and
 * the pair sums fit 32, so the result is the plain integer dot product mod 2^32. */
EXPORT void oracle_qgemm_accumulate(unsigned batch, const uint8_t* a, unsigned stride_a,
                                    const int8_t* b, unsigned stride_b, unsigned m, unsigned n,
                                    unsigned k, int32_t* c, unsigned stride_c) {
  for (unsigned bt = 0; bt < batch; ++bt) {
    const uint8_t* pa = a + (size_t)bt * stride_a;
    const int8_t* pb = b + (size_t)bt * stride_b;
    int32_t* pc = c + (size_t)bt * stride_c;
#pragma omp parallel for
    for (unsigned i = 0; i < m; ++i) {
      uint32_t* row = (uint32_t*)(pc + (size_t)i * n);
      for (unsigned kk = 0; kk < k; ++kk) {
        const int32_t av = pa[(size_t)i * k + kk];
        const int8_t* brow = pb + (size_t)kk * n;
        for (unsigned j = 0; j < n; ++j) row[j] += (uint32_t)(av * (int32_t)brow[j]);
      }
    }
  }
}

/* quantizedMatmulN1 (kernel/tfcc_mklquantizationmatmul.avx256.cpp:63-80): n == 1, batch == 1. */
EXPORT void oracle_qgemm_n1(const uint8_t* a, const int32_t* reduce_a, int32_t offset_a,
                            const int8_t* b, int32_t reduce_b, int32_t offset_b, unsigned m,
                            unsigned k, int32_t* c) {
  uint32_t global_offset = (uint32_t)offset_a * (uint32_t)offset_b * (uint32_t)k +
                           (uint32_t)reduce_b * (uint32_t)offset_a;
#pragma omp parallel for
  for (unsigned i = 0; i < m; ++i) {
    uint32_t result = 0;
    for (unsigned j = 0; j < k; ++j) result += (uint32_t)((int32_t)a[(size_t)i * k + j] * (int32_t)b[j]);
    c[i] = (int32_t)(result + global_offset + (uint32_t)reduce_a[i] * (uint32_t)offset_b);
  }
}

/* The whole operator with already-folded arguments: offset matrix, then the
 * accumulate pass, or the n == 1 fast path (tfcc_mklquantization.cpp:140-201). */
EXPORT void oracle_qmatmul(unsigned batch, const uint8_t* a, unsigned stride_a,
                           const int32_t* rs_a, unsigned stride_rs_a, int32_t off_a,
                           const int8_t* b, unsigned stride_b, const int32_t* rs_b,
                           unsigned stride_rs_b, int32_t off_b, unsigned m, unsigned n,
                           unsigned k, int32_t* c) {
  if (n == 1 && batch == 1) {
    oracle_qgemm_n1(a, rs_a, off_a, b, rs_b[0], off_b, m, k, c);
    return;
  }
  oracle_create_offset_matrix(batch, rs_a, m, stride_rs_a, rs_b, n, stride_rs_b, off_a, off_b,
                              (int32_t)k, c, m * n);
  oracle_qgemm_accumulate(batch, a, stride_a, b, stride_b, m, n, k, c, m * n);
}

/* _mkl_reduce_sum_row / _mkl_reduce_sum_column (tfcc_mklquantization.cpp:205-282). */
#define DEFINE_REDUCE(NAME, T)                                                              \
  EXPORT void oracle_reduce_sum_##NAME(const T* a, unsigned batch, unsigned row,            \
                                       unsigned column, int row_flag, int32_t* b) {         \
    if (row_flag) {                                                                         \
      _Pragma("omp parallel for") for (unsigned i = 0; i < batch * row; ++i) {              \
        int32_t tmp = 0;                                                                    \
        const T* pa = a + (size_t)i * column;                                               \
        for (unsigned kk = 0; kk < column; ++kk) tmp += (int32_t)pa[kk];                    \
        b[i] = tmp;                                                                         \
      }                                                                                     \
    } else {                                                                                \
      memset(b, 0, sizeof(int32_t) * (size_t)batch * column);                               \
      for (unsigned i = 0; i < batch; ++i) {                                                \
        const T* ra = a + (size_t)i * row * column;                                         \
        int32_t* rb = b + (size_t)i * column;                                               \
        for (unsigned j = 0; j < row; ++j) {                                                \
          const T* pa = ra + (size_t)j * column;                                            \
          for (unsigned kk = 0; kk < column; ++kk) rb[kk] += (int32_t)pa[kk];               \
        }                                                                                   \
      }                                                                                     \
    }                                                                                       \
  }
DEFINE_REDUCE(u8, uint8_t)
DEFINE_REDUCE(s8, int8_t)
DEFINE_REDUCE(s16, int16_t)

/* fp32 matmul with the batch / broadcast stride rules of
 * MKLBlasInterface<float>::matmul (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-186):
 * c[b] = bias + a[b or 0].b[b or 0].  The reference hands the arithmetic to
 * oneDNN v1.8.1 (dnnl::matmul, not vendored in the reference tree), whose
 * accumulation order is unspecified; this restatement accumulates in double
 * and rounds once, which is the ground truth the fp32 results are judged
 * against. */
EXPORT void oracle_sgemm_f64acc(unsigned batch, const float* a, unsigned stride_a,
                                const float* b, unsigned stride_b, const float* bias,
                                unsigned m, unsigned n, unsigned k, float* c, double* c64) {
  for (unsigned bt = 0; bt < batch; ++bt) {
    const float* pa = a + (size_t)bt * stride_a;
    const float* pb = b + (size_t)bt * stride_b;
#pragma omp parallel for
    for (unsigned i = 0; i < m; ++i) {
      double acc[n > 0 ? n : 1];
      for (unsigned j = 0; j < n; ++j) acc[j] = bias ? (double)bias[j] : 0.0;
      for (unsigned kk = 0; kk < k; ++kk) {
        const double av = pa[(size_t)i * k + kk];
        const float* brow = pb + (size_t)kk * n;
        for (unsigned j = 0; j < n; ++j) acc[j] += av * (double)brow[j];
      }
      for (unsigned j = 0; j < n; ++j) {
        size_t o = ((size_t)bt * m + i) * n + j;
        if (c) c[o] = (float)acc[j];
        if (c64) c64[o] = acc[j];
      }
    }
  }
}
