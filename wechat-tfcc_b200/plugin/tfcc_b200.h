// tfcc/b200 -- a TFCC backend for B200 that provides the matmul hot path.
//
// Written against the reference's own headers (include path: <reference>/tfcc/core) and
// meant to sit beside tfcc/cuda and tfcc/mkl.  It supplies
//   * B200Device / B200Session       the pattern of CUDADevice / CUDASession
//                                    (tfcc/cuda/framework/tfcc_cudadevice.cpp:36-108,
//                                     tfcc/cuda/framework/tfcc_cudasession.cpp:27-90)
//   * B200BlasInterface<T>           BlasInterface<T>::matmul x2
//                                    (tfcc/core/interfaces/tfcc_blasinterface.h:41,55)
//   * B200DataInterface<T>           set / get / zeros / copy, so data::set, data::get and
//                                    Constant upload work (tfcc/core/interfaces/tfcc_datainterface.h)
//   * tfcc::b200::quantization       matmul and reduce_sum with the signatures of
//                                    tfcc/mkl/operations/tfcc_mklquantization.h:39-51
// and forwards all arithmetic to libtfcc_b200 (include/tfcc_b200.h).  Nothing else of the
// eighteen interface families is provided: other operators keep throwing NotImplementedError
// as the core's defaults do.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "tfcc.h"
#include "interfaces/tfcc_blasinterface.h"
#include "interfaces/tfcc_datainterface.h"
#include "interfaces/tfcc_activationinterface.h"
#include "interfaces/tfcc_basicinterface.h"
#include "interfaces/tfcc_interface.h"
#include "interfaces/tfcc_normalizationinterface.h"
#include "interfaces/tfcc_quantizationinterface.h"
#include "utils/tfcc_initializer.h"

namespace tfcc {

// Failure reported by the kernel library or the CUDA runtime (cf. CUDARuntimeError,
// tfcc/cuda/exceptions/tfcc_cudaruntimeerror.h).
class B200RuntimeError : public Exception {
  int _status;
  std::string _reason;

 public:
  explicit B200RuntimeError(int status);
  const char* reason() const noexcept override;
  int status() const { return _status; }
};

class B200Device : public Device {
  int _cudaDevice;
  bool _tf32;

 public:
  explicit B200Device(unsigned deviceID);
  B200Device(unsigned deviceID, std::unique_ptr<Allocator> allocator);
  ~B200Device();

  void attach() override;

  // Opt-in single-pass TF32 products (about 1e-3 relative); the default is fp32 results
  // within 1e-5.  Mirrors CUDADevice::enableTensorCore (tfcc/cuda/framework/tfcc_cudadevice.h:39-41).
  void enableTF32() { _tf32 = true; }
  void disableTF32() { _tf32 = false; }
  bool isTF32Enabled() const { return _tf32; }
  int precisionMode() const;
  int cudaDevice() const { return _cudaDevice; }

  static unsigned getDeviceCount();
};

class B200Session : public Session {
  B200Device& _device;
  cudaStream_t _stream;
  int* _status;       // device word the kernels OR give-up bits into
  void* _scratch;     // grown on demand, reused across calls
  size_t _scratchBytes;
  bool _destroying;

 public:
  explicit B200Session(B200Device& device);
  B200Session(B200Device& device, std::unique_ptr<Allocator> allocator);
  ~B200Session();

  void sync() const override;
  Device& getDevice() override;
  const Device& getDevice() const override;

  cudaStream_t stream() const { return _stream; }
  int* deviceStatus() const { return _status; }
  // Scratch of at least `bytes` from the session allocator (valid until the next request).
  void* scratch(size_t bytes);
};

template <class T>
class B200BlasInterface : public BlasInterface<T> {
 public:
  Variable<T> matmul(const Tensor<T>& a, const Tensor<T>& b) override;
  Variable<T> matmul(const Tensor<T>& a, const Tensor<T>& b, const Tensor<T>& c) override;
};

template <class T>
class B200DataInterface : public DataInterface<T> {
 public:
  void set(T* dst, const T* data, size_t len) override;
  void set(Variable<T>& a, const T* data) override;
  void set(Variable<T>& a, std::vector<T>&& data) override;
  void get(const Tensor<T>& a, T* data) override;
  void zeros(Variable<T>& a) override;
  Variable<T> copy(const Tensor<T>& a) override;
};

// quantize / requantize / dequantize on the device, ranges kept in device memory
// (tfcc/core/interfaces/tfcc_quantizationinterface.h:39-138; semantics of
// tfcc/mkl/interfaces/tfcc_mklquantizationinterface.cpp).  T is one of the six quantization
// types (int8..uint32).
template <class T>
class B200QuantizationInterface : public QuantizationInterface<T> {
 public:
  std::tuple<Variable<T>, Variable<float>, Variable<float>> quantize(const Tensor<float>& a) override;
  Variable<T> quantize(const Tensor<float>& a, const Tensor<float>& minValue,
                       const Tensor<float>& maxValue) override;
  Variable<T> requantize(const Tensor<int8_t>& a, const Tensor<float>& minInput,
                         const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                         const Tensor<float>& maxOutput) override;
  Variable<T> requantize(const Tensor<uint8_t>& a, const Tensor<float>& minInput,
                         const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                         const Tensor<float>& maxOutput) override;
  Variable<T> requantize(const Tensor<int16_t>& a, const Tensor<float>& minInput,
                         const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                         const Tensor<float>& maxOutput) override;
  Variable<T> requantize(const Tensor<uint16_t>& a, const Tensor<float>& minInput,
                         const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                         const Tensor<float>& maxOutput) override;
  Variable<T> requantize(const Tensor<int32_t>& a, const Tensor<float>& minInput,
                         const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                         const Tensor<float>& maxOutput) override;
  Variable<T> requantize(const Tensor<uint32_t>& a, const Tensor<float>& minInput,
                         const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                         const Tensor<float>& maxOutput) override;
  Variable<float> dequantize(const Tensor<T>& a, const Tensor<float>& minValue,
                             const Tensor<float>& maxValue) override;
};

// The operators between the matmuls of an attention / feed-forward block, float only and only
// the cases such a block uses; everything else keeps the core's NotImplementedError default.
//   softmax over the last axis, geluAccurate     (tfcc/core/interfaces/tfcc_activationinterface.h:38,45)
//   layerNormalize                               (tfcc/core/interfaces/tfcc_normalizationinterface.h:39-41)
//   transpose with perm (0,2,1,3) or "swap the last two axes"
//                                                (tfcc/core/interfaces/tfcc_basicinterface.h:47)
class B200ActivationInterface : public ActivationInterface<float> {
 public:
  Variable<float> softmax(const Tensor<float>& a, size_t axis) override;
  Variable<float> geluAccurate(const Tensor<float>& a) override;
};

class B200NormalizationInterface : public NormalizationInterface<float> {
 public:
  Variable<float> layerNormalize(const Tensor<float>& a, const Tensor<float>& gamma,
                                 const Tensor<float>& beta, float epsilon,
                                 size_t beginNormAxis) override;
};

class B200BasicInterface : public BasicInterface<float> {
 public:
  Variable<float> transpose(const Tensor<float>& a, const std::vector<size_t>& perm) override;
};

template <class T>
Interface<T> get_b200_interface(T, B200Device& device);

// Binds the calling thread to the least used B200 device and a fresh session on it
// (cf. initialize_cuda, tfcc/cuda/utils/tfcc_cudautils.cpp:23-50).
void initialize_b200();
void initialize_b200(unsigned deviceID);

namespace b200 {

// softmax(scale * Q K^T) V per head in one kernel (tfccb200_attention_f32).  q, k and v are
// [batch, seq, heads*dim] tensors, or the three column slices of one packed
// [batch, seq, 3*heads*dim] tensor given through attention_packed.  Stands for the transposes,
// batched matmuls, scale and softmax of the reference graph (see include/tfcc_b200.h).
Variable<float> attention(const Tensor<float>& q, const Tensor<float>& k, const Tensor<float>& v,
                          unsigned heads, float scale);
Variable<float> attention_packed(const Tensor<float>& qkv, unsigned heads, float scale);

// Derived constants, computed once per weight and kept as runtime constants of the current
// scope -- what the reference's Constant preprocess hook is for
// (tfcc/core/framework/tfcc_constant.cpp:70-106; cache: tfcc_constantmanager.cpp:38-64):
//   * the int32 column sums of an int8 weight, the reduceSumB argument of the quantized matmul,
//     so that reduce_sum(B, false) runs when the weight is first used and never again;
//   * several float weights (or biases) with the same row count joined along their columns, so
//     that the Q / K / V projections of an attention block become one matmul.
const Constant<int32_t>& cached_column_sums(const std::string& weightName);
const Constant<float>& cached_concat_columns(const std::string& packedName,
                                             const std::vector<std::string>& names);

namespace parallel {

// The N split of one large product over several GPUs driven by this process, one Device per
// GPU as in tfcc/core/utils/tfcc_initializer.cpp:50-66.  B is column-sharded, every GPU
// multiplies its shard and stores each finished tile into all GPUs' C over NVLink from the
// GEMM epilogue; no separate all-gather pass runs (tfccb200_group_*, include/tfcc_b200.h).
class NSplitGroup {
  void* _group;
  std::vector<unsigned> _devices;

 public:
  explicit NSplitGroup(const std::vector<unsigned>& deviceIDs);
  ~NSplitGroup();
  NSplitGroup(const NSplitGroup&) = delete;
  NSplitGroup& operator=(const NSplitGroup&) = delete;

  size_t size() const { return _devices.size(); }
  cudaStream_t stream(size_t member) const;

  // c = a . b for row-major host matrices (pinned for overlapped copies); synchronous.
  void matmul_host(const float* a, const float* b, float* c, unsigned m, unsigned n, unsigned k);
  // Device-resident operands: a[i] [m,k], bShards[i] [k,nShard] and c[i] [m, size()*nShard]
  // live on member i's GPU.  Queued on the members' group streams; sync() waits.
  void matmul(const std::vector<const float*>& a, const std::vector<const float*>& bShards,
              const std::vector<float*>& c, unsigned m, unsigned nShard, unsigned k);
  void sync();
};

}  // namespace parallel

namespace quantization {

std::tuple<Variable<int32_t>, Variable<float>, Variable<float>> matmul(
    const Tensor<uint8_t>& a, const Tensor<int32_t>& reduceSumA, const Tensor<float>& minA,
    const Tensor<float>& maxA, const Tensor<int8_t>& b, const Tensor<int32_t>& reduceSumB,
    const Tensor<float>& minB, const Tensor<float>& maxB);

template <class T>
Variable<int32_t> reduce_sum(const Tensor<T>& a, bool row);

}  // namespace quantization
}  // namespace b200

}  // namespace tfcc
