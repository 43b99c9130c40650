#include "tfcc_b200.h"

#include <algorithm>
#include <utility>

#include "tfcc_b200.h"
#include "../../include/tfcc_b200.h"

namespace tfcc {

namespace {

inline void check_cuda(cudaError_t e) {
  if (e != cudaSuccess) throw B200RuntimeError(static_cast<int>(e));
}

inline void check_status(int st) {
  if (st == TFCCB200_OK) return;
  if (st == TFCCB200_EINVAL || st == TFCCB200_EALIGN || st == TFCCB200_EOVERFLOW ||
      st == TFCCB200_EUNSUPPORTED)
    throw InvalidArgumentError(tfccb200_strerror(st));
  if (st == TFCCB200_EWORKSPACE) throw ResourceExhaustedError();
  throw B200RuntimeError(st);
}

B200Session* current_session() {
  B200Session* s = dynamic_cast<B200Session*>(Session::getThreadDefault());
  if (s == nullptr) throw RuntimeError("the thread default session is not a B200 session");
  return s;
}

B200Device* current_device() {
  B200Device* d = dynamic_cast<B200Device*>(Device::getThreadDefault());
  if (d == nullptr) throw RuntimeError("the thread default device is not a B200 device");
  return d;
}

template <class T>
std::shared_ptr<ConstantManager<T>> make_constant_manager(
    const std::function<void*(size_t)>& realMalloc, const std::function<void(void*)>& realFree) {
  auto m = std::make_shared<ConstantManager<T>>();
  m->getAllocator().setRealMalloc(realMalloc);
  m->getAllocator().setRealFree(realFree);
  return m;
}

// Shapes, strides and batch count exactly as the reference backends derive them
// (tfcc/mkl/interfaces/tfcc_mklblasinterface.cpp:127-151).
struct MatmulGeometry {
  unsigned m, n, k, strideA, strideB, strideC, batch;
  std::vector<unsigned> resultShape;
};

template <class TA, class TB>
MatmulGeometry matmul_geometry(const Tensor<TA>& a, const Tensor<TB>& b) {
  MatmulGeometry g;
  g.m = a.shape(a.shape().size() - 2);
  g.n = b.shape(b.shape().size() - 1);
  g.k = a.shape(a.shape().size() - 1);
  g.strideA = g.m * g.k;
  g.strideB = g.n * g.k;
  g.strideC = g.m * g.n;
  if (a.shape().size() != b.shape().size()) {
    g.strideA = a.shape().size() == 2 ? 0 : g.strideA;
    g.strideB = b.shape().size() == 2 ? 0 : g.strideB;
  }
  g.resultShape = a.shape().size() > b.shape().size() ? a.shape().toVector() : b.shape().toVector();
  g.resultShape[g.resultShape.size() - 2] = g.m;
  g.resultShape[g.resultShape.size() - 1] = g.n;
  unsigned long long area = 1;
  for (unsigned d : g.resultShape) area *= d;
  g.batch = static_cast<unsigned>(area / (static_cast<unsigned long long>(g.m) * g.n));
  return g;
}

}  // namespace

// ---------------------------------------------------------------- exception
B200RuntimeError::B200RuntimeError(int status) : _status(status) {
  _reason = std::string("tfcc_b200 [") + std::to_string(status) + "] " + tfccb200_strerror(status);
}

const char* B200RuntimeError::reason() const noexcept { return _reason.c_str(); }

// ---------------------------------------------------------------- device
unsigned B200Device::getDeviceCount() {
  int n = 0;
  check_cuda(cudaGetDeviceCount(&n));
  return static_cast<unsigned>(n);
}

B200Device::B200Device(unsigned deviceID)
    : B200Device(deviceID, std::unique_ptr<Allocator>(new FlexAllocator())) {
  size_t freeBytes = 0, totalBytes = 0;
  check_cuda(cudaSetDevice(_cudaDevice));
  check_cuda(cudaMemGetInfo(&freeBytes, &totalBytes));
  FlexAllocator* alloc = dynamic_cast<FlexAllocator*>(_allocator.get());
  if (alloc) alloc->setLimit(totalBytes * 9 / 10);
}

B200Device::B200Device(unsigned deviceID, std::unique_ptr<Allocator> allocator)
    : Device(deviceID & 0x00ffffff, std::move(allocator)),
      _cudaDevice(static_cast<int>(deviceID & 0x00ffffff)),
      _tf32(false) {
  const int dev = _cudaDevice;
  std::function<void*(size_t)> realMalloc = [dev](size_t len) -> void* {
    void* p = nullptr;
    if (cudaSetDevice(dev) != cudaSuccess) return nullptr;
    if (cudaMalloc(&p, len) != cudaSuccess) return nullptr;
    return p;
  };
  std::function<void(void*)> realFree = [](void* p) {
    cudaError_t e = cudaFree(p);
    if (e != cudaSuccess && e != cudaErrorCudartUnloading) throw B200RuntimeError(static_cast<int>(e));
  };
  _allocator->setRealMalloc(realMalloc);
  _allocator->setRealFree(realFree);

  _floatConstantManager = make_constant_manager<float>(realMalloc, realFree);
  _doubleConstantManager = make_constant_manager<double>(realMalloc, realFree);
  _int8ConstantManager = make_constant_manager<int8_t>(realMalloc, realFree);
  _uint8ConstantManager = make_constant_manager<uint8_t>(realMalloc, realFree);
  _int16ConstantManager = make_constant_manager<int16_t>(realMalloc, realFree);
  _uint16ConstantManager = make_constant_manager<uint16_t>(realMalloc, realFree);
  _int32ConstantManager = make_constant_manager<int32_t>(realMalloc, realFree);
  _uint32ConstantManager = make_constant_manager<uint32_t>(realMalloc, realFree);
  _int64ConstantManager = make_constant_manager<int64_t>(realMalloc, realFree);
  _uint64ConstantManager = make_constant_manager<uint64_t>(realMalloc, realFree);

  _floatInterface = get_b200_interface(float(), *this);
  _doubleInterface = get_b200_interface(double(), *this);
  _int8Interface = get_b200_interface(int8_t(), *this);
  _uint8Interface = get_b200_interface(uint8_t(), *this);
  _int16Interface = get_b200_interface(int16_t(), *this);
  _uint16Interface = get_b200_interface(uint16_t(), *this);
  _int32Interface = get_b200_interface(int32_t(), *this);
  _uint32Interface = get_b200_interface(uint32_t(), *this);
  _int64Interface = get_b200_interface(int64_t(), *this);
  _uint64Interface = get_b200_interface(uint64_t(), *this);
}

B200Device::~B200Device() {}

void B200Device::attach() { check_cuda(cudaSetDevice(_cudaDevice)); }

int B200Device::precisionMode() const {
  return _tf32 ? TFCCB200_PRECISION_TF32 : TFCCB200_PRECISION_FP32;
}

// ---------------------------------------------------------------- session
B200Session::B200Session(B200Device& device)
    : B200Session(device, std::unique_ptr<Allocator>(new FlexAllocator())) {
  size_t freeBytes = 0, totalBytes = 0;
  check_cuda(cudaMemGetInfo(&freeBytes, &totalBytes));
  FlexAllocator* alloc = dynamic_cast<FlexAllocator*>(_allocator.get());
  if (alloc) alloc->setLimit(totalBytes * 6 / 10);
}

B200Session::B200Session(B200Device& device, std::unique_ptr<Allocator> allocator)
    : Session(std::move(allocator)),
      _device(device),
      _stream(nullptr),
      _status(nullptr),
      _scratch(nullptr),
      _scratchBytes(0),
      _destroying(false) {
  _device.attach();
  check_cuda(cudaStreamCreateWithFlags(&_stream, cudaStreamNonBlocking));
  _allocator->setRealMalloc([this](size_t len) { return this->_device.malloc(len); });
  _allocator->setRealFree([this](void* p) {
    this->sync();
    this->_device.free(p);
  });
  _status = static_cast<int*>(_device.malloc(sizeof(int)));
  if (_status == nullptr) throw ResourceExhaustedError();
  check_cuda(cudaMemsetAsync(_status, 0, sizeof(int), _stream));
}

B200Session::~B200Session() {
  _destroying = true;
  cudaStreamSynchronize(_stream);
  // the session allocator refuses to be destroyed while any of its blocks is still out
  if (_scratch) _allocator->free(_scratch);
  _scratch = nullptr;
  preRelease();
  _device.free(_status);
  cudaStreamDestroy(_stream);
}

void B200Session::sync() const {
  cudaError_t e = cudaStreamSynchronize(_stream);
  if (e != cudaSuccess) {
    if (e == cudaErrorCudartUnloading && _destroying) return;
    throw B200RuntimeError(static_cast<int>(e));
  }
  if (_destroying) return;
  // Device-side give-ups (bounded waits that ran out) surface here, like any asynchronous fault.
  int st = 0;
  check_cuda(cudaMemcpy(&st, _status, sizeof(int), cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(_status, 0, sizeof(int));
    throw B200RuntimeError(TFCCB200_EDEVICE);
  }
}

Device& B200Session::getDevice() { return _device; }
const Device& B200Session::getDevice() const { return _device; }

void* B200Session::scratch(size_t bytes) {
  if (bytes <= _scratchBytes) return _scratch;
  if (_scratch) _allocator->free(_scratch);  // the allocator syncs before memory really goes back
  _scratch = nullptr;
  _scratchBytes = 0;
  void* p = _allocator->malloc(bytes);
  if (p == nullptr) throw ResourceExhaustedError();
  _scratch = p;
  _scratchBytes = bytes;
  return p;
}

// ---------------------------------------------------------------- blas
template <class T>
Variable<T> B200BlasInterface<T>::matmul(const Tensor<T>&, const Tensor<T>&) {
  throw NotImplementedError();  // float only, as the MKL backend (tfcc_mklblasinterface.cpp:35-39)
}

template <class T>
Variable<T> B200BlasInterface<T>::matmul(const Tensor<T>&, const Tensor<T>&, const Tensor<T>&) {
  throw NotImplementedError();
}

static Variable<float> b200_matmul(const Tensor<float>& a, const Tensor<float>& b,
                                   const float* bias) {
  MatmulGeometry g = matmul_geometry(a, b);
  Variable<float> result(Shape(g.resultShape));
  B200Session* session = current_session();
  const int mode = current_device()->precisionMode();
  const size_t ws = tfccb200_sgemm_workspace(g.m, g.n, g.k, g.batch, mode);
  void* scratch = ws ? session->scratch(ws) : nullptr;
  check_status(tfccb200_sgemm(session->stream(), a.data(), g.strideA, b.data(), g.strideB,
                              result.data(), g.strideC, bias, g.m, g.n, g.k, g.batch, mode,
                              scratch, ws, session->deviceStatus()));
  return result;
}

template <>
Variable<float> B200BlasInterface<float>::matmul(const Tensor<float>& a, const Tensor<float>& b) {
  return b200_matmul(a, b, nullptr);
}

template <>
Variable<float> B200BlasInterface<float>::matmul(const Tensor<float>& a, const Tensor<float>& b,
                                                 const Tensor<float>& c) {
  return b200_matmul(a, b, c.data());
}

// ---------------------------------------------------------------- data
template <class T>
void B200DataInterface<T>::set(T* dst, const T* data, size_t len) {
  B200Session* session = current_session();
  check_cuda(cudaMemcpyAsync(dst, data, len * sizeof(T), cudaMemcpyHostToDevice, session->stream()));
  check_cuda(cudaStreamSynchronize(session->stream()));  // the host buffer may go away
}

template <class T>
void B200DataInterface<T>::set(Variable<T>& a, const T* data) {
  set(a.data(), data, a.size());
}

template <class T>
void B200DataInterface<T>::set(Variable<T>& a, std::vector<T>&& data) {
  set(a.data(), data.data(), a.size());
}

template <class T>
void B200DataInterface<T>::get(const Tensor<T>& a, T* data) {
  a.sync();
  check_cuda(cudaMemcpy(data, a.data(), a.size() * sizeof(T), cudaMemcpyDeviceToHost));
}

template <class T>
void B200DataInterface<T>::zeros(Variable<T>& a) {
  check_cuda(cudaMemsetAsync(a.data(), 0, a.size() * sizeof(T), current_session()->stream()));
}

template <class T>
Variable<T> B200DataInterface<T>::copy(const Tensor<T>& a) {
  Variable<T> result(a.shape());
  check_cuda(cudaMemcpyAsync(result.data(), a.data(), a.size() * sizeof(T),
                             cudaMemcpyDeviceToDevice, current_session()->stream()));
  return result;
}

// ---------------------------------------------------------------- quantization interface
namespace {

template <class T> struct TypeId;
template <> struct TypeId<int8_t> { static constexpr int value = TFCCB200_TYPE_S8; };
template <> struct TypeId<uint8_t> { static constexpr int value = TFCCB200_TYPE_U8; };
template <> struct TypeId<int16_t> { static constexpr int value = TFCCB200_TYPE_S16; };
template <> struct TypeId<uint16_t> { static constexpr int value = TFCCB200_TYPE_U16; };
template <> struct TypeId<int32_t> { static constexpr int value = TFCCB200_TYPE_S32; };
template <> struct TypeId<uint32_t> { static constexpr int value = TFCCB200_TYPE_U32; };

void check_range_tensor(const Tensor<float>& t, const char* message) {
  if (t.size() != 1 || t.shape().size() != 1) throw InvalidArgumentError(message);
}

template <class TO, class TI>
Variable<TO> b200_requantize(const Tensor<TI>& a, const Tensor<float>& minInput,
                             const Tensor<float>& maxInput, const Tensor<float>& minOutput,
                             const Tensor<float>& maxOutput) {
  if (a.size() == 0) throw InvalidArgumentError("invalid tensor");
  check_range_tensor(minInput, "invalid minInput");
  check_range_tensor(maxInput, "invalid maxInput");
  check_range_tensor(minOutput, "invalid minOutput");
  check_range_tensor(maxOutput, "invalid maxOutput");
  Variable<TO> result(a.shape());
  check_status(tfccb200_requantize(current_session()->stream(), a.data(), TypeId<TI>::value,
                                   a.size(), minInput.data(), maxInput.data(), minOutput.data(),
                                   maxOutput.data(), result.data(), TypeId<TO>::value));
  return result;
}

}  // namespace

template <class T>
std::tuple<Variable<T>, Variable<float>, Variable<float>> B200QuantizationInterface<T>::quantize(
    const Tensor<float>& a) {
  if (a.size() == 0) throw InvalidArgumentError("invalid tensor");
  Variable<T> result(a.shape());
  Variable<float> range({2});
  B200Session* session = current_session();
  check_status(tfccb200_minmax_f32(session->stream(), a.data(), a.size(), range.data()));
  check_status(tfccb200_quantize_f32(session->stream(), a.data(), a.size(), range.data(),
                                     range.data() + 1, result.data(), TypeId<T>::value));
  Variable<float> minValue({1}), maxValue({1});
  check_cuda(cudaMemcpyAsync(minValue.data(), range.data(), sizeof(float), cudaMemcpyDeviceToDevice,
                             session->stream()));
  check_cuda(cudaMemcpyAsync(maxValue.data(), range.data() + 1, sizeof(float),
                             cudaMemcpyDeviceToDevice, session->stream()));
  return std::make_tuple(std::move(result), std::move(minValue), std::move(maxValue));
}

template <class T>
Variable<T> B200QuantizationInterface<T>::quantize(const Tensor<float>& a,
                                                   const Tensor<float>& minValue,
                                                   const Tensor<float>& maxValue) {
  if (a.size() == 0) throw InvalidArgumentError("invalid tensor");
  check_range_tensor(minValue, "invalid minValue");
  check_range_tensor(maxValue, "invalid maxValue");
  Variable<T> result(a.shape());
  check_status(tfccb200_quantize_f32(current_session()->stream(), a.data(), a.size(),
                                     minValue.data(), maxValue.data(), result.data(),
                                     TypeId<T>::value));
  return result;
}

#define TFCC_B200_REQUANTIZE(TI)                                                                 \
  template <class T>                                                                             \
  Variable<T> B200QuantizationInterface<T>::requantize(                                          \
      const Tensor<TI>& a, const Tensor<float>& minInput, const Tensor<float>& maxInput,         \
      const Tensor<float>& minOutput, const Tensor<float>& maxOutput) {                          \
    return b200_requantize<T, TI>(a, minInput, maxInput, minOutput, maxOutput);                  \
  }
TFCC_B200_REQUANTIZE(int8_t)
TFCC_B200_REQUANTIZE(uint8_t)
TFCC_B200_REQUANTIZE(int16_t)
TFCC_B200_REQUANTIZE(uint16_t)
TFCC_B200_REQUANTIZE(int32_t)
TFCC_B200_REQUANTIZE(uint32_t)
#undef TFCC_B200_REQUANTIZE

template <class T>
Variable<float> B200QuantizationInterface<T>::dequantize(const Tensor<T>& a,
                                                         const Tensor<float>& minValue,
                                                         const Tensor<float>& maxValue) {
  if (a.size() == 0) throw InvalidArgumentError("invalid tensor");
  check_range_tensor(minValue, "invalid minValue");
  check_range_tensor(maxValue, "invalid maxValue");
  Variable<float> result(a.shape());
  check_status(tfccb200_dequantize_f32(current_session()->stream(), a.data(), TypeId<T>::value,
                                       a.size(), minValue.data(), maxValue.data(), result.data()));
  return result;
}

template class B200QuantizationInterface<int8_t>;
template class B200QuantizationInterface<uint8_t>;
template class B200QuantizationInterface<int16_t>;
template class B200QuantizationInterface<uint16_t>;
template class B200QuantizationInterface<int32_t>;
template class B200QuantizationInterface<uint32_t>;

// ---------------------------------------------------------------- attention / FFN glue (float)
Variable<float> B200ActivationInterface::softmax(const Tensor<float>& a, size_t axis) {
  if (a.size() == 0) throw InvalidArgumentError("invalid tensor");
  if (axis + 1 != a.shape().size()) throw NotImplementedError();  // last axis only
  const unsigned cols = a.shape(axis);
  Variable<float> result(a.shape());
  check_status(tfccb200_softmax_f32(current_session()->stream(), a.data(), a.size() / cols, cols,
                                    1.0f, result.data()));
  return result;
}

Variable<float> B200ActivationInterface::geluAccurate(const Tensor<float>& a) {
  if (a.size() == 0) throw InvalidArgumentError("invalid tensor");
  Variable<float> result(a.shape());
  check_status(tfccb200_gelu_f32(current_session()->stream(), a.data(), a.size(), result.data()));
  return result;
}

Variable<float> B200NormalizationInterface::layerNormalize(const Tensor<float>& a,
                                                           const Tensor<float>& gamma,
                                                           const Tensor<float>& beta,
                                                           float epsilon, size_t beginNormAxis) {
  if (a.size() == 0 || beginNormAxis >= a.shape().size())
    throw InvalidArgumentError("invalid tensor or axis");
  unsigned cols = 1;
  for (size_t i = beginNormAxis; i < a.shape().size(); ++i) cols *= a.shape(i);
  if (gamma.size() != cols || beta.size() != cols)
    throw InvalidArgumentError("gamma or beta don't match the normalized axes");
  Variable<float> result(a.shape());
  check_status(tfccb200_layer_norm_f32(current_session()->stream(), a.data(), nullptr, gamma.data(),
                                       beta.data(), epsilon, a.size() / cols, cols, result.data()));
  return result;
}

Variable<float> B200BasicInterface::transpose(const Tensor<float>& a,
                                              const std::vector<size_t>& perm) {
  const size_t rank = a.shape().size();
  std::vector<unsigned> s(rank);
  for (size_t i = 0; i < rank; ++i) s[i] = a.shape(perm[i]);
  bool swap_last2 = rank >= 2 && perm[rank - 1] == rank - 2 && perm[rank - 2] == rank - 1;
  for (size_t i = 0; swap_last2 && i + 2 < rank; ++i) swap_last2 = perm[i] == i;
  const bool is0213 =
      rank == 4 && perm[0] == 0 && perm[1] == 2 && perm[2] == 1 && perm[3] == 3;
  if (!swap_last2 && !is0213) throw NotImplementedError();
  Variable<float> result{Shape(s)};
  void* stream = current_session()->stream();
  if (swap_last2) {
    const unsigned r = a.shape(rank - 2), c = a.shape(rank - 1);
    check_status(tfccb200_transpose_last2_f32(stream, a.data(), a.size() / (r * c), r, c,
                                              result.data()));
  } else {
    check_status(tfccb200_permute_0213_f32(stream, a.data(), a.shape(0), a.shape(1), a.shape(2),
                                           a.shape(3), result.data()));
  }
  return result;
}

// ---------------------------------------------------------------- registration
namespace {
template <class T>
void set_float_glue_interfaces(Interface<T>&) {}
template <>
void set_float_glue_interfaces<float>(Interface<float>& interface) {
  interface.setActivationInterface(
      std::unique_ptr<ActivationInterface<float>>(new B200ActivationInterface()));
  interface.setNormalizationInterface(
      std::unique_ptr<NormalizationInterface<float>>(new B200NormalizationInterface()));
  interface.setBasicInterface(std::unique_ptr<BasicInterface<float>>(new B200BasicInterface()));
}

template <class T>
void set_quantization_interface(Interface<T>&) {}  // only the six quantization types have one
#define TFCC_B200_SET_QUANTIZATION(type)                                          \
  template <>                                                                     \
  void set_quantization_interface<type>(Interface<type> & interface) {            \
    interface.setQuantizationInterface(                                           \
        std::unique_ptr<QuantizationInterface<type>>(new B200QuantizationInterface<type>())); \
  }
TFCC_B200_SET_QUANTIZATION(int8_t)
TFCC_B200_SET_QUANTIZATION(uint8_t)
TFCC_B200_SET_QUANTIZATION(int16_t)
TFCC_B200_SET_QUANTIZATION(uint16_t)
TFCC_B200_SET_QUANTIZATION(int32_t)
TFCC_B200_SET_QUANTIZATION(uint32_t)
#undef TFCC_B200_SET_QUANTIZATION
}  // namespace

template <class T>
Interface<T> get_b200_interface(T, B200Device&) {
  Interface<T> interface;
  interface.setBlasInterface(std::unique_ptr<BlasInterface<T>>(new B200BlasInterface<T>()));
  interface.setDataInterface(std::unique_ptr<DataInterface<T>>(new B200DataInterface<T>()));
  set_quantization_interface<T>(interface);
  set_float_glue_interfaces<T>(interface);
  return interface;
}

#define TFCC_B200_INSTANTIATE(type)                                   \
  template class B200BlasInterface<type>;                             \
  template class B200DataInterface<type>;                             \
  template Interface<type> get_b200_interface(type, B200Device& device);
TFCC_B200_INSTANTIATE(float)
TFCC_B200_INSTANTIATE(double)
TFCC_B200_INSTANTIATE(int8_t)
TFCC_B200_INSTANTIATE(uint8_t)
TFCC_B200_INSTANTIATE(int16_t)
TFCC_B200_INSTANTIATE(uint16_t)
TFCC_B200_INSTANTIATE(int32_t)
TFCC_B200_INSTANTIATE(uint32_t)
TFCC_B200_INSTANTIATE(int64_t)
TFCC_B200_INSTANTIATE(uint64_t)
#undef TFCC_B200_INSTANTIATE

static Initializer& b200_initializer() {
  static Initializer initializer(
      B200Device::getDeviceCount(),
      [](size_t i) { return std::shared_ptr<Device>(new B200Device(static_cast<unsigned>(i))); },
      [](Device& device) {
        return std::shared_ptr<Session>(new B200Session(*dynamic_cast<B200Device*>(&device)));
      });
  return initializer;
}

static InitializerGuard& b200_initializer_guard() {
  thread_local InitializerGuard guard;
  return guard;
}

void initialize_b200() {
  if (Device::getThreadDefault() == nullptr || Session::getThreadDefault() == nullptr) {
    InitializerGuard& guard = b200_initializer_guard();
    guard = b200_initializer().allocate();
    Device::setThreadDefault(&guard.getDevice());
    Session::setThreadDefault(&guard.getSession());
  }
  Device::getThreadDefault()->attach();
}

void initialize_b200(unsigned deviceID) {
  if (Device::getThreadDefault() == nullptr || Session::getThreadDefault() == nullptr) {
    InitializerGuard& guard = b200_initializer_guard();
    guard = b200_initializer().allocate(deviceID);
    Device::setThreadDefault(&guard.getDevice());
    Session::setThreadDefault(&guard.getSession());
  }
  Device::getThreadDefault()->attach();
}

// ---------------------------------------------------------------- attention, constants, groups
namespace b200 {

namespace {

Variable<float> run_attention(const float* q, const float* k, const float* v, unsigned batch,
                              unsigned seq, unsigned heads, unsigned width, unsigned ld, float scale) {
  if (heads == 0 || width % heads != 0) throw InvalidArgumentError("heads does not divide the width");
  Variable<float> result({batch, seq, width});
  B200Session* session = current_session();
  check_status(tfccb200_attention_f32(session->stream(), q, k, v, result.data(), batch, seq, heads,
                                      width / heads, ld, width, scale, session->deviceStatus()));
  return result;
}

}  // namespace

Variable<float> attention(const Tensor<float>& q, const Tensor<float>& k, const Tensor<float>& v,
                          unsigned heads, float scale) {
  if (q.shape().size() != 3 || q.size() == 0) throw InvalidArgumentError("invalid tensor q");
  if (k.shape() != q.shape() || v.shape() != q.shape())
    throw InvalidArgumentError("q, k and v don't match");
  return run_attention(q.data(), k.data(), v.data(), q.shape(0), q.shape(1), heads, q.shape(2),
                       q.shape(2), scale);
}

Variable<float> attention_packed(const Tensor<float>& qkv, unsigned heads, float scale) {
  if (qkv.shape().size() != 3 || qkv.size() == 0 || qkv.shape(2) % 3 != 0)
    throw InvalidArgumentError("invalid packed tensor qkv");
  const unsigned width = qkv.shape(2) / 3;
  return run_attention(qkv.data(), qkv.data() + width, qkv.data() + 2 * width, qkv.shape(0),
                       qkv.shape(1), heads, width, qkv.shape(2), scale);
}

const Constant<int32_t>& cached_column_sums(const std::string& weightName) {
  const std::string derived = weightName + "/b200_column_sums";
  if (Constant<int32_t>* hit = Constant<int32_t>::tryGetRuntimeConstant(derived)) return *hit;
  const Constant<int8_t>& w = Constant<int8_t>::getConstant(weightName);
  Variable<int32_t> sums = quantization::reduce_sum(static_cast<const Tensor<int8_t>&>(w), false);
  std::vector<int32_t> host = data::get(sums);
  Constant<int32_t>::setRuntimeConstantIfNotExist(derived, sums.shape(), host);
  return *Constant<int32_t>::tryGetRuntimeConstant(derived);
}

const Constant<float>& cached_concat_columns(const std::string& packedName,
                                             const std::vector<std::string>& names) {
  if (Constant<float>* hit = Constant<float>::tryGetRuntimeConstant(packedName)) return *hit;
  if (names.empty()) throw InvalidArgumentError("nothing to concatenate");
  std::vector<std::vector<float>> parts;
  std::vector<unsigned> widths;
  unsigned rows = 0, total = 0;
  bool rank1 = false;
  for (const std::string& name : names) {
    const Constant<float>& c = Constant<float>::getConstant(name);
    if (c.shape().size() != 1 && c.shape().size() != 2)
      throw InvalidArgumentError("only rank-1 and rank-2 constants can be joined");
    const unsigned r = c.shape().size() == 2 ? c.shape(0) : 1;
    const unsigned wcols = c.shape(c.shape().size() - 1);
    if (parts.empty()) {
      rows = r;
      rank1 = c.shape().size() == 1;
    } else if (r != rows || rank1 != (c.shape().size() == 1)) {
      throw InvalidArgumentError("constants to join don't match");
    }
    parts.push_back(data::get(c));
    widths.push_back(wcols);
    total += wcols;
  }
  std::vector<float> joined(static_cast<size_t>(rows) * total);
  for (unsigned r = 0; r < rows; ++r) {
    size_t at = static_cast<size_t>(r) * total;
    for (size_t i = 0; i < parts.size(); ++i) {
      std::copy(parts[i].begin() + static_cast<size_t>(r) * widths[i],
                parts[i].begin() + static_cast<size_t>(r + 1) * widths[i], joined.begin() + at);
      at += widths[i];
    }
  }
  Shape shape = rank1 ? Shape({total}) : Shape({rows, total});
  Constant<float>::setRuntimeConstantIfNotExist(packedName, shape, joined);
  return *Constant<float>::tryGetRuntimeConstant(packedName);
}

namespace parallel {

NSplitGroup::NSplitGroup(const std::vector<unsigned>& deviceIDs) : _group(nullptr), _devices(deviceIDs) {
  std::vector<int> devs(deviceIDs.begin(), deviceIDs.end());
  tfccb200_group* g = nullptr;
  check_status(tfccb200_group_create(static_cast<int>(devs.size()), devs.data(), &g));
  _group = g;
}

NSplitGroup::~NSplitGroup() {
  if (_group) tfccb200_group_destroy(static_cast<tfccb200_group*>(_group));
}

cudaStream_t NSplitGroup::stream(size_t member) const {
  return static_cast<cudaStream_t>(
      tfccb200_group_stream(static_cast<tfccb200_group*>(_group), static_cast<int>(member)));
}

void NSplitGroup::matmul_host(const float* a, const float* b, float* c, unsigned m, unsigned n,
                              unsigned k) {
  check_status(tfccb200_group_sgemm_nsplit_host(static_cast<tfccb200_group*>(_group), a, b, c, m, n,
                                                k, TFCCB200_PRECISION_FP32));
}

void NSplitGroup::matmul(const std::vector<const float*>& a, const std::vector<const float*>& bShards,
                         const std::vector<float*>& c, unsigned m, unsigned nShard, unsigned k) {
  if (a.size() != size() || bShards.size() != size() || c.size() != size())
    throw InvalidArgumentError("one operand per group member is required");
  check_status(tfccb200_group_sgemm_nsplit(static_cast<tfccb200_group*>(_group), a.data(),
                                           bShards.data(), c.data(), nullptr, m, nShard, k,
                                           TFCCB200_PRECISION_FP32));
}

void NSplitGroup::sync() { check_status(tfccb200_group_sync(static_cast<tfccb200_group*>(_group))); }

}  // namespace parallel

namespace quantization {

// Argument checks and messages of tfcc::mkl::quantization::matmul
// (tfcc/mkl/operations/tfcc_mklquantization.cpp:75-118).
std::tuple<Variable<int32_t>, Variable<float>, Variable<float>> matmul(
    const Tensor<uint8_t>& a, const Tensor<int32_t>& reduceSumA, const Tensor<float>& minA,
    const Tensor<float>& maxA, const Tensor<int8_t>& b, const Tensor<int32_t>& reduceSumB,
    const Tensor<float>& minB, const Tensor<float>& maxB) {
  if (a.size() == 0 || a.shape().size() < 2) throw InvalidArgumentError("invalid input tensor a");
  if (reduceSumA.size() == 0) throw InvalidArgumentError("invalid tensor reduceSumA");
  if (minA.size() != 1 || minA.shape().size() != 1) throw InvalidArgumentError("invalid tensor minA");
  if (maxA.size() != 1 || maxA.shape().size() != 1) throw InvalidArgumentError("invalid tensor maxA");
  if (b.size() == 0 || b.shape().size() < 2) throw InvalidArgumentError("invalid input tensor b");
  if (reduceSumB.size() == 0) throw InvalidArgumentError("invalid tensor reduceSumB");
  if (minB.size() != 1 || minB.shape().size() != 1) throw InvalidArgumentError("invalid tensor minB");
  if (maxB.size() != 1 || maxB.shape().size() != 1) throw InvalidArgumentError("invalid tensor maxB");
  if (a.shape(a.shape().size() - 1) != b.shape(b.shape().size() - 2))
    throw InvalidArgumentError("tensor a and b don't match");
  if (a.shape().size() != b.shape().size() && a.shape().size() != 2 && b.shape().size() != 2)
    throw InvalidArgumentError("tensor a and b don't match");
  if (a.shape(a.shape().size() - 2) != reduceSumA.shape(reduceSumA.shape().size() - 1))
    throw InvalidArgumentError("tensor a and reduceSumA don't match");
  if (b.shape(b.shape().size() - 1) != reduceSumB.shape(reduceSumB.shape().size() - 1))
    throw InvalidArgumentError("tensor b and reduceSumB don't match");
  if (a.shape().size() == b.shape().size()) {
    for (size_t i = 0; i + 2 < a.shape().size(); ++i)
      if (a.shape(i) != b.shape(i)) throw InvalidArgumentError("tensor a and b don't match");
  }

  MatmulGeometry g = matmul_geometry(a, b);
  const unsigned strideRsA = reduceSumA.shape().size() == 1 ? 0 : g.m;
  const unsigned strideRsB = reduceSumB.shape().size() == 1 ? 0 : g.n;
  // rank-2 operands are shared over the batch even when both ranks are equal to 2
  const unsigned strideA = a.shape().size() == 2 ? 0 : g.m * g.k;
  const unsigned strideB = b.shape().size() == 2 ? 0 : g.k * g.n;

  Variable<int32_t> result(Shape(g.resultShape));
  Variable<float> minResult({1}), maxResult({1});
  B200Session* session = current_session();

  // The ranges live in device memory: offsets and result range are derived there by the
  // library's prologue kernel, the GEMM reads them from device memory, and no value returns
  // to the host -- the call stays asynchronous like every other operator of the backend.
  Variable<int32_t> offsets({2});
  check_status(tfccb200_qgemm_u8s8s32_dev(
      session->stream(), a.data(), strideA, reduceSumA.data(), strideRsA, minA.data(), maxA.data(),
      b.data(), strideB, reduceSumB.data(), strideRsB, minB.data(), maxB.data(), result.data(),
      g.m * g.n, minResult.data(), maxResult.data(), offsets.data(), g.m, g.n, g.k, g.batch,
      TFCCB200_PATH_AUTO, session->deviceStatus()));
  return std::make_tuple(std::move(result), std::move(minResult), std::move(maxResult));
}

template <class T>
struct ReduceEntry;
template <>
struct ReduceEntry<int8_t> {
  static int call(void* s, const int8_t* p, unsigned b, unsigned r, unsigned c, int f, int32_t* d) {
    return tfccb200_reduce_sum_s8(s, p, b, r, c, f, d);
  }
};
template <>
struct ReduceEntry<uint8_t> {
  static int call(void* s, const uint8_t* p, unsigned b, unsigned r, unsigned c, int f, int32_t* d) {
    return tfccb200_reduce_sum_u8(s, p, b, r, c, f, d);
  }
};
template <>
struct ReduceEntry<int16_t> {
  static int call(void* s, const int16_t* p, unsigned b, unsigned r, unsigned c, int f, int32_t* d) {
    return tfccb200_reduce_sum_s16(s, p, b, r, c, f, d);
  }
};

// tfcc::mkl::quantization::reduce_sum (tfcc_mklquantization.cpp:284-318).
template <class T>
Variable<int32_t> reduce_sum(const Tensor<T>& a, bool row) {
  if (a.size() == 0 || a.shape().size() < 2) throw InvalidArgumentError("invalid input tensor a");
  std::vector<unsigned> newS = a.shape().toVector();
  newS.pop_back();
  newS.pop_back();
  const unsigned r = a.shape(a.shape().size() - 2);
  const unsigned c = a.shape(a.shape().size() - 1);
  const unsigned batch = a.size() / r / c;
  newS.push_back(row ? r : c);
  Variable<int32_t> result(Shape(std::move(newS)));
  check_status(ReduceEntry<T>::call(current_session()->stream(), a.data(), batch, r, c, row ? 1 : 0,
                                    result.data()));
  return result;
}

template Variable<int32_t> reduce_sum(const Tensor<int8_t>& a, bool row);
template Variable<int32_t> reduce_sum(const Tensor<uint8_t>& a, bool row);
template Variable<int32_t> reduce_sum(const Tensor<int16_t>& a, bool row);

}  // namespace quantization
}  // namespace b200

}  // namespace tfcc
