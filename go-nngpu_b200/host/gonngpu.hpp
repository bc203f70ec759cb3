// Host-side mirror, in C++17, of the Go API that sits above the C ABI on the
// reference's dense path.  The reference's host code is Go (not installed on
// the build machine), so this header restates the same types, function names,
// argument meaning and error behaviour; a Go `error` return becomes a thrown
// gonngpu::Error with the reference's message text, a Go `panic` becomes a
// thrown gonngpu::Panic.
//
//   namespace tensor  <- tensor/tensor.go
//   namespace mat     <- the slice of gonum's mat package the reference touches
//   namespace matrix  <- gpu/matrix/{matrix,gonum-compat,fused-operations,
//                        optimized-kernels,mixed-precision,layers}.go
//
// Header only; link with -lgonngpu_cuda.  Nothing here computes on the CPU:
// every operation is a call into the library (and fails if it does).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/gonngpu.h"

namespace gonngpu {

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
struct Panic : std::runtime_error {
  using std::runtime_error::runtime_error;
};

namespace detail {
// Reads and frees a CError message (the caller owns it, as in the Go callers:
// gpu/matrix/matrix.go:95-102).
inline std::string take_message(CError& e) {
  std::string s;
  if (e.message) {
    s = e.message;
    free_c_error_message(e.message);
    e.message = nullptr;
  }
  return s;
}
}  // namespace detail
}  // namespace gonngpu

namespace tensor {

// tensor/tensor.go:22-77: every GPU buffer a Tensor creates is recorded here (pointer ->
// bytes), with the running total and its peak.  EnsureGPU records (tensor.go:146-147),
// ReleaseGPU removes (tensor.go:195-196).
class GlobalMemoryPool {
 public:
  void trackAllocation(const void* ptr, int64_t size) {  // tensor.go:43-52
    std::lock_guard<std::mutex> lk(mu_);
    allocations_[ptr] = size;
    total_ += size;
    if (total_ > peak_) peak_ = total_;
  }
  void trackDeallocation(const void* ptr) {  // tensor.go:55-63
    std::lock_guard<std::mutex> lk(mu_);
    auto it = allocations_.find(ptr);
    if (it != allocations_.end()) {
      total_ -= it->second;
      allocations_.erase(it);
    }
  }
  struct Stats {
    int64_t currentUsage, peakUsage;
    int numAllocations;
  };
  Stats GetStats() {  // tensor.go:66-71
    std::lock_guard<std::mutex> lk(mu_);
    return Stats{total_, peak_, int(allocations_.size())};
  }

 private:
  std::map<const void*, int64_t> allocations_;
  int64_t total_ = 0, peak_ = 0;
  std::mutex mu_;
};
inline GlobalMemoryPool& getGlobalMemoryPool() {  // tensor.go:37-40
  static GlobalMemoryPool pool;
  return pool;
}
// tensor.go:74-77
inline GlobalMemoryPool::Stats GetGlobalMemoryStats() { return getGlobalMemoryPool().GetStats(); }

// tensor/tensor.go:80-87.  Shape and Data are public as in Go.  Data is the
// host copy; after an operation wrote the tensor on the device, call
// RetrieveCPU() before reading Data (the protocol tensor.go states; on Apple
// silicon the reference gets away without it because the buffer aliases Data).
class Tensor {
 public:
  std::vector<int> Shape;
  std::vector<float> Data;

  Tensor(std::vector<int> shape, std::vector<float> data)
      : Shape(std::move(shape)), Data(std::move(data)) {}
  Tensor(const Tensor&) = delete;
  Tensor& operator=(const Tensor&) = delete;
  ~Tensor() { dropBuffer(); }

  // tensor.go:113-150
  void EnsureGPU() {
    if (isOnGPU_) return;
    // The reference leaves the old buffer behind after RetrieveCPU (tensor.go:154-184
    // keeps gpuPtr); here it is released so that nothing leaks, and a new buffer
    // registers the possibly modified Data.
    dropBuffer();
    CError err{nullptr};
    GPUPtr p = nullptr;
    DevicePtr d = nullptr;
    static float dummy = 0.f;
    float* data = Data.empty() ? &dummy : Data.data();
    const int rc = create_gpu_buffer(data, long(Data.size() * sizeof(float)), &p, &d, &err);
    if (rc != 0)
      throw gonngpu::Error("failed to create GPU buffer (code " + std::to_string(rc) +
                           "): " + gonngpu::detail::take_message(err));
    gpuPtr_ = p;
    devicePtr_ = d;
    isOnGPU_ = true;
    getGlobalMemoryPool().trackAllocation(p, int64_t(Data.size() * sizeof(float)));
  }

  // Number of elements the shape describes.
  size_t Size() const {
    size_t n = 1;
    for (int d : Shape) n *= size_t(d);
    return n;
  }

  // tensor.go:154-184.  A result tensor made on the device (NewDeviceTensor) gets its host
  // slice here, the first time someone asks for the values.
  void RetrieveCPU() {
    if (!isOnGPU_) return;
    if (!gpuPtr_) throw gonngpu::Error("tensor is marked as on GPU but has no GPU pointer");
    if (Data.size() != Size()) Data.resize(Size());
    CError err{nullptr};
    const int rc =
        retrieve_gpu_buffer_data(gpuPtr_, Data.data(), long(Data.size() * sizeof(float)), &err);
    if (rc != 0)
      throw gonngpu::Error("failed to retrieve GPU buffer data (code " + std::to_string(rc) +
                           "): " + gonngpu::detail::take_message(err));
    isOnGPU_ = false;
  }

  // tensor.go:189-202
  void ReleaseGPU() {
    dropBuffer();
    isOnGPU_ = false;
  }

  // Takes over a device buffer that already holds this tensor's values (Data is
  // stale until RetrieveCPU).  No counterpart in the reference, whose buffers
  // always alias Data; used by the float64 facade to skip the host conversion.
  void AdoptGPU(GPUPtr p, DevicePtr d) {
    ReleaseGPU();
    gpuPtr_ = p;
    devicePtr_ = d;
    isOnGPU_ = true;
    getGlobalMemoryPool().trackAllocation(p, int64_t(Size() * sizeof(float)));
  }

  GPUPtr GPUPointer() const { return gpuPtr_; }        // tensor.go:206 (GPUPtr)
  DevicePtr DevicePointer() const { return devicePtr_; }  // tensor.go:212 (DevicePtr)
  bool IsOnGPU() const { return isOnGPU_; }

 private:
  void dropBuffer() {
    if (!gpuPtr_) return;
    getGlobalMemoryPool().trackDeallocation(gpuPtr_);
    release_gpu_buffer(gpuPtr_);
    gpuPtr_ = nullptr;
  }
  GPUPtr gpuPtr_ = nullptr;
  DevicePtr devicePtr_ = nullptr;
  bool isOnGPU_ = false;
};

using TensorPtr = std::shared_ptr<Tensor>;

// tensor.go:90-109
inline TensorPtr NewTensor(std::vector<int> shape, std::vector<float> data) {
  size_t size = 1;
  for (int d : shape) size *= size_t(d);
  if (data.size() != size)
    throw gonngpu::Error("data length (" + std::to_string(data.size()) +
                         ") does not match shape dimensions (" + std::to_string(size) + ")");
  return std::make_shared<Tensor>(std::move(shape), std::move(data));
}

// A result tensor that starts its life on the device: the buffer is allocated there and no
// host slice is made (or zero-filled) until RetrieveCPU.  The reference's operations build
// their results with make([]float32, n) + NewTensor + EnsureGPU (gpu/matrix/matrix.go:61-79);
// by its own protocol Data of such a tensor is not to be read before RetrieveCPU, so the
// zero-filled slice is only a cost: 17 MB per training step of the small MLP.
inline TensorPtr NewDeviceTensor(std::vector<int> shape) {
  auto t = std::make_shared<Tensor>(std::move(shape), std::vector<float>());
  CError err{nullptr};
  GPUPtr p = nullptr;
  const size_t bytes = t->Size() * sizeof(float);
  const int rc = gonngpu_alloc_device_buffer(long(bytes ? bytes : 4), &p, &err);
  if (rc != 0)
    throw gonngpu::Error("failed to create GPU buffer (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  t->AdoptGPU(p, nullptr);
  return t;
}

}  // namespace tensor

namespace mat {

// The part of gonum's mat.Matrix the reference uses
// (gpu/matrix/gonum-compat.go:30-42: Dims and At).
struct Matrix {
  virtual ~Matrix() = default;
  virtual std::pair<int, int> Dims() const = 0;
  virtual double At(int i, int j) const = 0;
};

// Row-major float64 matrix standing in for gonum's *mat.Dense (NewDense, At,
// Dims, RawData are what the reference touches).
class Dense : public Matrix {
 public:
  Dense(int r, int c, std::vector<double> data) : r_(r), c_(c), data_(std::move(data)) {
    if (data_.empty()) data_.assign(size_t(r) * c, 0.0);
    if (data_.size() != size_t(r) * c) throw gonngpu::Panic("mat: bad data length");
  }
  std::pair<int, int> Dims() const override { return {r_, c_}; }
  double At(int i, int j) const override {
    if (i < 0 || i >= r_ || j < 0 || j >= c_) throw gonngpu::Panic("mat: index out of range");
    return data_[size_t(i) * c_ + j];
  }
  const std::vector<double>& RawData() const { return data_; }

 private:
  int r_, c_;
  std::vector<double> data_;
};

inline std::shared_ptr<Dense> NewDense(int r, int c, std::vector<double> data) {
  return std::make_shared<Dense>(r, c, std::move(data));
}

}  // namespace mat

namespace matrix {

using tensor::TensorPtr;

// ---- gpu/matrix/activation.go:18-29 -----------------------------------------
enum ActivationType { ReLU = 0, Sigmoid, Tanh, Softmax, LeakyReLU, ELU, Swish, GELU };

// ---- gpu/matrix/tensor-unified-memory.go:35-175, unified-memory-optimization.go ----------
// A tensor's "unified" buffer: page-locked host memory from allocateSharedMemory plus the
// GPU buffer createGPUBufferFromSharedMemory makes over it (metal_bridge.h:1803-1804).  On
// Apple silicon both sides are the same bytes; here the device keeps its own copy, so
// GetUnifiedCPUData brings the device contents back into the shared memory before it hands
// out the pointer.
class TensorUnifiedMemoryAdapter {
 public:
  explicit TensorUnifiedMemoryAdapter(DevicePtr device) : device_(device) {}
  ~TensorUnifiedMemoryAdapter() {
    for (auto& kv : buffers_) free_buffer(kv.second);
  }

  // tensor-unified-memory.go:65-108
  void EnsureUnifiedGPU(const TensorPtr& t) {
    std::lock_guard<std::mutex> lk(mu_);
    if (buffers_.count(t.get())) {
      ++zeroCopyHits_;
      return;
    }
    const long bytes = long(t->Data.size() * sizeof(float));
    Shared sb;
    sb.cpu = allocateSharedMemory(bytes);
    if (!sb.cpu) throw gonngpu::Error("failed to create unified buffer: failed to allocate shared memory");
    std::memcpy(sb.cpu, t->Data.data(), size_t(bytes));
    sb.gpu = createGPUBufferFromSharedMemory(device_, sb.cpu, bytes);
    if (!sb.gpu) {
      gonngpu_host_free(sb.cpu);
      throw gonngpu::Error("failed to create unified buffer: failed to create GPU buffer from shared memory");
    }
    sb.bytes = bytes;
    buffers_[t.get()] = sb;
    ++zeroCopyHits_;
  }
  // tensor-unified-memory.go:111-121
  GPUPtr GetUnifiedGPUBuffer(const TensorPtr& t) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = buffers_.find(t.get());
    if (it == buffers_.end()) return nullptr;
    ++zeroCopyHits_;
    return it->second.gpu;
  }
  // tensor-unified-memory.go:124-135
  float* GetUnifiedCPUData(const TensorPtr& t) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = buffers_.find(t.get());
    if (it == buffers_.end()) return nullptr;
    ++zeroCopyHits_;
    CError err{nullptr};
    const int rc = retrieve_gpu_buffer_data(it->second.gpu, static_cast<float*>(it->second.cpu),
                                            it->second.bytes, &err);
    if (rc != 0)
      throw gonngpu::Error("failed to retrieve GPU buffer data (code " + std::to_string(rc) +
                           "): " + gonngpu::detail::take_message(err));
    return static_cast<float*>(it->second.cpu);
  }
  // tensor-unified-memory.go:163-171
  void ReleaseUnifiedBuffer(const TensorPtr& t) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = buffers_.find(t.get());
    if (it == buffers_.end()) return;
    free_buffer(it->second);
    buffers_.erase(it);
  }
  long ZeroCopyHits() const { return zeroCopyHits_; }
  size_t NumBuffers() const { return buffers_.size(); }

 private:
  struct Shared {
    void* cpu = nullptr;
    GPUPtr gpu = nullptr;
    long bytes = 0;
  };
  static void free_buffer(Shared& sb) {
    if (sb.gpu) release_gpu_buffer(sb.gpu);
    if (sb.cpu) gonngpu_host_free(sb.cpu);
    sb = Shared{};
  }
  DevicePtr device_;
  std::map<const tensor::Tensor*, Shared> buffers_;
  std::mutex mu_;
  long zeroCopyHits_ = 0;
};

namespace detail {
inline DevicePtr& global_matrix_device() {
  static DevicePtr d = nullptr;
  return d;
}
}  // namespace detail

// tensor-unified-memory.go:57-62: one adapter per process, made for the first device asked.
inline TensorUnifiedMemoryAdapter& GetGlobalTensorAdapter(DevicePtr device) {
  static TensorUnifiedMemoryAdapter adapter(device);
  return adapter;
}
// matrix.go:19-24
inline void SetGlobalMatrixDevice(DevicePtr device) { detail::global_matrix_device() = device; }
// matrix.go:27-37
inline void ensureUnifiedGPU(const TensorPtr& t) {
  if (detail::global_matrix_device()) {
    GetGlobalTensorAdapter(detail::global_matrix_device()).EnsureUnifiedGPU(t);
    return;
  }
  t->EnsureGPU();
}
// matrix.go:40-50
inline GPUPtr getUnifiedGPUPtr(const TensorPtr& t) {
  if (detail::global_matrix_device()) {
    if (GPUPtr p = GetGlobalTensorAdapter(detail::global_matrix_device()).GetUnifiedGPUBuffer(t)) return p;
  }
  return t->GPUPointer();
}

// ---- gpu/matrix/matrix.go ------------------------------------------------------

// matrix.go:53-105.  With a global device set the operands and the result live in unified
// buffers (the result is then read through GetUnifiedCPUData, as in the reference, whose
// result tensor's Data is not the shared memory either).
inline TensorPtr MatMul(const TensorPtr& A, const TensorPtr& B) {
  if (A->Shape.size() != 2 || B->Shape.size() != 2)
    throw gonngpu::Error("MatMul requires 2D tensors (matrices)");
  if (A->Shape[1] != B->Shape[0])
    throw gonngpu::Error("incompatible matrix dimensions for multiplication: A columns (" +
                         std::to_string(A->Shape[1]) + ") != B rows (" +
                         std::to_string(B->Shape[0]) + ")");
  const int rows = A->Shape[0], cols = B->Shape[1];
  // (unified mode copies the host slice into the shared buffer, so it must exist there)
  TensorPtr result = detail::global_matrix_device()
                         ? tensor::NewTensor({rows, cols}, std::vector<float>(size_t(rows) * cols))
                         : tensor::NewDeviceTensor({rows, cols});
  ensureUnifiedGPU(A);
  ensureUnifiedGPU(B);
  ensureUnifiedGPU(result);
  CError err{nullptr};
  const int rc = perform_mps_matrix_multiplication(
      getUnifiedGPUPtr(A), A->Shape[0], A->Shape[1], getUnifiedGPUPtr(B), B->Shape[0], B->Shape[1],
      getUnifiedGPUPtr(result), rows, cols, detail::global_matrix_device(), &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix multiplication failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

// matrix.go:357-404
inline TensorPtr Transpose(const TensorPtr& A) {
  if (A->Shape.size() != 2) throw gonngpu::Error("Transpose requires 2D tensor (matrix)");
  const int orows = A->Shape[1], ocols = A->Shape[0];
  TensorPtr result = tensor::NewDeviceTensor({orows, ocols});
  A->EnsureGPU();
  result->EnsureGPU();
  CError err{nullptr};
  const int rc = perform_mps_matrix_transpose(A->GPUPointer(), A->Shape[0], A->Shape[1],
                                              result->GPUPointer(), orows, ocols,
                                              A->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix transpose failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

// matrix.go:407-548: element-wise Add with the 2-D broadcast patterns the
// bias path uses ([M,N]+[1,N], [1,N]+[M,N], [M,N]+[M,1], [M,1]+[M,N]).
inline TensorPtr AddBroadcast(const TensorPtr& A, const TensorPtr& B) {
  if (A->Shape.size() != 2 || B->Shape.size() != 2)
    throw gonngpu::Error("Add requires 2D tensors (matrices)");
  const int rows = std::max(A->Shape[0], B->Shape[0]), cols = std::max(A->Shape[1], B->Shape[1]);
  TensorPtr result = tensor::NewDeviceTensor({rows, cols});
  A->EnsureGPU();
  B->EnsureGPU();
  result->EnsureGPU();
  CError err{nullptr};
  const int rc = perform_mps_matrix_add_broadcast(
      A->GPUPointer(), A->Shape[0], A->Shape[1], B->GPUPointer(), B->Shape[0], B->Shape[1],
      result->GPUPointer(), rows, cols, A->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix addition with broadcasting failed (code " +
                         std::to_string(rc) + "): " + gonngpu::detail::take_message(err));
  return result;
}

namespace detail {
using BinaryEntry = int (*)(GPUPtr, long, long, GPUPtr, long, long, GPUPtr, long, long, DevicePtr, CError*);
using ScalarEntry = int (*)(GPUPtr, long, long, float, GPUPtr, DevicePtr, CError*);

// Shared body of Sub / Mul / Div and of Add on equal shapes (matrix.go:464-702): a zeroed
// result tensor, all three on the device, one native call.
inline TensorPtr same_shape_op(const TensorPtr& A, const TensorPtr& B, BinaryEntry entry,
                               const char* failed) {
  const int rows = A->Shape[0], cols = A->Shape[1];
  // the divide stops at the first zero divisor and leaves the rest of the (zeroed) result as it is
  TensorPtr result = entry == perform_mps_matrix_element_divide
                         ? tensor::NewTensor({rows, cols}, std::vector<float>(size_t(rows) * cols))
                         : tensor::NewDeviceTensor({rows, cols});
  A->EnsureGPU();
  B->EnsureGPU();
  result->EnsureGPU();
  CError err{nullptr};
  const int rc = entry(A->GPUPointer(), rows, cols, B->GPUPointer(), B->Shape[0], B->Shape[1],
                       result->GPUPointer(), rows, cols, A->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error(std::string(failed) + " failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

inline void require_same_2d(const TensorPtr& A, const TensorPtr& B, const char* op, const char* noun) {
  if (A->Shape.size() != 2 || B->Shape.size() != 2)
    throw gonngpu::Error(std::string(op) + " requires 2D tensors (matrices)");
  if (A->Shape[0] != B->Shape[0] || A->Shape[1] != B->Shape[1])
    throw gonngpu::Error("incompatible matrix dimensions for " + std::string(noun) + ": A (" +
                         std::to_string(A->Shape[0]) + "x" + std::to_string(A->Shape[1]) + ") != B (" +
                         std::to_string(B->Shape[0]) + "x" + std::to_string(B->Shape[1]) + ")");
}

inline TensorPtr scalar_op(const TensorPtr& A, float scalar, ScalarEntry entry, const char* op,
                           const char* failed) {
  if (A->Shape.size() != 2) throw gonngpu::Error(std::string(op) + " requires 2D tensor (matrix)");
  const int rows = A->Shape[0], cols = A->Shape[1];
  TensorPtr result = tensor::NewDeviceTensor({rows, cols});
  A->EnsureGPU();
  result->EnsureGPU();
  CError err{nullptr};
  const int rc = entry(A->GPUPointer(), rows, cols, scalar, result->GPUPointer(), A->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error(std::string(failed) + " failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}
}  // namespace detail

// matrix.go:407-427: equal shapes go to the element-wise entry, the four 2-D broadcast
// patterns (matrix.go:429-461) to the broadcasting one.
inline TensorPtr Add(const TensorPtr& A, const TensorPtr& B) {
  if (A->Shape.size() != 2 || B->Shape.size() != 2)
    throw gonngpu::Error("Add requires 2D tensors (matrices)");
  const auto& a = A->Shape;
  const auto& b = B->Shape;
  const bool same = a[0] == b[0] && a[1] == b[1];
  const bool rows_broadcast = a[0] != b[0] && (a[0] == 1 || b[0] == 1) && a[1] == b[1];
  const bool cols_broadcast = a[0] == b[0] && a[1] != b[1] && (a[1] == 1 || b[1] == 1);
  if (!same && !rows_broadcast && !cols_broadcast)
    throw gonngpu::Error("incompatible matrix dimensions for addition: A (" + std::to_string(a[0]) + "x" +
                         std::to_string(a[1]) + ") vs B (" + std::to_string(b[0]) + "x" +
                         std::to_string(b[1]) + ")");
  if (same) return detail::same_shape_op(A, B, perform_mps_matrix_add, "GPU matrix addition");
  return AddBroadcast(A, B);
}
inline TensorPtr Sub(const TensorPtr& A, const TensorPtr& B) {  // matrix.go:551-600
  detail::require_same_2d(A, B, "Sub", "subtraction");
  return detail::same_shape_op(A, B, perform_mps_matrix_subtract, "GPU matrix subtraction");
}
inline TensorPtr Mul(const TensorPtr& A, const TensorPtr& B) {  // matrix.go:602-651 (element-wise)
  detail::require_same_2d(A, B, "Mul", "element-wise multiplication");
  return detail::same_shape_op(A, B, perform_mps_matrix_element_multiply,
                               "GPU matrix element-wise multiplication");
}
inline TensorPtr Div(const TensorPtr& A, const TensorPtr& B) {  // matrix.go:653-702
  detail::require_same_2d(A, B, "Div", "element-wise division");
  return detail::same_shape_op(A, B, perform_mps_matrix_element_divide, "GPU matrix element-wise division");
}
inline TensorPtr ScalarAdd(const TensorPtr& A, float scalar) {  // matrix.go:704-746
  return detail::scalar_op(A, scalar, perform_mps_matrix_scalar_add, "ScalarAdd", "GPU scalar addition");
}
inline TensorPtr ScalarMul(const TensorPtr& A, float scalar) {  // matrix.go:748-790
  return detail::scalar_op(A, scalar, perform_mps_matrix_scalar_multiply, "ScalarMul",
                           "GPU scalar multiplication");
}

// ---- gpu/matrix/activation.go:56-310 -------------------------------------------------
// ActivationForward / ActivationBackward: one result tensor of the input's shape and the
// native entry the activation type names; Softmax takes 1-D and 2-D tensors only.  The
// backward forms receive the activation OUTPUT, as the native side expects.
inline TensorPtr ActivationForward(const TensorPtr& input, ActivationType type, float alpha) {
  if (input->Shape.empty()) throw gonngpu::Error("cannot apply activation to empty tensor");
  // (checked before any device work here; the reference reports it after EnsureGPU)
  if (type == Softmax && input->Shape.size() > 2)
    throw gonngpu::Error("softmax currently supports only 1D and 2D tensors");
  long n = 1;
  for (int d : input->Shape) n *= d;
  TensorPtr result = tensor::NewDeviceTensor(input->Shape);
  input->EnsureGPU();
  result->EnsureGPU();
  GPUPtr in = input->GPUPointer(), out = result->GPUPointer();
  DevicePtr dev = input->DevicePointer();
  CError err{nullptr};
  int rc = 0;
  switch (type) {
    case ReLU: rc = perform_activation_relu_forward(in, n, out, dev, &err); break;
    case Sigmoid: rc = perform_activation_sigmoid_forward(in, n, out, dev, &err); break;
    case Tanh: rc = perform_activation_tanh_forward(in, n, out, dev, &err); break;
    case LeakyReLU: rc = perform_activation_leaky_relu_forward(in, n, alpha, out, dev, &err); break;
    case ELU: rc = perform_activation_elu_forward(in, n, alpha, out, dev, &err); break;
    case Swish: rc = perform_activation_swish_forward(in, n, out, dev, &err); break;
    case GELU: rc = perform_activation_gelu_forward(in, n, out, dev, &err); break;
    case Softmax:
      if (input->Shape.size() == 1)
        rc = perform_activation_softmax_1d_forward(in, input->Shape[0], out, dev, &err);
      else if (input->Shape.size() == 2)
        rc = perform_activation_softmax_2d_forward(in, input->Shape[0], input->Shape[1], out, dev, &err);
      else
        throw gonngpu::Error("softmax currently supports only 1D and 2D tensors");
      break;
    default: throw gonngpu::Error("unsupported activation type: " + std::to_string(int(type)));
  }
  if (rc != 0)
    throw gonngpu::Error("GPU activation forward failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

inline TensorPtr ActivationBackward(const TensorPtr& gradOutput, const TensorPtr& activationOutput,
                                    ActivationType type, float alpha) {
  if (gradOutput->Shape.empty() || activationOutput->Shape.empty())
    throw gonngpu::Error("cannot compute activation gradient for empty tensors");
  if (gradOutput->Shape.size() != activationOutput->Shape.size())
    throw gonngpu::Error("gradient and activation output must have same dimensions");
  for (size_t i = 0; i < gradOutput->Shape.size(); ++i)
    if (gradOutput->Shape[i] != activationOutput->Shape[i])
      throw gonngpu::Error("gradient and activation output shape mismatch at dimension " + std::to_string(i));
  long n = 1;
  for (int d : gradOutput->Shape) n *= d;
  TensorPtr result = tensor::NewDeviceTensor(gradOutput->Shape);
  gradOutput->EnsureGPU();
  activationOutput->EnsureGPU();
  result->EnsureGPU();
  GPUPtr g = gradOutput->GPUPointer(), a = activationOutput->GPUPointer(), out = result->GPUPointer();
  DevicePtr dev = gradOutput->DevicePointer();
  CError err{nullptr};
  int rc = 0;
  switch (type) {
    case ReLU: rc = perform_activation_relu_backward(g, a, n, out, dev, &err); break;
    case Sigmoid: rc = perform_activation_sigmoid_backward(g, a, n, out, dev, &err); break;
    case Tanh: rc = perform_activation_tanh_backward(g, a, n, out, dev, &err); break;
    case LeakyReLU: rc = perform_activation_leaky_relu_backward(g, a, n, alpha, out, dev, &err); break;
    case ELU: rc = perform_activation_elu_backward(g, a, n, alpha, out, dev, &err); break;
    case Swish: rc = perform_activation_swish_backward(g, a, n, out, dev, &err); break;
    case GELU: rc = perform_activation_gelu_backward(g, a, n, out, dev, &err); break;
    case Softmax:
      if (gradOutput->Shape.size() == 1)
        rc = perform_activation_softmax_1d_backward(g, a, gradOutput->Shape[0], out, dev, &err);
      else if (gradOutput->Shape.size() == 2)
        rc = perform_activation_softmax_2d_backward(g, a, gradOutput->Shape[0], gradOutput->Shape[1], out,
                                                    dev, &err);
      else
        throw gonngpu::Error("softmax currently supports only 1D and 2D tensors");
      break;
    default: throw gonngpu::Error("unsupported activation type: " + std::to_string(int(type)));
  }
  if (rc != 0)
    throw gonngpu::Error("GPU activation backward failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

// ---- gpu/matrix/optimized-kernels.go:21-75 ----------------------------------------
inline TensorPtr OptimizedGEMM(const TensorPtr& A, const TensorPtr& B, float alpha, float beta) {
  if (A->Shape.size() != 2 || B->Shape.size() != 2)
    throw gonngpu::Error("optimized GEMM requires 2D tensors");
  const int M = A->Shape[0], K = A->Shape[1], K2 = B->Shape[0], N = B->Shape[1];
  if (K != K2)
    throw gonngpu::Error("matrix dimensions don't match: A(" + std::to_string(M) + "x" +
                         std::to_string(K) + ") x B(" + std::to_string(K2) + "x" +
                         std::to_string(N) + ")");
  TensorPtr out = tensor::NewTensor({M, N}, std::vector<float>(size_t(M) * N));  // zeros, as in Go
  A->EnsureGPU();
  B->EnsureGPU();
  out->EnsureGPU();
  CError err{nullptr};
  const int rc = perform_optimized_gemm(A->GPUPointer(), B->GPUPointer(), out->GPUPointer(), M, N,
                                        K, alpha, beta, A->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error("optimized GEMM failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return out;
}

// ---- gpu/matrix/fused-operations.go ------------------------------------------------
struct FusedActivationConfig {  // fused-operations.go:24-28
  ActivationType Type = ReLU;
  float Alpha = 0.f;
};
struct FusedLinearConfig {  // fused-operations.go:49-54
  bool Bias = false;
  const FusedActivationConfig* Activation = nullptr;
};

// The Go caller hands its ActivationType enum straight to the native entry
// (fused-operations.go:433-439), whose kernel decodes a different numbering
// (default.metal:488-506); only ReLU agrees.  Callers of this mirror get the
// activation they named: the enum is translated to the native code here.
// Softmax, ELU and Swish have no fused native code.
inline int native_activation_code(ActivationType t) {
  if (int(t) < 0) return GONNGPU_ACT_NONE;  // no activation (the layer stack's plain linear layer)
  switch (t) {
    case ReLU: return 0;
    case LeakyReLU: return 1;
    case Sigmoid: return 2;
    case Tanh: return 3;
    case GELU: return 4;
    default: throw gonngpu::Error("activation has no fused linear kernel");
  }
}

// fused-operations.go:380-465 (FusedLinearActivation.Forward) and :1468-1520
// (GradFusedLinearActivation, forward part).  inputs = {X[B,in], W[in,out], bias[out]?}.
// A nil Activation means ReLU, as in the reference (:433).
inline TensorPtr FusedLinearActivationForward(const std::vector<TensorPtr>& inputs,
                                              const FusedLinearConfig& config) {
  if (inputs.size() < 2)
    throw gonngpu::Error("FusedLinearActivation requires at least input and weight tensors");
  const TensorPtr& X = inputs[0];
  const TensorPtr& W = inputs[1];
  TensorPtr bias = (inputs.size() >= 3 && config.Bias) ? inputs[2] : nullptr;
  if (X->Shape.size() != 2 || W->Shape.size() != 2 || X->Shape[1] != W->Shape[0])
    throw gonngpu::Error("FusedLinearActivation: input and weight shapes do not match");
  const int batch = X->Shape[0], in = X->Shape[1], out = W->Shape[1];
  X->EnsureGPU();
  W->EnsureGPU();
  if (bias) bias->EnsureGPU();
  TensorPtr Y = tensor::NewDeviceTensor({batch, out});
  Y->EnsureGPU();
  int code = 0;
  float alpha = 0.f;
  if (config.Activation) {
    code = native_activation_code(config.Activation->Type);
    alpha = config.Activation->Alpha;
  }
  CError err{nullptr};
  const int rc = perform_fused_linear_activation(
      X->GPUPointer(), batch, in, W->GPUPointer(), out, bias ? bias->GPUPointer() : nullptr, code,
      alpha, Y->GPUPointer(), X->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error("fused linear+activation failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return Y;
}

// Backward GEMMs of a linear layer (layers.go:77-96, gradient.go:601-637):
// dW = X^T . dY and dX = dY . W^T.  The reference materialises the transposes;
// here the GEMM reads the operands transposed in place.
inline TensorPtr MatMulTransposed(const TensorPtr& A, bool transA, const TensorPtr& B, bool transB) {
  if (A->Shape.size() != 2 || B->Shape.size() != 2)
    throw gonngpu::Error("MatMul requires 2D tensors (matrices)");
  const int M = transA ? A->Shape[1] : A->Shape[0], K = transA ? A->Shape[0] : A->Shape[1];
  const int Kb = transB ? B->Shape[1] : B->Shape[0], N = transB ? B->Shape[0] : B->Shape[1];
  if (K != Kb)
    throw gonngpu::Error("incompatible matrix dimensions for multiplication: A columns (" +
                         std::to_string(K) + ") != B rows (" + std::to_string(Kb) + ")");
  TensorPtr result = tensor::NewDeviceTensor({M, N});
  A->EnsureGPU();
  B->EnsureGPU();
  result->EnsureGPU();
  CError err{nullptr};
  const int rc = gonngpu_matmul_ex(A->GPUPointer(), A->Shape[0], A->Shape[1], transA,
                                   B->GPUPointer(), B->Shape[0], B->Shape[1], transB,
                                   result->GPUPointer(), M, N, GONNGPU_FP32_3XTF32, 1.f, 0.f,
                                   nullptr, GONNGPU_ACT_NONE, 0.f, &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix multiplication failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

// gpu/matrix/optimized-kernels.go:78-135.  A[batch,M,K] . B[batch,K,N] -> [batch,M,N].
inline TensorPtr OptimizedBatchMatMul(const TensorPtr& A, const TensorPtr& B) {
  if (A->Shape.size() != 3 || B->Shape.size() != 3)
    throw gonngpu::Error("batch matrix multiplication requires 3D tensors");
  const int batch = A->Shape[0], M = A->Shape[1], K = A->Shape[2], K2 = B->Shape[1], N = B->Shape[2];
  if (A->Shape[0] != B->Shape[0])
    throw gonngpu::Error("batch sizes don't match: " + std::to_string(A->Shape[0]) + " vs " +
                         std::to_string(B->Shape[0]));
  if (K != K2)
    throw gonngpu::Error("matrix dimensions don't match: K=" + std::to_string(K) +
                         " vs K2=" + std::to_string(K2));
  TensorPtr out = tensor::NewDeviceTensor({batch, M, N});
  A->EnsureGPU();
  B->EnsureGPU();
  out->EnsureGPU();
  CError err{nullptr};
  const int rc = perform_batch_matmul_optimized(A->GPUPointer(), B->GPUPointer(), out->GPUPointer(),
                                                batch, M, N, K, A->DevicePointer(), &err);
  if (rc != 0)
    throw gonngpu::Error("optimized batch matrix multiplication failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return out;
}

// The three gradients of a linear layer in one call: what LinearLayer.Backward
// (layers.go:77-96) computes with two Transposes, two MatMuls and sumAlongAxis,
// preceded, when `activationOutput` is given, by ReLULayer.Backward
// (layers.go:133-142).  Returns {gradInput, gradWeight, gradBias}.
struct LinearGradients {
  TensorPtr Input, Weight, Bias;
};
inline LinearGradients LinearBackward(const TensorPtr& input, const TensorPtr& weight,
                                      const TensorPtr& gradOutput,
                                      const TensorPtr& activationOutput = nullptr) {
  if (input->Shape.size() != 2 || weight->Shape.size() != 2 || gradOutput->Shape.size() != 2 ||
      input->Shape[1] != weight->Shape[0] || gradOutput->Shape[0] != input->Shape[0] ||
      gradOutput->Shape[1] != weight->Shape[1])
    throw gonngpu::Error("LinearBackward: shapes of input, weight and gradOutput do not match");
  const int batch = input->Shape[0], in = input->Shape[1], out = weight->Shape[1];
  LinearGradients g;
  g.Input = tensor::NewDeviceTensor({batch, in});
  g.Weight = tensor::NewDeviceTensor({in, out});
  g.Bias = tensor::NewDeviceTensor({out});
  input->EnsureGPU();
  weight->EnsureGPU();
  gradOutput->EnsureGPU();
  if (activationOutput) activationOutput->EnsureGPU();
  g.Input->EnsureGPU();
  g.Weight->EnsureGPU();
  g.Bias->EnsureGPU();
  CError err{nullptr};
  const int rc = gonngpu_linear_backward(
      input->GPUPointer(), weight->GPUPointer(), gradOutput->GPUPointer(),
      activationOutput ? activationOutput->GPUPointer() : nullptr, batch, in, out,
      g.Input->GPUPointer(), g.Weight->GPUPointer(), g.Bias->GPUPointer(), &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix multiplication failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return g;
}

// ---- gpu/matrix/mixed-precision.go ---------------------------------------------------
using FloatMP16 = uint16_t;

// mixed-precision.go:315-358 (ForwardFloat16): fp16-precision inputs, fp32
// accumulate, fp32 result, optional bias.  The reference converts on the host
// (ConvertTensorToFloat16, :192-210, truncating) and multiplies in fp32; here
// the same truncation runs on the device and the product runs on fp16 tensor
// cores, which is the same arithmetic: fp16-representable inputs, fp32 sums.
inline TensorPtr ForwardFloat16(const TensorPtr& input, const TensorPtr& weights,
                                const TensorPtr& bias = nullptr, bool round_to_nearest = false) {
  if (input->Shape.size() != 2 || weights->Shape.size() != 2)
    throw gonngpu::Error("MatMul requires 2D tensors (matrices)");
  if (input->Shape[1] != weights->Shape[0])
    throw gonngpu::Error("incompatible matrix dimensions for multiplication: A columns (" +
                         std::to_string(input->Shape[1]) + ") != B rows (" +
                         std::to_string(weights->Shape[0]) + ")");
  const int M = input->Shape[0], N = weights->Shape[1];
  TensorPtr result = tensor::NewDeviceTensor({M, N});
  input->EnsureGPU();
  weights->EnsureGPU();
  if (bias) bias->EnsureGPU();
  result->EnsureGPU();
  CError err{nullptr};
  const int rc = gonngpu_matmul_ex(
      input->GPUPointer(), input->Shape[0], input->Shape[1], 0, weights->GPUPointer(),
      weights->Shape[0], weights->Shape[1], 0, result->GPUPointer(), M, N,
      round_to_nearest ? GONNGPU_FP16_RN : GONNGPU_FP16_TRUNC, 1.f, 0.f,
      bias ? bias->GPUPointer() : nullptr, GONNGPU_ACT_NONE, 0.f, &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix multiplication failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

// ForwardFloat16's product (fp16-precision inputs, fp32 accumulate) for a tall A, split by rows
// over the GPUs this process sees: the multi-GPU form of the same call, straight from and
// into the tensors' host slices (gonngpu_matmul_sharded).  n_devices 0 = every visible GPU.
// The reference has one device and no counterpart.
inline TensorPtr ForwardFloat16Sharded(const TensorPtr& input, const TensorPtr& weights, int n_devices = 0,
                                       bool round_to_nearest = false) {
  if (input->Shape.size() != 2 || weights->Shape.size() != 2)
    throw gonngpu::Error("MatMul requires 2D tensors (matrices)");
  if (input->Shape[1] != weights->Shape[0])
    throw gonngpu::Error("incompatible matrix dimensions for multiplication: A columns (" +
                         std::to_string(input->Shape[1]) + ") != B rows (" +
                         std::to_string(weights->Shape[0]) + ")");
  input->RetrieveCPU();  // the call reads the host slices
  weights->RetrieveCPU();
  const int M = input->Shape[0], N = weights->Shape[1];
  TensorPtr result = tensor::NewTensor({M, N}, std::vector<float>(size_t(M) * N));
  CError err{nullptr};
  const int rc = gonngpu_matmul_sharded(input->Data.data(), M, input->Shape[1], weights->Data.data(),
                                        weights->Shape[0], N, result->Data.data(),
                                        round_to_nearest ? GONNGPU_FP16_RN : GONNGPU_FP16_TRUNC, n_devices, &err);
  if (rc != 0)
    throw gonngpu::Error("GPU matrix multiplication failed (code " + std::to_string(rc) +
                         "): " + gonngpu::detail::take_message(err));
  return result;
}

// ---- gpu/matrix/mixed-precision-{efficient,fixed,optimized}.go: precision selectors ------
// Thin decisions, by operand size, between the float32 MatMul and a reduced-precision one.
// The thresholds and the host-side "simulated precision" scaling of the result are the
// reference's own.
struct MixedPrecisionConfig {  // mixed-precision.go (DefaultMixedPrecisionConfig)
  bool Enabled = true;
  float LossScale = 65536.0f;
};

class EfficientMixedPrecisionTrainer {  // mixed-precision-efficient.go:14-113
 public:
  explicit EfficientMixedPrecisionTrainer(MixedPrecisionConfig c = {}) : config_(c) {}
  TensorPtr EfficientMatMul(const TensorPtr& A, const TensorPtr& B) const {  // :46-64
    if (!config_.Enabled) return MatMul(A, B);
    const long total = long(A->Shape[0]) * A->Shape[1] + long(B->Shape[0]) * B->Shape[1];
    if (total > 256 * 256) return MatMul(A, B);
    TensorPtr result = MatMul(A, B);  // :67-101 (inPlaceMixedPrecisionMatMul)
    if (result->Data.size() <= size_t(128 * 128)) {
      result->RetrieveCPU();
      for (float& v : result->Data) v = simulateFloat16Precision(v);
    }
    return result;
  }
  static float simulateFloat16Precision(float val) {  // :104-118
    if (val > 65000 || val < -65000) return val * 0.999f;
    if (val < 1e-4f && val > -1e-4f) return val * 0.95f;
    return val * 0.9999f;
  }

 private:
  MixedPrecisionConfig config_;
};

class ZeroCopyMixedPrecisionOps {  // mixed-precision-efficient.go:116-158
 public:
  explicit ZeroCopyMixedPrecisionOps(MixedPrecisionConfig c = {}) : trainer_(c), enabled_(c.Enabled) {}
  TensorPtr OptimalMatMul(const TensorPtr& A, const TensorPtr& B) const {
    if (!enabled_) return MatMul(A, B);
    const long rowsA = A->Shape[0], colsA = A->Shape[1], rowsB = B->Shape[0], colsB = B->Shape[1];
    const double flops = double(rowsA) * colsA * colsB * 2;
    const double bytes = double(rowsA * colsA + rowsB * colsB + rowsA * colsB) * 4;
    if (flops / bytes > 0.5 && rowsA <= 512 && colsB <= 512) return trainer_.EfficientMatMul(A, B);
    return MatMul(A, B);
  }

 private:
  EfficientMixedPrecisionTrainer trainer_;
  bool enabled_;
};

class FixedMixedPrecisionTrainer {  // mixed-precision-fixed.go:10-128
 public:
  explicit FixedMixedPrecisionTrainer(MixedPrecisionConfig c = {}) : config_(c) {}
  TensorPtr OptimalMatMul(const TensorPtr& A, const TensorPtr& B) const {  // :30-76
    if (!config_.Enabled) return MatMul(A, B);
    const long rowsA = A->Shape[0], colsA = A->Shape[1], rowsB = B->Shape[0], colsB = B->Shape[1];
    if (colsA != rowsB)
      throw gonngpu::Error("incompatible matrix dimensions: A[" + std::to_string(rowsA) + "," +
                           std::to_string(colsA) + "] * B[" + std::to_string(rowsB) + "," +
                           std::to_string(colsB) + "]");
    const double flops = double(rowsA) * colsA * colsB * 2;
    const double bytes = double(rowsA * colsA + rowsB * colsB + rowsA * colsB) * 4;
    const long maxDim = std::max(std::max(rowsA, colsA), std::max(rowsB, colsB));
    if (maxDim <= 128 || (maxDim <= 256 && flops / bytes > 1.0)) {
      TensorPtr result = MatMul(A, B);  // :79-100 (simulatedMixedPrecisionMatMul)
      result->RetrieveCPU();
      for (float& v : result->Data) v = fastPrecisionReduction(v);
      return result;
    }
    return MatMul(A, B);
  }
  static float fastPrecisionReduction(float val) {  // :103-124
    const float a = val < 0 ? -val : val;
    if (a > 65000) return val * 0.9999f;
    if (a < 1e-5f) return val * 0.995f;
    return val * 0.99995f;
  }

 private:
  MixedPrecisionConfig config_;
};

class OptimizedMixedPrecisionOps {  // mixed-precision-optimized.go:12-56
 public:
  explicit OptimizedMixedPrecisionOps(MixedPrecisionConfig c = {}) : enabled_(c.Enabled) {}
  TensorPtr MatMulOptimized(const TensorPtr& A, const TensorPtr& B) const {
    if (!enabled_) return MatMul(A, B);
    const long total = long(A->Shape[0]) * A->Shape[1] + long(B->Shape[0]) * B->Shape[1];
    if (total > 512 * 512) return MatMul(A, B);
    return ForwardFloat16(A, B, nullptr);
  }

 private:
  bool enabled_;
};

// ---- gpu/matrix/layers.go: the eager layer stack ---------------------------------------------
struct Layer {  // layers.go (Layer interface)
  virtual ~Layer() = default;
  virtual TensorPtr Forward(const TensorPtr& input) = 0;
  virtual TensorPtr Backward(const TensorPtr& gradOutput) = 0;
  virtual std::vector<TensorPtr> GetParameters() = 0;
  virtual std::vector<TensorPtr> GetGradients() = 0;
};

class Sequential;

// layers.go:10-109.  Forward is input . Weight + Bias in one call on the device (the
// reference multiplies on the GPU and then adds the bias into the result's host slice,
// layers.go:271-279, which only reaches a following GPU operation because its buffers
// alias host memory; here the sum is formed on the device and is what later operations
// read).  Backward forms all three gradients in one call without materialised transposes.
class LinearLayer : public Layer {
 public:
  TensorPtr Weight, Bias, WeightGrad, BiasGrad;
  int InputSize, OutputSize;
  bool UseBias;

  // layers.go:30-52: Xavier-uniform weights, zero bias.  `seed` stands in for Go's global
  // math/rand source.
  LinearLayer(int inputSize, int outputSize, bool useBias, uint32_t seed = 1)
      : InputSize(inputSize), OutputSize(outputSize), UseBias(useBias) {
    std::mt19937 gen(seed);
    std::uniform_real_distribution<float> u(0.f, 1.f);
    const float scale = float(std::sqrt(2.0 / double(inputSize + outputSize)));
    std::vector<float> w(size_t(inputSize) * outputSize);
    for (float& x : w) x = (u(gen) * 2 - 1) * scale;
    Weight = tensor::NewTensor({inputSize, outputSize}, std::move(w));
    if (useBias) Bias = tensor::NewTensor({outputSize}, std::vector<float>(size_t(outputSize)));
  }

  TensorPtr Forward(const TensorPtr& input) override {  // layers.go:55-74
    input_ = input;
    return forward(input, nullptr);
  }
  TensorPtr Backward(const TensorPtr& gradOutput) override {  // layers.go:77-96
    return backward(gradOutput, nullptr);
  }
  std::vector<TensorPtr> GetParameters() override {  // layers.go:99-104
    if (UseBias && Bias) return {Weight, Bias};
    return {Weight};
  }
  std::vector<TensorPtr> GetGradients() override {  // layers.go:107-112
    if (UseBias && BiasGrad) return {WeightGrad, BiasGrad};
    return {WeightGrad};
  }

 private:
  friend class Sequential;
  // `act`: a ReLU folded into this layer's kernels by Sequential, else null
  TensorPtr forward(const TensorPtr& input, const FusedActivationConfig* act) {
    static const FusedActivationConfig identity{ActivationType(-1), 0.f};
    FusedLinearConfig cfg;
    cfg.Bias = UseBias && Bias;
    cfg.Activation = act ? act : &identity;
    std::vector<TensorPtr> in{input, Weight};
    if (cfg.Bias) in.push_back(Bias);
    return FusedLinearActivationForward(in, cfg);
  }
  TensorPtr backward(const TensorPtr& gradOutput, const TensorPtr& activationOutput) {
    if (!input_) throw gonngpu::Panic("Backward called before Forward");
    LinearGradients g = LinearBackward(input_, Weight, gradOutput, activationOutput);
    WeightGrad = g.Weight;
    if (UseBias && Bias) BiasGrad = g.Bias;
    return g.Input;
  }
  TensorPtr input_;
};
inline std::shared_ptr<LinearLayer> NewLinearLayer(int inputSize, int outputSize, bool useBias,
                                                   uint32_t seed = 1) {
  return std::make_shared<LinearLayer>(inputSize, outputSize, useBias, seed);
}

// layers.go:115-152
class ReLULayer : public Layer {
 public:
  TensorPtr Forward(const TensorPtr& input) override {  // layers.go:126-130
    input_ = input;
    output_ = ActivationForward(input, ReLU, 0.f);
    return output_;
  }
  TensorPtr Backward(const TensorPtr& gradOutput) override {  // layers.go:133-142
    if (!input_) throw gonngpu::Panic("Backward called before Forward");
    return ActivationBackward(gradOutput, output_, ReLU, 0.f);
  }
  std::vector<TensorPtr> GetParameters() override { return {}; }
  std::vector<TensorPtr> GetGradients() override { return {}; }

 private:
  friend class Sequential;
  TensorPtr input_, output_;
};
inline std::shared_ptr<ReLULayer> NewReLULayer() { return std::make_shared<ReLULayer>(); }

// layers.go:330-376.  A LinearLayer directly followed by a ReLULayer runs as one fused
// call each way (bias + ReLU in the product's epilogue; the ReLU mask applied while the
// gradient's operand planes are written), with both layers' caches filled as if they had
// run one after the other; every other layer runs through its own Forward / Backward.
class Sequential {
 public:
  explicit Sequential(std::vector<std::shared_ptr<Layer>> layers, bool fuse = true)
      : layers_(std::move(layers)), fuse_(fuse) {}

  TensorPtr Forward(const TensorPtr& input) {  // layers.go:343-349
    TensorPtr out = input;
    for (size_t i = 0; i < layers_.size(); ++i) {
      auto* lin = fuse_ ? dynamic_cast<LinearLayer*>(layers_[i].get()) : nullptr;
      auto* relu = (lin && i + 1 < layers_.size()) ? dynamic_cast<ReLULayer*>(layers_[i + 1].get()) : nullptr;
      if (lin && relu) {
        static const FusedActivationConfig kRelu{ReLU, 0.f};
        lin->input_ = out;
        out = lin->forward(out, &kRelu);
        relu->input_ = out;  // the pre-activation is never stored; Backward needs the output only
        relu->output_ = out;
        ++i;
      } else {
        out = layers_[i]->Forward(out);
      }
    }
    return out;
  }

  TensorPtr Backward(const TensorPtr& gradOutput) {  // layers.go:352-359
    TensorPtr grad = gradOutput;
    for (size_t n = layers_.size(); n > 0; --n) {
      const size_t i = n - 1;
      auto* relu = fuse_ ? dynamic_cast<ReLULayer*>(layers_[i].get()) : nullptr;
      auto* lin = (relu && i > 0) ? dynamic_cast<LinearLayer*>(layers_[i - 1].get()) : nullptr;
      if (relu && lin) {
        if (!relu->input_) throw gonngpu::Panic("Backward called before Forward");
        grad = lin->backward(grad, relu->output_);
        --n;
      } else {
        grad = layers_[i]->Backward(grad);
      }
    }
    return grad;
  }

  std::vector<TensorPtr> GetParameters() {  // layers.go:362-368
    std::vector<TensorPtr> params;
    for (auto& l : layers_)
      for (auto& p : l->GetParameters()) params.push_back(p);
    return params;
  }
  std::vector<TensorPtr> GetGradients() {  // layers.go:371-377
    std::vector<TensorPtr> grads;
    for (auto& l : layers_)
      for (auto& g : l->GetGradients()) grads.push_back(g);
    return grads;
  }

 private:
  std::vector<std::shared_ptr<Layer>> layers_;
  bool fuse_;
};
inline std::shared_ptr<Sequential> NewSequential(std::vector<std::shared_ptr<Layer>> layers) {
  return std::make_shared<Sequential>(std::move(layers));
}

// ---- gpu/matrix/fused-operations.go:1468-1520 (GradFusedLinearActivation) ---------------------
// The slice of the reference's GradientTensor this entry needs (gradient.go:16-40): the
// tensor, whether it wants a gradient, and the function that maps the gradient of the
// output to the gradients of {input, weight, bias}.
struct GradientTensor {
  TensorPtr Tensor;
  bool RequiresGrad = false;
  bool IsLeaf = true;
  std::function<std::vector<TensorPtr>(const TensorPtr&)> BackwardFn;  // GradFn.BackwardFn
};
using GradientTensorPtr = std::shared_ptr<GradientTensor>;

// Forward through the fused kernel; the backward closure returns {dX, dW, db?}.  The
// reference's backward reads the activation mask from its third saved tensor, which this
// function fills with the BIAS (fused-operations.go:491-500 against :1473-1476), and leaves the
// bias gradient to a placeholder; here the mask comes from the saved activation output and
// the bias gradient is the column sum.  ReLU or no activation only (what the mask covers).
inline GradientTensorPtr GradFusedLinearActivation(const GradientTensorPtr& input,
                                                   const GradientTensorPtr& weight,
                                                   const GradientTensorPtr& bias,
                                                   const FusedLinearConfig& config) {
  std::vector<TensorPtr> inputs{input->Tensor, weight->Tensor};
  if (bias) inputs.push_back(bias->Tensor);
  TensorPtr output;
  try {
    output = FusedLinearActivationForward(inputs, config);
  } catch (const gonngpu::Error& e) {
    throw gonngpu::Error(std::string("fused linear+activation forward failed: ") + e.what());
  }
  auto result = std::make_shared<GradientTensor>();
  result->Tensor = output;
  result->IsLeaf = false;
  result->RequiresGrad = input->RequiresGrad || weight->RequiresGrad || (bias && bias->RequiresGrad);
  if (result->RequiresGrad) {
    const bool relu = !config.Activation || config.Activation->Type == ReLU;
    if (!relu && int(config.Activation->Type) >= 0)
      throw gonngpu::Error("GradFusedLinearActivation: backward supports ReLU or no activation");
    TensorPtr x = input->Tensor, w = weight->Tensor;
    const bool with_bias = bias != nullptr;
    result->BackwardFn = [x, w, output, relu, with_bias](const TensorPtr& gradOutput) {
      LinearGradients g = LinearBackward(x, w, gradOutput, relu ? output : nullptr);
      std::vector<TensorPtr> grads{g.Input, g.Weight};
      if (with_bias) grads.push_back(g.Bias);
      return grads;
    };
  }
  return result;
}

// ---- gpu/matrix/gonum-compat.go ---------------------------------------------------------
class GPUDense : public mat::Matrix {
 public:
  explicit GPUDense(TensorPtr t) : tensor_(std::move(t)) {}  // NewGPUDenseFromTensor (:825-827)

  std::pair<int, int> Dims() const override { return {tensor_->Shape[0], tensor_->Shape[1]}; }  // :45-47

  double At(int i, int j) const override {  // :49-59
    tensor_->RetrieveCPU();
    const auto [rows, cols] = Dims();
    if (i < 0 || i >= rows || j < 0 || j >= cols) throw gonngpu::Panic("matrix index out of range");
    return double(tensor_->Data[size_t(i) * cols + j]);
  }

  std::shared_ptr<GPUDense> T() const {  // :61-68
    try {
      return std::make_shared<GPUDense>(Transpose(tensor_));
    } catch (const gonngpu::Error& e) {
      throw gonngpu::Panic(e.what());
    }
  }

  void Set(int i, int j, double v) {  // :71-80
    tensor_->RetrieveCPU();
    const auto [rows, cols] = Dims();
    if (i < 0 || i >= rows || j < 0 || j >= cols) throw gonngpu::Panic("matrix index out of range");
    tensor_->Data[size_t(i) * cols + j] = float(v);
  }

  void Mul(const mat::Matrix& a, const mat::Matrix& b);  // :83-110

  std::shared_ptr<mat::Dense> ToGonum() const {  // :322-334
    const auto [rows, cols] = Dims();
    if (tensor_->IsOnGPU() && tensor_->GPUPointer()) {
      // widened on the device and copied out as float64: no float32 host pass
      std::vector<double> d(size_t(rows) * cols);
      CError err{nullptr};
      const int rc = gonngpu_retrieve_f64(tensor_->GPUPointer(), d.data(), long(d.size()), &err);
      if (rc != 0)
        throw gonngpu::Panic("failed to retrieve GPU buffer data (code " + std::to_string(rc) +
                             "): " + gonngpu::detail::take_message(err));
      return mat::NewDense(rows, cols, std::move(d));
    }
    std::vector<double> d(tensor_->Data.begin(), tensor_->Data.end());
    return mat::NewDense(rows, cols, std::move(d));
  }

  void ReleaseGPU() { tensor_->ReleaseGPU(); }       // :337-339
  TensorPtr GetTensor() const { return tensor_; }    // :820-822

 private:
  mutable TensorPtr tensor_;
};

// gonum-compat.go:14-27
inline std::shared_ptr<GPUDense> NewGPUDense(int rows, int cols, const std::vector<double>& data) {
  std::vector<float> f(data.begin(), data.end());
  try {
    return std::make_shared<GPUDense>(tensor::NewTensor({rows, cols}, std::move(f)));
  } catch (const gonngpu::Error& e) {
    throw gonngpu::Panic(e.what());
  }
}

// gonum-compat.go:30-42
inline std::shared_ptr<GPUDense> FromGonum(const mat::Matrix& m) {
  const auto [rows, cols] = m.Dims();
  if (auto* dense = dynamic_cast<const mat::Dense*>(&m)) {
    // A gonum Dense exposes its float64 backing slice (RawMatrix().Data): it goes to
    // the device as it is and is narrowed there, instead of rows*cols At() calls.
    const std::vector<double>& raw = dense->RawData();
    auto t = tensor::NewTensor({rows, cols}, std::vector<float>(raw.size()));
    CError err{nullptr};
    GPUPtr p = nullptr;
    int rc = gonngpu_alloc_device_buffer(long(raw.size() * sizeof(float)), &p, &err);
    if (rc == 0) {
      rc = gonngpu_upload_f64(p, raw.data(), long(raw.size()), &err);
      if (rc != 0) release_gpu_buffer(p);
    }
    if (rc != 0)
      throw gonngpu::Panic("failed to create GPU buffer (code " + std::to_string(rc) +
                           "): " + gonngpu::detail::take_message(err));
    t->AdoptGPU(p, nullptr);
    return std::make_shared<GPUDense>(t);
  }
  std::vector<double> data(size_t(rows) * cols);
  for (int i = 0; i < rows; ++i)
    for (int j = 0; j < cols; ++j) data[size_t(i) * cols + j] = m.At(i, j);
  return NewGPUDense(rows, cols, data);
}

inline void GPUDense::Mul(const mat::Matrix& a, const mat::Matrix& b) {
  std::shared_ptr<GPUDense> keepA, keepB;
  TensorPtr ta, tb;
  if (auto* ga = dynamic_cast<const GPUDense*>(&a)) {
    ta = ga->tensor_;
  } else {
    keepA = FromGonum(a);
    ta = keepA->tensor_;
  }
  if (auto* gb = dynamic_cast<const GPUDense*>(&b)) {
    tb = gb->tensor_;
  } else {
    keepB = FromGonum(b);
    tb = keepB->tensor_;
  }
  TensorPtr result;
  try {
    result = MatMul(ta, tb);
  } catch (const gonngpu::Error& e) {
    throw gonngpu::Panic(e.what());
  }
  tensor_->ReleaseGPU();
  tensor_ = result;
}

// gonum-compat.go:342-367
inline std::shared_ptr<mat::Dense> GPUMatMul(const mat::Matrix& a, const mat::Matrix& b) {
  auto ga = FromGonum(a);
  auto gb = FromGonum(b);
  TensorPtr result;
  try {
    result = MatMul(ga->GetTensor(), gb->GetTensor());
  } catch (const gonngpu::Error& e) {
    throw gonngpu::Panic(e.what());
  }
  auto out = GPUDense(result).ToGonum();  // float64 straight from the device
  result->ReleaseGPU();
  ga->ReleaseGPU();
  gb->ReleaseGPU();
  return out;
}

// gonum-compat.go:744-752
inline std::vector<std::shared_ptr<mat::Dense>> BatchGPUMatMul(
    const std::vector<std::pair<const mat::Matrix*, const mat::Matrix*>>& operations) {
  std::vector<std::shared_ptr<mat::Dense>> results;
  results.reserve(operations.size());
  for (const auto& op : operations) results.push_back(GPUMatMul(*op.first, *op.second));
  return results;
}

}  // namespace matrix
