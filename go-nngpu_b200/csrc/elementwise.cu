// Element-wise family of the dense path's callers: add / subtract / multiply /
// divide of equal-shaped matrices, scalar add / multiply, and the sigmoid, tanh
// and leaky-ReLU activations with their derivatives.  In the reference these
// are CPU loops over the shared buffer (internal/cgo/metal_bridge_matrix.m:172-543,
// metal_bridge_activation.m:83-430); here they are HBM-bound streaming kernels
// (16-byte accesses, grid-stride), so that a chain of eager layers stays on the
// device between its GEMMs.
#include "kernels.h"

namespace gonn {

namespace {

__device__ __forceinline__ float ew_apply(int op, float a, float b, float s) {
  switch (op) {
    case EW_ADD: return a + b;
    case EW_SUB: return a - b;
    case EW_MUL: return a * b;
    case EW_DIV: return a / b;
    case EW_SCALAR_ADD: return a + s;
    case EW_SCALAR_MUL: return a * s;
    case EW_SIGMOID: {  // metal_bridge_activation.m:105-106: input clamped to [-88, 88]
      const float x = fmaxf(-88.0f, fminf(88.0f, a));
      return 1.0f / (1.0f + expf(-x));
    }
    case EW_SIGMOID_BWD: return a * b * (1.0f - b);  // a = grad_out, b = sigmoid output
    case EW_TANH: {
      const float x = fmaxf(-88.0f, fminf(88.0f, a));
      return tanhf(x);
    }
    case EW_TANH_BWD: return a * (1.0f - b * b);     // b = tanh output
    case EW_LEAKY: return (a > 0.0f) ? a : s * a;
    case EW_LEAKY_BWD: return a * ((b > 0.0f) ? 1.0f : s);  // b = activation output
    default: return a;
  }
}

template <int OP>
__global__ void __launch_bounds__(256) ew_kernel(const float* __restrict__ a,
                                                 const float* __restrict__ b, float* __restrict__ c,
                                                 uint64_t n, float s, int vec) {
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (vec) {
    const uint64_t q = n >> 2;
    for (; i < q; i += stride) {
      const float4 x = __ldcs(reinterpret_cast<const float4*>(a) + i);
      float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
      if (b) y = __ldcs(reinterpret_cast<const float4*>(b) + i);
      float4 r;
      r.x = ew_apply(OP, x.x, y.x, s);
      r.y = ew_apply(OP, x.y, y.y, s);
      r.z = ew_apply(OP, x.z, y.z, s);
      r.w = ew_apply(OP, x.w, y.w, s);
      reinterpret_cast<float4*>(c)[i] = r;
    }
    // tail (n % 4 elements)
    const uint64_t t = (q << 2) + blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (t < n) c[t] = ew_apply(OP, a[t], b ? b[t] : 0.f, s);
  } else {
    for (; i < n; i += stride) c[i] = ew_apply(OP, a[i], b ? b[i] : 0.f, s);
  }
}

// Smallest index whose value is exactly zero (either sign), or n.
__global__ void __launch_bounds__(256) first_zero_kernel(const float* __restrict__ b, uint64_t n,
                                                         unsigned long long* __restrict__ out) {
  unsigned long long best = ~0ull;
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x) {
    if (b[i] == 0.0f) {
      best = i;
      break;  // indices only grow along this thread's stride
    }
  }
  if (best != ~0ull) atomicMin(out, best);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

void launch_elementwise(int op, const float* a, const float* b, float* c, uint64_t n, float scalar,
                        cudaStream_t stream) {
  if (n == 0) return;
  const int vec = aligned16(a) && aligned16(c) && (!b || aligned16(b)) && n >= 4;
  const uint64_t items = vec ? (n >> 2) : n;
  uint64_t grid = (items + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) grid = 1;
#define GONN_EW(OPC) \
  case OPC: ew_kernel<OPC><<<uint32_t(grid), 256, 0, stream>>>(a, b, c, n, scalar, vec); break;
  switch (op) {
    GONN_EW(EW_ADD) GONN_EW(EW_SUB) GONN_EW(EW_MUL) GONN_EW(EW_DIV) GONN_EW(EW_SCALAR_ADD)
    GONN_EW(EW_SCALAR_MUL) GONN_EW(EW_SIGMOID) GONN_EW(EW_SIGMOID_BWD) GONN_EW(EW_TANH)
    GONN_EW(EW_TANH_BWD) GONN_EW(EW_LEAKY) GONN_EW(EW_LEAKY_BWD)
    default: break;
  }
#undef GONN_EW
}

void launch_first_zero(const float* b, uint64_t n, unsigned long long* out, cudaStream_t stream) {
  if (n == 0) return;
  uint64_t grid = (n + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  first_zero_kernel<<<uint32_t(grid), 256, 0, stream>>>(b, n, out);
}

}  // namespace gonn
