// Element-wise family of the dense path's callers: add / subtract / multiply /
// divide of equal-shaped matrices, scalar add / multiply, the sigmoid, tanh,
// leaky-ReLU, ELU, Swish and GELU activations with their derivatives, and the
// row softmax.  In the reference these are CPU loops over the shared buffer
// (internal/cgo/metal_bridge_matrix.m:172-543, metal_bridge_activation.m:83-703);
// here they are HBM-bound streaming kernels (16-byte accesses, grid-stride), so
// that a chain of eager layers stays on the device between its GEMMs.
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
    case EW_ELU:  // metal_bridge_activation.m:456-465
      return (a > 0.0f) ? a : s * (expf(fmaxf(-88.0f, a)) - 1.0f);
    case EW_ELU_BWD: return a * ((b > 0.0f) ? 1.0f : b + s);  // b = ELU output (:496-507)
    case EW_SWISH: {  // :533-539: the clamped input is also the factor
      const float x = fmaxf(-88.0f, fminf(88.0f, a));
      return x * (1.0f / (1.0f + expf(-x)));
    }
    case EW_SWISH_BWD: {  // :570-600: three Newton steps recover x from y = x*sigmoid(x)
      const float y = b;
      if (fabsf(y) < 1e-8f) return a * 0.5f;
      float x = y;
#pragma unroll
      for (int it = 0; it < 3; it++) {
        const float sg = 1.0f / (1.0f + expf(-x));
        const float f = x * sg - y;
        const float df = sg + x * sg * (1.0f - sg);
        if (fabsf(df) > 1e-8f) x = x - f / df;
      }
      const float sg = 1.0f / (1.0f + expf(-x));
      return a * (sg + x * sg * (1.0f - sg));
    }
    case EW_GELU: {  // :625-636
      const float inner = fmaxf(-88.0f, fminf(88.0f, 0.7978845608028654f * (a + 0.044715f * (a * a * a))));
      return 0.5f * a * (1.0f + tanhf(inner));
    }
    case EW_GELU_BWD: {  // :665-699: Newton on GELU(x) = y, then the analytic derivative
      const float k = 0.7978845608028654f, c3 = 0.044715f;
      const float y = b;
      float x = y;
#pragma unroll
      for (int it = 0; it < 3; it++) {
        const float inner = fmaxf(-88.0f, fminf(88.0f, k * (x + c3 * (x * x * x))));
        const float th = tanhf(inner);
        const float f = 0.5f * x * (1.0f + th) - y;
        const float df = 0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * (k * (1.0f + 3.0f * c3 * x * x));
        if (fabsf(df) > 1e-8f) x = x - f / df;
      }
      const float inner = fmaxf(-88.0f, fminf(88.0f, k * (x + c3 * (x * x * x))));
      const float th = tanhf(inner);
      return a * (0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * (k * (1.0f + 3.0f * c3 * x * x)));
    }
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

// ---- row softmax ---------------------------------------------------------------
// GROUP threads share one row (32: a warp, 256: the whole block).  Forward is the
// reference's three passes (row max, exp and sum, divide;
// metal_bridge_activation.m:300-321); backward is
// grad_in = y * (grad_out - dot(grad_out, y)) (:349-362).  A row is read from HBM
// once: later passes hit L1/L2 (a row is at most a few MB here).
template <int GROUP, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, w) : v + w;
  }
  if (GROUP == 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // smem reuse across successive reductions
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = smem[0];
#pragma unroll
  for (int w = 1; w < 8; w++) r = IS_MAX ? fmaxf(r, smem[w]) : r + smem[w];
  return r;
}

template <int GROUP>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float* __restrict__ in,
                                                          float* __restrict__ out, uint64_t rows,
                                                          uint64_t features) {
  __shared__ float smem[8];
  const int per_block = 256 / GROUP;
  const int sub = threadIdx.x / GROUP, lane = threadIdx.x % GROUP;
  for (uint64_t base = uint64_t(blockIdx.x) * per_block; base < rows; base += uint64_t(gridDim.x) * per_block) {
    const uint64_t row = base + sub;
    const bool live = row < rows;  // whole groups only: a warp is never split across rows
    const float* x = in + row * features;
    float* y = out + row * features;
    float m = -INFINITY;
    if (live)
      for (uint64_t i = lane; i < features; i += GROUP) m = fmaxf(m, x[i]);
    m = group_reduce<GROUP, true>(m, smem);
    float sum = 0.f;
    if (live)
      for (uint64_t i = lane; i < features; i += GROUP) {
        const float e = expf(x[i] - m);
        y[i] = e;
        sum += e;
      }
    sum = group_reduce<GROUP, false>(sum, smem);
    if (live)
      for (uint64_t i = lane; i < features; i += GROUP) y[i] = y[i] / sum;  // own writes only
  }
}

template <int GROUP>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float* __restrict__ grad_out,
                                                          const float* __restrict__ act,
                                                          float* __restrict__ grad_in, uint64_t rows,
                                                          uint64_t features) {
  __shared__ float smem[8];
  const int per_block = 256 / GROUP;
  const int sub = threadIdx.x / GROUP, lane = threadIdx.x % GROUP;
  for (uint64_t base = uint64_t(blockIdx.x) * per_block; base < rows; base += uint64_t(gridDim.x) * per_block) {
    const uint64_t row = base + sub;
    const bool live = row < rows;
    const float* g = grad_out + row * features;
    const float* y = act + row * features;
    float dot = 0.f;
    if (live)
      for (uint64_t i = lane; i < features; i += GROUP) dot += g[i] * y[i];
    dot = group_reduce<GROUP, false>(dot, smem);
    if (live)
      for (uint64_t i = lane; i < features; i += GROUP) grad_in[row * features + i] = y[i] * (g[i] - dot);
  }
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
    GONN_EW(EW_TANH_BWD) GONN_EW(EW_LEAKY) GONN_EW(EW_LEAKY_BWD) GONN_EW(EW_ELU) GONN_EW(EW_ELU_BWD)
    GONN_EW(EW_SWISH) GONN_EW(EW_SWISH_BWD) GONN_EW(EW_GELU) GONN_EW(EW_GELU_BWD)
    default: break;
  }
#undef GONN_EW
}

void launch_softmax(const float* in_or_grad, const float* act, float* out, uint64_t rows,
                    uint64_t features, bool backward, cudaStream_t stream) {
  if (rows == 0 || features == 0) return;
  const bool wide = features > 512;  // a block per row once a warp would loop > 16 times
  const uint64_t per_block = wide ? 1 : 8;
  uint64_t grid = (rows + per_block - 1) / per_block;
  if (grid > 148 * 8) grid = 148 * 8;
  if (backward) {
    if (wide) softmax_bwd_kernel<256><<<uint32_t(grid), 256, 0, stream>>>(in_or_grad, act, out, rows, features);
    else softmax_bwd_kernel<32><<<uint32_t(grid), 256, 0, stream>>>(in_or_grad, act, out, rows, features);
  } else {
    if (wide) softmax_fwd_kernel<256><<<uint32_t(grid), 256, 0, stream>>>(in_or_grad, out, rows, features);
    else softmax_fwd_kernel<32><<<uint32_t(grid), 256, 0, stream>>>(in_or_grad, out, rows, features);
  }
}

void launch_first_zero(const float* b, uint64_t n, unsigned long long* out, cudaStream_t stream) {
  if (n == 0) return;
  uint64_t grid = (n + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  first_zero_kernel<<<uint32_t(grid), 256, 0, stream>>>(b, n, out);
}

}  // namespace gonn
