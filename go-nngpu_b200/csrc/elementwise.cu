// Element-wise family of the dense path's callers: add / subtract / multiply /
// divide of equal-shaped matrices, scalar add / multiply, the sigmoid, tanh,
// leaky-ReLU, ELU, Swish and GELU activations with their derivatives, and the
// row softmax.  In the reference these are CPU loops over the shared buffer
// (internal/cgo/metal_bridge_matrix.m:172-543, metal_bridge_activation.m:83-703);
// here they are HBM-bound streaming kernels (16-byte accesses, grid-stride), so
// that a chain of eager layers stays on the device between its GEMMs.
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

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
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
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
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
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
// GROUP threads share one row: 4, 8, 16 or 32 lanes of a warp (short rows, several
// rows per warp, so a warp's loads stay contiguous), or the whole 256-thread block.
// Forward is the reference's formula, y = expf(x - rowmax) / sum
// (metal_bridge_activation.m:300-321), as three reads of x and ONE write of y: the
// second and third read hit L1/L2, so HBM sees one read and one write per element.
// Backward is grad_in = y * (grad_out - dot(grad_out, y)) (:349-362).  VEC: 16-byte
// accesses (block-per-row form, features a multiple of 4, 16-byte aligned rows).
template <int GROUP, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* smem) {
#pragma unroll
  for (int o = (GROUP < 32 ? GROUP : 32) / 2; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, w) : v + w;
  }
  if (GROUP <= 32) return v;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // smem is reused by successive reductions
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = smem[0];
#pragma unroll
  for (int w = 1; w < 8; w++) r = IS_MAX ? fmaxf(r, smem[w]) : r + smem[w];
  return r;
}

template <int GROUP, bool VEC>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float* in, float* out, uint64_t rows,
                                                          uint64_t features) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  __shared__ float smem[8];
  constexpr int per_block = 256 / GROUP;
  const int sub = threadIdx.x / GROUP, lane = threadIdx.x % GROUP;
  for (uint64_t base = uint64_t(blockIdx.x) * per_block; base < rows; base += uint64_t(gridDim.x) * per_block) {
    const uint64_t row = base + sub;
    const bool live = row < rows;  // a group is never split across rows
    const float* x = in + (live ? row : 0) * features;
    float* y = out + (live ? row : 0) * features;
    float m = -INFINITY, sum = 0.f;
    if (VEC) {
      const float4* x4 = reinterpret_cast<const float4*>(x);
      const uint64_t q = features >> 2;
      for (uint64_t i = lane; live && i < q; i += GROUP) {
        const float4 v = x4[i];
        m = fmaxf(m, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
      }
      m = group_reduce<GROUP, true>(m, smem);
      for (uint64_t i = lane; live && i < q; i += GROUP) {
        const float4 v = x4[i];
        sum += (expf(v.x - m) + expf(v.y - m)) + (expf(v.z - m) + expf(v.w - m));
      }
      sum = group_reduce<GROUP, false>(sum, smem);
      for (uint64_t i = lane; live && i < q; i += GROUP) {
        const float4 v = x4[i];
        reinterpret_cast<float4*>(y)[i] =
            make_float4(expf(v.x - m) / sum, expf(v.y - m) / sum, expf(v.z - m) / sum, expf(v.w - m) / sum);
      }
    } else {
      for (uint64_t i = lane; live && i < features; i += GROUP) m = fmaxf(m, x[i]);
      m = group_reduce<GROUP, true>(m, smem);
      for (uint64_t i = lane; live && i < features; i += GROUP) sum += expf(x[i] - m);
      sum = group_reduce<GROUP, false>(sum, smem);
      for (uint64_t i = lane; live && i < features; i += GROUP) y[i] = expf(x[i] - m) / sum;
    }
  }
}

template <int GROUP, bool VEC>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float* grad_out, const float* act,
                                                          float* grad_in, uint64_t rows,
                                                          uint64_t features) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  __shared__ float smem[8];
  constexpr int per_block = 256 / GROUP;
  const int sub = threadIdx.x / GROUP, lane = threadIdx.x % GROUP;
  for (uint64_t base = uint64_t(blockIdx.x) * per_block; base < rows; base += uint64_t(gridDim.x) * per_block) {
    const uint64_t row = base + sub;
    const bool live = row < rows;
    const float* g = grad_out + (live ? row : 0) * features;
    const float* y = act + (live ? row : 0) * features;
    float* o = grad_in + (live ? row : 0) * features;
    float dot = 0.f;
    if (VEC) {
      const uint64_t q = features >> 2;
      for (uint64_t i = lane; live && i < q; i += GROUP) {
        const float4 a = reinterpret_cast<const float4*>(g)[i], b = reinterpret_cast<const float4*>(y)[i];
        dot += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
      }
      dot = group_reduce<GROUP, false>(dot, smem);
      for (uint64_t i = lane; live && i < q; i += GROUP) {
        const float4 a = reinterpret_cast<const float4*>(g)[i], b = reinterpret_cast<const float4*>(y)[i];
        reinterpret_cast<float4*>(o)[i] =
            make_float4(b.x * (a.x - dot), b.y * (a.y - dot), b.z * (a.z - dot), b.w * (a.w - dot));
      }
    } else {
      for (uint64_t i = lane; live && i < features; i += GROUP) dot += g[i] * y[i];
      dot = group_reduce<GROUP, false>(dot, smem);
      for (uint64_t i = lane; live && i < features; i += GROUP) o[i] = y[i] * (g[i] - dot);
    }
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
  case OPC: launch_kernel(ew_kernel<OPC>, dim3(uint32_t(grid)), dim3(256), 0, stream, a, b, c, n, scalar, vec); break;
  switch (op) {
    GONN_EW(EW_ADD) GONN_EW(EW_SUB) GONN_EW(EW_MUL) GONN_EW(EW_DIV) GONN_EW(EW_SCALAR_ADD)
    GONN_EW(EW_SCALAR_MUL) GONN_EW(EW_SIGMOID) GONN_EW(EW_SIGMOID_BWD) GONN_EW(EW_TANH)
    GONN_EW(EW_TANH_BWD) GONN_EW(EW_LEAKY) GONN_EW(EW_LEAKY_BWD) GONN_EW(EW_ELU) GONN_EW(EW_ELU_BWD)
    GONN_EW(EW_SWISH) GONN_EW(EW_SWISH_BWD) GONN_EW(EW_GELU) GONN_EW(EW_GELU_BWD)
    default: break;
  }
#undef GONN_EW
}

// Register-cached form for rows of at most GROUP * PER units (a unit is one float,
// or a float4 with VEC): x is read from memory exactly once, R rows per group are in
// flight at a time so that short rows still keep enough loads outstanding.
template <int GROUP, int PER, bool VEC, int R, bool BWD>
__global__ void __launch_bounds__(256) softmax_reg_kernel(const float* in_or_grad, const float* act,
                                                          float* out, uint64_t rows, uint64_t features) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  __shared__ float smem[8];
  constexpr int per_block = 256 / GROUP;
  constexpr int W = VEC ? 4 : 1;
  const int sub = threadIdx.x / GROUP, lane = threadIdx.x % GROUP;
  const uint64_t units = VEC ? features >> 2 : features;
  for (uint64_t base = uint64_t(blockIdx.x) * per_block * R; base < rows;
       base += uint64_t(gridDim.x) * per_block * R) {
    float a[R][PER][W], b[BWD ? R : 1][BWD ? PER : 1][W];
    bool live[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint64_t row = base + uint64_t(r) * per_block + sub;
      live[r] = row < rows;
      const float* x = in_or_grad + (live[r] ? row : 0) * features;
      const float* y = BWD ? act + (live[r] ? row : 0) * features : nullptr;
#pragma unroll
      for (int k = 0; k < PER; k++) {
        const uint64_t i = uint64_t(lane) + uint64_t(k) * GROUP;
        const bool in_row = live[r] && i < units;
        if (VEC) {
          float4 v = BWD ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
          if (in_row) v = reinterpret_cast<const float4*>(x)[i];
          a[r][k][0] = v.x; a[r][k][W > 1 ? 1 : 0] = v.y; a[r][k][W > 1 ? 2 : 0] = v.z; a[r][k][W > 1 ? 3 : 0] = v.w;
          if (BWD) {
            float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
            if (in_row) u = reinterpret_cast<const float4*>(y)[i];
            b[r][k][0] = u.x; b[r][k][W > 1 ? 1 : 0] = u.y; b[r][k][W > 1 ? 2 : 0] = u.z; b[r][k][W > 1 ? 3 : 0] = u.w;
          }
        } else {
          a[r][k][0] = in_row ? x[i] : (BWD ? 0.f : -INFINITY);
          if (BWD) b[r][k][0] = in_row ? y[i] : 0.f;
        }
      }
    }
    float red[R], scale[R];
    if (!BWD) {
#pragma unroll
      for (int r = 0; r < R; r++) {
        float m = -INFINITY;
#pragma unroll
        for (int k = 0; k < PER; k++)
#pragma unroll
          for (int w = 0; w < W; w++) m = fmaxf(m, a[r][k][w]);
        red[r] = m;
      }
#pragma unroll
      for (int r = 0; r < R; r++) red[r] = group_reduce<GROUP, true>(red[r], smem);
#pragma unroll
      for (int r = 0; r < R; r++) {
        const float m = live[r] ? red[r] : 0.f;  // keeps -inf - -inf out of dead rows
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < PER; k++)
#pragma unroll
          for (int w = 0; w < W; w++) {
            a[r][k][w] = expf(a[r][k][w] - m);   // padding: expf(-inf) = 0
            s += a[r][k][w];
          }
        scale[r] = s;
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; r++) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < PER; k++)
#pragma unroll
          for (int w = 0; w < W; w++) s += a[r][k][w] * b[r][k][w];
        scale[r] = s;
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) scale[r] = group_reduce<GROUP, false>(scale[r], smem);
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint64_t row = base + uint64_t(r) * per_block + sub;
      float* o = out + (live[r] ? row : 0) * features;
#pragma unroll
      for (int k = 0; k < PER; k++) {
        const uint64_t i = uint64_t(lane) + uint64_t(k) * GROUP;
        if (!(live[r] && i < units)) continue;
        float res[W];
#pragma unroll
        for (int w = 0; w < W; w++)
          res[w] = BWD ? b[r][k][w] * (a[r][k][w] - scale[r]) : a[r][k][w] / scale[r];
        if (VEC) reinterpret_cast<float4*>(o)[i] = make_float4(res[0], res[W > 1 ? 1 : 0], res[W > 1 ? 2 : 0], res[W > 1 ? 3 : 0]);
        else o[i] = res[0];
      }
    }
  }
}

template <int GROUP, int PER, bool VEC, int R>
void softmax_reg_dispatch(const float* in_or_grad, const float* act, float* out, uint64_t rows,
                          uint64_t features, bool backward, cudaStream_t stream) {
  const uint64_t per_iter = uint64_t(256 / GROUP) * R;
  uint64_t grid = (rows + per_iter - 1) / per_iter;
  if (grid > 148 * 8) grid = 148 * 8;
  if (backward)
    launch_kernel(softmax_reg_kernel<GROUP, PER, VEC, R, true>, dim3(uint32_t(grid)), dim3(256), 0, stream, in_or_grad, act, out, rows, features);
  else
    launch_kernel(softmax_reg_kernel<GROUP, PER, VEC, R, false>, dim3(uint32_t(grid)), dim3(256), 0, stream, in_or_grad, act, out, rows, features);
}

template <int GROUP, bool VEC>
void softmax_dispatch(const float* in_or_grad, const float* act, float* out, uint64_t rows,
                      uint64_t features, bool backward, cudaStream_t stream) {
  const uint64_t per_block = 256 / GROUP;
  uint64_t grid = (rows + per_block - 1) / per_block;
  if (grid > 148 * 8) grid = 148 * 8;
  if (backward)
    launch_kernel(softmax_bwd_kernel<GROUP, VEC>, dim3(uint32_t(grid)), dim3(256), 0, stream, in_or_grad, act, out, rows, features);
  else
    launch_kernel(softmax_fwd_kernel<GROUP, VEC>, dim3(uint32_t(grid)), dim3(256), 0, stream, in_or_grad, out, rows, features);
}

void launch_softmax(const float* in_or_grad, const float* act, float* out, uint64_t rows,
                    uint64_t features, bool backward, cudaStream_t stream) {
  if (rows == 0 || features == 0) return;
  const bool vec_ok = (features & 3) == 0 && aligned16(in_or_grad) && aligned16(out) && (!act || aligned16(act));
#define GONN_REG(G, P, V, R) \
  softmax_reg_dispatch<G, P, V, R>(in_or_grad, act, out, rows, features, backward, stream)
#define GONN_SM(G, V) softmax_dispatch<G, V>(in_or_grad, act, out, rows, features, backward, stream)
  if (vec_ok && features <= 16) GONN_REG(4, 1, true, 4);
  else if (vec_ok && features <= 32) GONN_REG(8, 1, true, 4);
  else if (vec_ok && features <= 128) GONN_REG(32, 1, true, 2);
  else if (vec_ok && features <= 512) GONN_REG(32, 4, true, 1);
  else if (features <= 4) GONN_REG(4, 1, false, 8);
  else if (features <= 8) GONN_REG(8, 1, false, 8);
  else if (features <= 16) GONN_REG(16, 1, false, 8);
  else if (features <= 32) GONN_REG(32, 1, false, 8);
  else if (features <= 128) GONN_REG(32, 4, false, 2);
  else if (features <= 512) GONN_REG(32, 16, false, 1);
  else if (vec_ok && features <= 2048) GONN_REG(256, 2, true, 1);
  else if (vec_ok && features <= 8192) GONN_REG(256, 8, true, 1);
  else if (features <= 1024) GONN_REG(256, 4, false, 1);
  else if (features <= 4096) GONN_REG(256, 16, false, 1);
  else if (vec_ok) GONN_SM(256, true);   // long rows: three passes, the later ones from L1/L2
  else GONN_SM(256, false);
#undef GONN_REG
#undef GONN_SM
}

void launch_first_zero(const float* b, uint64_t n, unsigned long long* out, cudaStream_t stream) {
  if (n == 0) return;
  uint64_t grid = (n + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  launch_kernel(first_zero_kernel, dim3(uint32_t(grid)), dim3(256), 0, stream, b, n, out);
}

}  // namespace gonn
