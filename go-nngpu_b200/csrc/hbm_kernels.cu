// HBM-bound kernels of the dense path: Transpose, the operand pre-passes
// (fp32 -> fp16 plane, fp32 -> tf32 hi/lo planes), bias broadcast add, ReLU
// forward/backward and the bias-gradient column sum.  All are pure streaming
// kernels: coalesced 16-byte accesses where alignment allows, scalar edges.
#include <algorithm>
#include <cuda_fp16.h>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace gonn {

namespace {

// ------------------------------------------------------------------ transpose
// out[c, r] = in[r, c]; the element moves of
// internal/cgo/metal_bridge_matrix.m:159-166, tiled through shared memory so
// that both the read of `in` and the write of `out` are coalesced.
constexpr int TT = 64;  // tile edge
constexpr int TG = 8;   // tile rows per band of the block walk

template <bool VEC_IN, bool VEC_OUT>
__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ in,
                                                        float* __restrict__ out, uint32_t rows,
                                                        uint32_t cols, uint32_t tiles_r,
                                                        uint32_t tiles_c) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  __shared__ float tile[TT][TT + 1];  // tile[c][r]
  // Blocks walk bands of TG tile rows column by column, so that the blocks in flight
  // together read TG * 64 input rows and write runs of TG * 256 bytes of every output row
  // they touch (a plain row-major walk writes 256-byte pieces 4 * rows bytes apart).
  const uint32_t band = TG * tiles_c;
  const uint32_t first_r = (blockIdx.x / band) * TG;
  const uint32_t in_band = blockIdx.x % band;
  const uint32_t gsz = min(uint32_t(TG), tiles_r - first_r);
  const uint32_t tr = first_r + in_band % gsz, tc = in_band / gsz;
  const uint32_t r0 = tr * TT, c0 = tc * TT;
  const uint32_t tid = threadIdx.x;

  if (VEC_IN) {
    // 64 rows x 16 float4: thread -> (row = i / 16, c4 = i % 16)
#pragma unroll
    for (uint32_t it = 0; it < 4; ++it) {
      const uint32_t i = tid + it * 256;
      const uint32_t r = i >> 4, c = (i & 15u) << 2;
      if (r0 + r < rows && c0 + c < cols) {  // cols % 4 == 0: the float4 is whole
        const float4 v =
            __ldcs(reinterpret_cast<const float4*>(in + uint64_t(r0 + r) * cols + c0 + c));
        tile[c + 0][r] = v.x;
        tile[c + 1][r] = v.y;
        tile[c + 2][r] = v.z;
        tile[c + 3][r] = v.w;
      }
    }
  } else {
#pragma unroll 4
    for (uint32_t it = 0; it < 16; ++it) {
      const uint32_t i = tid + it * 256;
      const uint32_t r = i >> 6, c = i & 63u;
      if (r0 + r < rows && c0 + c < cols) tile[c][r] = in[uint64_t(r0 + r) * cols + c0 + c];
    }
  }
  __syncthreads();
  if (VEC_OUT) {
#pragma unroll
    for (uint32_t it = 0; it < 4; ++it) {
      const uint32_t i = tid + it * 256;
      const uint32_t c = i >> 4, r = (i & 15u) << 2;
      if (c0 + c < cols && r0 + r < rows) {  // rows % 4 == 0
        float4 v;
        v.x = tile[c][r + 0];
        v.y = tile[c][r + 1];
        v.z = tile[c][r + 2];
        v.w = tile[c][r + 3];
        __stcs(reinterpret_cast<float4*>(out + uint64_t(c0 + c) * rows + r0 + r), v);
      }
    }
  } else {
#pragma unroll 4
    for (uint32_t it = 0; it < 16; ++it) {
      const uint32_t i = tid + it * 256;
      const uint32_t c = i >> 6, r = i & 63u;
      if (c0 + c < cols && r0 + r < rows) out[uint64_t(c0 + c) * rows + r0 + r] = tile[c][r];
    }
  }
}

// ------------------------------------------------------------------ pre-passes
// fp32 -> fp16 by truncation, the bit recipe of Float32ToFloatMP16
// (gpu/matrix/mixed-precision.go:106-151): mantissa bits are dropped, not
// rounded; fp32 subnormals and anything below 2^-25 flush to signed zero;
// overflow gives infinity.
__device__ __forceinline__ uint16_t f32_to_f16_trunc(float f) {
  const uint32_t bits = __float_as_uint(f);
  const uint32_t sign = (bits >> 31) & 1u;
  const uint32_t exp = (bits >> 23) & 0xFFu;
  uint32_t mant = bits & 0x7FFFFFu;
  if (exp == 0) return uint16_t(sign << 15);
  if (exp == 0xFF) {
    return mant == 0 ? uint16_t((sign << 15) | 0x7C00u)
                     : uint16_t((sign << 15) | 0x7C00u | (mant >> 13));
  }
  const int32_t e = int32_t(exp) - 127 + 15;
  if (e >= 31) return uint16_t((sign << 15) | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return uint16_t(sign << 15);
    mant = (mant | 0x800000u) >> uint32_t(1 - e);
    return uint16_t((sign << 15) | (mant >> 13));
  }
  return uint16_t((sign << 15) | (uint32_t(e) << 10) | (mant >> 13));
}

__device__ __forceinline__ uint16_t f32_to_f16(float f, int mode) {
  return mode == F16_TRUNC ? f32_to_f16_trunc(f) : __half_as_ushort(__float2half_rn(f));
}

// Walks the (row, 4-element group) pairs of a matrix with `q` groups per row in steps of
// `stride` pairs without a division per step.
struct RowWalk {
  uint64_t r, g;      // current row and group within the row
  uint64_t dr, dg;    // stride / q, stride % q
  __device__ RowWalk(uint64_t start, uint64_t stride, uint64_t q)
      : r(start / q), g(start % q), dr(stride / q), dg(stride % q) {}
  __device__ __forceinline__ void next(uint64_t q) {
    r += dr;
    g += dg;
    if (g >= q) {
      g -= q;
      ++r;
    }
  }
};

__global__ void __launch_bounds__(256) cvt_f16_kernel(const float* __restrict__ src, uint64_t rows,
                                                      uint64_t cols, uint16_t* __restrict__ dst,
                                                      uint64_t pitch, int mode, int vec) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  const uint64_t start = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (vec) {  // cols % 4 == 0 and both bases 16-byte aligned; pitch % 8 == 0 always
    const uint64_t q = cols >> 2;
    RowWalk w2(start + stride, stride * 2, q);
    // two groups per trip: both loads are in flight before the first store
    RowWalk a(start, stride * 2, q);
    for (; w2.r < rows; a.next(q), w2.next(q)) {
      const float4 v0 = __ldcs(reinterpret_cast<const float4*>(src + a.r * cols + (a.g << 2)));
      const float4 v1 = __ldcs(reinterpret_cast<const float4*>(src + w2.r * cols + (w2.g << 2)));
      uint2 o0, o1;
      o0.x = uint32_t(f32_to_f16(v0.x, mode)) | (uint32_t(f32_to_f16(v0.y, mode)) << 16);
      o0.y = uint32_t(f32_to_f16(v0.z, mode)) | (uint32_t(f32_to_f16(v0.w, mode)) << 16);
      o1.x = uint32_t(f32_to_f16(v1.x, mode)) | (uint32_t(f32_to_f16(v1.y, mode)) << 16);
      o1.y = uint32_t(f32_to_f16(v1.z, mode)) | (uint32_t(f32_to_f16(v1.w, mode)) << 16);
      *reinterpret_cast<uint2*>(dst + a.r * pitch + (a.g << 2)) = o0;
      *reinterpret_cast<uint2*>(dst + w2.r * pitch + (w2.g << 2)) = o1;
    }
    if (a.r < rows) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(src + a.r * cols + (a.g << 2)));
      uint2 o;
      o.x = uint32_t(f32_to_f16(v.x, mode)) | (uint32_t(f32_to_f16(v.y, mode)) << 16);
      o.y = uint32_t(f32_to_f16(v.z, mode)) | (uint32_t(f32_to_f16(v.w, mode)) << 16);
      *reinterpret_cast<uint2*>(dst + a.r * pitch + (a.g << 2)) = o;
    }
  } else {
    for (RowWalk w(start, stride, cols); w.r < rows; w.next(cols))
      dst[w.r * pitch + w.g] = f32_to_f16(src[w.r * cols + w.g], mode);
  }
}

__device__ __forceinline__ float rna_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// `mask` (optional, same shape as src): elements whose mask value is not > 0 are
// taken as zero - the ReLU derivative of
// internal/cgo/metal_bridge_activation.m:74-77 applied while the operand planes
// of the backward GEMMs are written, so the masked gradient never exists in HBM.
__global__ void __launch_bounds__(256) split_tf32_kernel(const float* __restrict__ src,
                                                         const float* __restrict__ mask,
                                                         uint64_t rows, uint64_t cols,
                                                         float* __restrict__ hi,
                                                         float* __restrict__ lo, uint64_t pitch,
                                                         int vec) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  const uint64_t start = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (vec) {
    const uint64_t q = cols >> 2;
    for (RowWalk w(start, stride, q); w.r < rows; w.next(q)) {
      const uint64_t r = w.r, c = w.g << 2;
      float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * cols + c));
      if (mask) {
        const float4 m = __ldcs(reinterpret_cast<const float4*>(mask + r * cols + c));
        v.x = m.x > 0.0f ? v.x : 0.0f;
        v.y = m.y > 0.0f ? v.y : 0.0f;
        v.z = m.z > 0.0f ? v.z : 0.0f;
        v.w = m.w > 0.0f ? v.w : 0.0f;
      }
      float4 h, l;
      h.x = rna_tf32(v.x); l.x = rna_tf32(v.x - h.x);
      h.y = rna_tf32(v.y); l.y = rna_tf32(v.y - h.y);
      h.z = rna_tf32(v.z); l.z = rna_tf32(v.z - h.z);
      h.w = rna_tf32(v.w); l.w = rna_tf32(v.w - h.w);
      *reinterpret_cast<float4*>(hi + r * pitch + c) = h;
      *reinterpret_cast<float4*>(lo + r * pitch + c) = l;
    }
  } else {
    for (RowWalk w(start, stride, cols); w.r < rows; w.next(cols)) {
      const uint64_t i = w.r * cols + w.g;
      float x = src[i];
      if (mask && !(mask[i] > 0.0f)) x = 0.0f;
      const float h = rna_tf32(x);
      hi[w.r * pitch + w.g] = h;
      lo[w.r * pitch + w.g] = rna_tf32(x - h);
    }
  }
}

// The same split for the kernel that takes its correction terms from bf16 planes: hi as
// above, then bf16(hi) and bf16(x - hi) in two planes of `plane` elements behind `x2`.
// The two cross products hi.lo + lo.hi only have to be good to 2^-8 of themselves (they are
// 2^-11 of the product), which is what bf16 keeps; it also keeps fp32's exponent range.
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));  // a in the low half
  return r;
}
__global__ void __launch_bounds__(256) split_tf32_bf16_kernel(const float* __restrict__ src,
                                                              const float* __restrict__ mask,
                                                              uint64_t rows, uint64_t cols,
                                                              float* __restrict__ hi,
                                                              uint16_t* __restrict__ x2,
                                                              uint64_t pitch, uint64_t plane,
                                                              int vec) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  const uint64_t start = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (vec) {
    const uint64_t q = cols >> 2;
    for (RowWalk w(start, stride, q); w.r < rows; w.next(q)) {
      const uint64_t r = w.r, c = w.g << 2;
      float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * cols + c));
      if (mask) {
        const float4 m = __ldcs(reinterpret_cast<const float4*>(mask + r * cols + c));
        v.x = m.x > 0.0f ? v.x : 0.0f;
        v.y = m.y > 0.0f ? v.y : 0.0f;
        v.z = m.z > 0.0f ? v.z : 0.0f;
        v.w = m.w > 0.0f ? v.w : 0.0f;
      }
      float4 h;
      h.x = rna_tf32(v.x);
      h.y = rna_tf32(v.y);
      h.z = rna_tf32(v.z);
      h.w = rna_tf32(v.w);
      *reinterpret_cast<float4*>(hi + r * pitch + c) = h;
      uint2 hb, lb;
      hb.x = pack_bf16(h.x, h.y);
      hb.y = pack_bf16(h.z, h.w);
      lb.x = pack_bf16(v.x - h.x, v.y - h.y);
      lb.y = pack_bf16(v.z - h.z, v.w - h.w);
      *reinterpret_cast<uint2*>(x2 + r * pitch + c) = hb;
      *reinterpret_cast<uint2*>(x2 + plane + r * pitch + c) = lb;
    }
  } else {
    for (RowWalk w(start, stride, cols); w.r < rows; w.next(cols)) {
      const uint64_t i = w.r * cols + w.g;
      float x = src[i];
      if (mask && !(mask[i] > 0.0f)) x = 0.0f;
      const float h = rna_tf32(x);
      hi[w.r * pitch + w.g] = h;
      x2[w.r * pitch + w.g] = uint16_t(pack_bf16(h, 0.0f) & 0xFFFFu);
      x2[plane + w.r * pitch + w.g] = uint16_t(pack_bf16(x - h, 0.0f) & 0xFFFFu);
    }
  }
}

// ------------------------------------------------------------------ elementwise
// Bias broadcast add, the four patterns of
// internal/cgo/metal_bridge_matrix.m:273-312.
__global__ void __launch_bounds__(256) add_broadcast_kernel(const float* __restrict__ a,
                                                            const float* __restrict__ b,
                                                            float* __restrict__ c, uint64_t rows,
                                                            uint64_t cols, int mode) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  const uint64_t total = rows * cols;
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total;
       i += uint64_t(gridDim.x) * blockDim.x) {
    const uint64_t r = i / cols, col = i - r * cols;
    float v;
    switch (mode) {
      case 0: v = a[i] + b[col]; break;
      case 1: v = a[col] + b[i]; break;
      case 2: v = a[i] + b[r]; break;
      default: v = a[r] + b[i]; break;
    }
    c[i] = v;
  }
}

// ReLU forward / backward: internal/cgo/metal_bridge_activation.m:44-47, 74-77.
__global__ void __launch_bounds__(256) relu_fwd_kernel(const float* __restrict__ in,
                                                       float* __restrict__ out, uint64_t n) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x)
    out[i] = fmaxf(0.0f, in[i]);
}
__global__ void __launch_bounds__(256) relu_bwd_kernel(const float* __restrict__ go,
                                                       const float* __restrict__ act,
                                                       float* __restrict__ gi, uint64_t n) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x)
    gi[i] = (act[i] > 0.0f) ? go[i] : 0.0f;
}

// float64 <-> float32 for the gonum facade (gpu/matrix/gonum-compat.go:14-42 does
// float32(m.At(i, j)) per element on the host; :322-334 widens back).  Round to
// nearest even, overflow to infinity, NaN kept: the conversion Go's float32(x) does.
__global__ void __launch_bounds__(256) f64_to_f32_kernel(const double* __restrict__ in,
                                                         float* __restrict__ out, uint64_t n, int vec) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (vec) {  // 2 x 16-byte loads, one 16-byte store per thread and step
    const uint64_t q = n >> 2;
    for (; i < q; i += stride) {
      const double2 a = __ldcs(reinterpret_cast<const double2*>(in) + 2 * i);
      const double2 b = __ldcs(reinterpret_cast<const double2*>(in) + 2 * i + 1);
      reinterpret_cast<float4*>(out)[i] = make_float4(__double2float_rn(a.x), __double2float_rn(a.y),
                                                      __double2float_rn(b.x), __double2float_rn(b.y));
    }
    const uint64_t t = (q << 2) + blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (t < n) out[t] = __double2float_rn(in[t]);
  } else {
    for (; i < n; i += stride) out[i] = __double2float_rn(in[i]);
  }
}
__global__ void __launch_bounds__(256) f32_to_f64_kernel(const float* __restrict__ in,
                                                         double* __restrict__ out, uint64_t n, int vec) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  const uint64_t stride = uint64_t(gridDim.x) * blockDim.x;
  uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (vec) {
    const uint64_t q = n >> 2;
    for (; i < q; i += stride) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(in) + i);
      reinterpret_cast<double2*>(out)[2 * i] = make_double2(double(v.x), double(v.y));
      reinterpret_cast<double2*>(out)[2 * i + 1] = make_double2(double(v.z), double(v.w));
    }
    const uint64_t t = (q << 2) + blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
    if (t < n) out[t] = double(in[t]);
  } else {
    for (; i < n; i += stride) out[i] = double(in[i]);
  }
}

// Column sum (bias gradient, gpu/matrix/layers.go:281-294).  Block (x, y) adds rows
// [y * chunk_rows, (y + 1) * chunk_rows) of 32 columns, eight row lanes each in row order,
// lanes in lane order.  With one chunk that is the result.  With several, the partial sums
// go to `partial` [chunk][col] and the block that arrives last on the column block's counter
// adds them in chunk order (no block waits for another; the counter is left at zero), so
// the result is the same from run to run whatever the arrival order.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ in,
                                                     const float* __restrict__ mask, uint64_t rows,
                                                     uint64_t cols, float* __restrict__ out,
                                                     uint64_t chunk_rows, float* partial,
                                                     uint32_t* counters) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  __shared__ float part[8][33];
  __shared__ uint32_t last;
  const uint32_t cx = threadIdx.x & 31u, ry = threadIdx.x >> 5;
  const uint64_t col = blockIdx.x * 32ull + cx;
  const uint64_t r0 = blockIdx.y * chunk_rows;
  const uint64_t r1 = (r0 + chunk_rows < rows) ? r0 + chunk_rows : rows;
  float s = 0.f;
  if (col < cols)
    for (uint64_t r = r0 + ry; r < r1; r += 8) {
      const float v = in[r * cols + col];
      s += (!mask || mask[r * cols + col] > 0.0f) ? v : 0.0f;
    }
  part[ry][cx] = s;
  __syncthreads();
  float t = 0.f;
  if (ry == 0) {
#pragma unroll
    for (int k = 0; k < 8; ++k) t += part[k][cx];
  }
  if (gridDim.y == 1) {
    if (ry == 0 && col < cols) out[col] = t;
    return;
  }
  if (ry == 0 && col < cols) __stcg(partial + uint64_t(blockIdx.y) * cols + col, t);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t before = atomicAdd(counters + blockIdx.x, 1u);
    last = (before + 1u == gridDim.y) ? 1u : 0u;
    if (last) counters[blockIdx.x] = 0u;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (ry == 0 && col < cols) {
    float total = 0.f;
    for (uint32_t c = 0; c < gridDim.y; ++c) total += __ldcg(partial + uint64_t(c) * cols + col);
    out[col] = total;
  }
}

// The split of a layer's output gradient and its column sums (the bias gradient) in one pass:
// the linear backward needs both of the same masked values.  Blocks as in colsum_kernel, each
// thread four neighbouring columns: block (x, y) walks rows [y * chunk_rows, (y + 1) * chunk_rows)
// of 128 columns, writes their operand planes (tf32 hi/lo, or hi and the two bf16 planes) and
// adds them up; partial sums and the block that arrives last as in colsum_kernel.
// cols % 4 == 0 and 16-byte aligned bases (the launcher checks).
template <bool BF16X>
__global__ void __launch_bounds__(256) split_colsum_kernel(const float* __restrict__ src,
                                                           const float* __restrict__ mask,
                                                           uint64_t rows, uint64_t cols,
                                                           float* __restrict__ hi, void* low,
                                                           uint64_t pitch, uint64_t plane,
                                                           float* __restrict__ out,
                                                           uint64_t chunk_rows, float* partial,
                                                           uint32_t* counters) {
  ptx::grid_dependency_release();  // programmatic dependent launch: see launch.cuh
  ptx::grid_dependency_wait();
  __shared__ float4 part[8][33];
  __shared__ uint32_t last;
  const uint32_t cx = threadIdx.x & 31u, ry = threadIdx.x >> 5;
  const uint64_t c = (blockIdx.x * 32ull + cx) << 2;
  const uint64_t r0 = blockIdx.y * chunk_rows;
  const uint64_t r1 = (r0 + chunk_rows < rows) ? r0 + chunk_rows : rows;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < cols)
    for (uint64_t r = r0 + ry; r < r1; r += 8) {
      float4 v = __ldcs(reinterpret_cast<const float4*>(src + r * cols + c));
      if (mask) {
        const float4 m = __ldcs(reinterpret_cast<const float4*>(mask + r * cols + c));
        v.x = m.x > 0.0f ? v.x : 0.0f;
        v.y = m.y > 0.0f ? v.y : 0.0f;
        v.z = m.z > 0.0f ? v.z : 0.0f;
        v.w = m.w > 0.0f ? v.w : 0.0f;
      }
      s.x += v.x;
      s.y += v.y;
      s.z += v.z;
      s.w += v.w;
      float4 h;
      h.x = rna_tf32(v.x);
      h.y = rna_tf32(v.y);
      h.z = rna_tf32(v.z);
      h.w = rna_tf32(v.w);
      *reinterpret_cast<float4*>(hi + r * pitch + c) = h;
      if (BF16X) {
        uint16_t* x2 = static_cast<uint16_t*>(low);
        uint2 hb, lb;
        hb.x = pack_bf16(h.x, h.y);
        hb.y = pack_bf16(h.z, h.w);
        lb.x = pack_bf16(v.x - h.x, v.y - h.y);
        lb.y = pack_bf16(v.z - h.z, v.w - h.w);
        *reinterpret_cast<uint2*>(x2 + r * pitch + c) = hb;
        *reinterpret_cast<uint2*>(x2 + plane + r * pitch + c) = lb;
      } else {
        float4 l;
        l.x = rna_tf32(v.x - h.x);
        l.y = rna_tf32(v.y - h.y);
        l.z = rna_tf32(v.z - h.z);
        l.w = rna_tf32(v.w - h.w);
        *reinterpret_cast<float4*>(static_cast<float*>(low) + r * pitch + c) = l;
      }
    }
  part[ry][cx] = s;
  __syncthreads();
  float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
  if (ry == 0) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      t.x += part[k][cx].x;
      t.y += part[k][cx].y;
      t.z += part[k][cx].z;
      t.w += part[k][cx].w;
    }
  }
  if (gridDim.y == 1) {
    if (ry == 0 && c < cols) *reinterpret_cast<float4*>(out + c) = t;
    return;
  }
  if (ry == 0 && c < cols) __stcg(reinterpret_cast<float4*>(partial + uint64_t(blockIdx.y) * cols + c), t);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t before = atomicAdd(counters + blockIdx.x, 1u);
    last = (before + 1u == gridDim.y) ? 1u : 0u;
    if (last) counters[blockIdx.x] = 0u;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (ry == 0 && c < cols) {
    float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k = 0; k < gridDim.y; ++k) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + uint64_t(k) * cols + c));
      total.x += v.x;
      total.y += v.y;
      total.z += v.z;
      total.w += v.w;
    }
    *reinterpret_cast<float4*>(out + c) = total;
  }
}

inline uint32_t stream_grid(uint64_t work_items, uint32_t threads, uint32_t cap) {
  uint64_t g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  return uint32_t(g < cap ? g : cap);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

void launch_transpose(const float* in, uint64_t rows, uint64_t cols, float* out, int /*sm_count*/,
                      cudaStream_t stream) {
  if (rows == 0 || cols == 0) return;
  const uint32_t tiles_r = uint32_t((rows + TT - 1) / TT), tiles_c = uint32_t((cols + TT - 1) / TT);
  const uint32_t grid = tiles_r * tiles_c;
  const bool vin = (cols % 4 == 0) && aligned16(in);
  const bool vout = (rows % 4 == 0) && aligned16(out);
  if (vin && vout)
    launch_kernel(transpose_kernel<true, true>, dim3(grid), dim3(256), 0, stream, in, out, uint32_t(rows), uint32_t(cols), tiles_r,
                  tiles_c);
  else if (vin)
    launch_kernel(transpose_kernel<true, false>, dim3(grid), dim3(256), 0, stream, in, out, uint32_t(rows), uint32_t(cols), tiles_r,
                  tiles_c);
  else if (vout)
    launch_kernel(transpose_kernel<false, true>, dim3(grid), dim3(256), 0, stream, in, out, uint32_t(rows), uint32_t(cols), tiles_r,
                  tiles_c);
  else
    launch_kernel(transpose_kernel<false, false>, dim3(grid), dim3(256), 0, stream, in, out, uint32_t(rows), uint32_t(cols), tiles_r,
                  tiles_c);
}

void launch_cvt_f16(const float* src, uint64_t rows, uint64_t cols, void* dst, uint64_t pitch,
                    int mode, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return;
  const int vec = (cols % 4 == 0) && aligned16(src) && aligned16(dst) && (pitch % 4 == 0);
  const uint64_t items = vec ? rows * (cols / 4) : rows * cols;
  launch_kernel(cvt_f16_kernel, dim3(stream_grid(items, 256, 148 * 16)), dim3(256), 0, stream, 
      src, rows, cols, static_cast<uint16_t*>(dst), pitch, mode, vec);
}

void launch_split_tf32(const float* src, uint64_t rows, uint64_t cols, float* hi, float* lo,
                       uint64_t pitch, cudaStream_t stream, const float* mask) {
  if (rows == 0 || cols == 0) return;
  const int vec = (cols % 4 == 0) && aligned16(src) && aligned16(hi) && aligned16(lo) &&
                  (pitch % 4 == 0) && (!mask || aligned16(mask));
  const uint64_t items = vec ? rows * (cols / 4) : rows * cols;
  launch_kernel(split_tf32_kernel, dim3(stream_grid(items, 256, 148 * 16)), dim3(256), 0, stream, src, mask, rows, cols, hi,
                                                                           lo, pitch, vec);
}

void launch_split_tf32_bf16(const float* src, uint64_t rows, uint64_t cols, float* hi, void* x2,
                            uint64_t pitch, cudaStream_t stream, const float* mask) {
  if (rows == 0 || cols == 0) return;
  const int vec = (cols % 4 == 0) && aligned16(src) && aligned16(hi) && aligned16(x2) &&
                  (pitch % 8 == 0) && (!mask || aligned16(mask));
  const uint64_t items = vec ? rows * (cols / 4) : rows * cols;
  launch_kernel(split_tf32_bf16_kernel, dim3(stream_grid(items, 256, 148 * 16)), dim3(256), 0, stream,
                src, mask, rows, cols, hi, static_cast<uint16_t*>(x2), pitch, rows * pitch, vec);
}

bool launch_split_colsum(const float* src, uint64_t rows, uint64_t cols, float* hi, void* low, bool bf16x,
                         uint64_t pitch, float* colsum, cudaStream_t stream, const float* mask, float* ws,
                         size_t ws_floats, uint32_t* counters, uint32_t counter_slots) {
  if (rows == 0 || cols == 0) return false;
  if (cols % 4 || pitch % 8 || !aligned16(src) || !aligned16(hi) || !aligned16(low) || !aligned16(colsum) ||
      (mask && !aligned16(mask)))
    return false;
  const uint32_t col_blocks = uint32_t((cols + 127) / 128);
  // row chunks of at least 32 rows, enough of them to put about four blocks on every SM
  uint64_t chunks = 1;
  if (ws && counters && aligned16(ws) && col_blocks <= counter_slots && rows >= 64) {
    chunks = std::min<uint64_t>(rows / 32, std::max<uint64_t>(1, 592 / col_blocks));
    while (chunks > 1 && chunks * cols > ws_floats) --chunks;
  }
  uint64_t chunk_rows = (rows + chunks - 1) / chunks;
  chunk_rows = (chunk_rows + 7) / 8 * 8;
  chunks = (rows + chunk_rows - 1) / chunk_rows;
  if (chunks < 1) chunks = 1;
  if (chunks > 65535) return false;
  const dim3 grid(col_blocks, uint32_t(chunks));
  if (bf16x)
    launch_kernel(split_colsum_kernel<true>, grid, dim3(256), 0, stream, src, mask, rows, cols, hi, low, pitch,
                  rows * pitch, colsum, chunk_rows, ws, counters);
  else
    launch_kernel(split_colsum_kernel<false>, grid, dim3(256), 0, stream, src, mask, rows, cols, hi, low, pitch,
                  rows * pitch, colsum, chunk_rows, ws, counters);
  return true;
}

void launch_add_broadcast(const float* a, const float* b, float* c, uint64_t rows, uint64_t cols,
                          int mode, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return;
  launch_kernel(add_broadcast_kernel, dim3(stream_grid(rows * cols, 256, 148 * 16)), dim3(256), 0, stream, a, b, c, rows,
                                                                                    cols, mode);
}

void launch_relu_forward(const float* in, float* out, uint64_t n, cudaStream_t stream) {
  if (n == 0) return;
  launch_kernel(relu_fwd_kernel, dim3(stream_grid(n, 256, 148 * 16)), dim3(256), 0, stream, in, out, n);
}

void launch_relu_backward(const float* grad_out, const float* act_out, float* grad_in, uint64_t n,
                          cudaStream_t stream) {
  if (n == 0) return;
  launch_kernel(relu_bwd_kernel, dim3(stream_grid(n, 256, 148 * 16)), dim3(256), 0, stream, grad_out, act_out, grad_in, n);
}

void launch_f64_to_f32(const double* in, float* out, uint64_t n, cudaStream_t stream) {
  if (n == 0) return;
  const int vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0 && n >= 4;
  launch_kernel(f64_to_f32_kernel, dim3(stream_grid(vec ? n >> 2 : n, 256, 148 * 16)), dim3(256), 0, stream, in, out, n, vec);
}

void launch_f32_to_f64(const float* in, double* out, uint64_t n, cudaStream_t stream) {
  if (n == 0) return;
  const int vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0 && n >= 4;
  launch_kernel(f32_to_f64_kernel, dim3(stream_grid(vec ? n >> 2 : n, 256, 148 * 16)), dim3(256), 0, stream, in, out, n, vec);
}

void launch_colsum(const float* in, uint64_t rows, uint64_t cols, float* out, cudaStream_t stream,
                   const float* mask, float* ws, size_t ws_floats, uint32_t* counters,
                   uint32_t counter_slots) {
  if (cols == 0) return;
  const uint32_t col_blocks = uint32_t((cols + 31) / 32);
  // row chunks of at least 64 rows, enough of them to put about two blocks on every SM
  uint64_t chunks = 1;
  if (ws && counters && col_blocks <= counter_slots && rows >= 128) {
    chunks = std::min<uint64_t>(rows / 64, std::max<uint64_t>(1, 296 / col_blocks));
    while (chunks > 1 && chunks * cols > ws_floats) --chunks;
  }
  uint64_t chunk_rows = (rows + chunks - 1) / chunks;
  chunk_rows = (chunk_rows + 7) / 8 * 8;
  chunks = rows ? (rows + chunk_rows - 1) / chunk_rows : 1;
  if (chunks < 1) chunks = 1;
  launch_kernel(colsum_kernel, dim3(col_blocks, uint32_t(chunks)), dim3(256), 0, stream, in, mask, rows, cols, out,
                chunk_rows, ws, counters);
}

}  // namespace gonn
