/* CPU restatement of the reference's dense path - TEST INFRASTRUCTURE ONLY.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
 * load this file; the product library never links or calls it.
 *
 * Each function follows the reference code cited above it (paths are inside
 * tsawler/go-nngpu).  The reference's own GEMM runs inside Apple's closed
 * MPSMatrixMultiplication and none of its tests asserts a MatMul or Transpose
 * result, so for GEMM and Transpose this oracle is "parity unpinned": it
 * restates the mathematical definition (float64 accumulation of the float32
 * inputs) and the index formula, and is cross-checked against numpy.  The ReLU
 * functions ARE pinned by the known-answer vectors of
 * gpu/matrix/activation_test.go:32-74 (see tests/golden/).
 *
 * Build: make -C oracle   (gcc -O2 -shared -fPIC)
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* C[M,N] = A[M,K].B[K,N] accumulated in float64 from float32 inputs: the
 * "float64 reference" the tolerances are stated against.  Operands are given
 * as stored; transA means A is stored [K,M], transB means B is stored [N,K]
 * (the reference reaches those by Transpose + MatMul,
 * gpu/matrix/layers.go:77-96). */
void oracle_gemm_f64(const float *A, const float *B, double *C, long M, long N, long K, int transA,
                     int transB) {
  for (long i = 0; i < M; i++) {
    for (long j = 0; j < N; j++) C[i * N + j] = 0.0;
    for (long k = 0; k < K; k++) {
      const double a = transA ? (double)A[k * M + i] : (double)A[i * K + k];
      if (transB) {
        for (long j = 0; j < N; j++) C[i * N + j] += a * (double)B[j * K + k];
      } else {
        for (long j = 0; j < N; j++) C[i * N + j] += a * (double)B[k * N + j];
      }
    }
  }
}

/* internal/cgo/metal_bridge_matrix.m:159-166 (the transpose loop) with the
 * dimension check of :145-148.  Returns -2 on mismatched dimensions. */
int oracle_transpose(const float *in, long inRows, long inCols, float *out, long outRows,
                     long outCols) {
  if (inRows != outCols || inCols != outRows) return -2;
  for (long i = 0; i < inRows; i++)
    for (long j = 0; j < inCols; j++) out[j * outCols + i] = in[i * inCols + j];
  return 0;
}

/* internal/cgo/default.metal:459-509, kernel fused_linear_activation: one
 * float32 dot product per output in index order, + bias[o], then the
 * activation switch (0 ReLU, 1 LeakyReLU, 2 Sigmoid, 3 Tanh, 4 tanh-GELU,
 * otherwise identity). */
void oracle_fused_linear_activation(const float *input, const float *weight, const float *bias,
                                    float *output, long batch_size, long input_size,
                                    long output_size, int activation_type, float activation_param) {
  for (long b = 0; b < batch_size; b++) {
    for (long o = 0; o < output_size; o++) {
      float sum = 0.0f;
      for (long i = 0; i < input_size; i++)
        sum += input[b * input_size + i] * weight[i * output_size + o];
      if (bias) sum += bias[o];
      float act;
      switch (activation_type) {
        case 0: act = fmaxf(sum, 0.0f); break;
        case 1: act = sum > 0 ? sum : sum * activation_param; break;
        case 2: act = 1.0f / (1.0f + expf(-sum)); break;
        case 3: act = tanhf(sum); break;
        case 4:
          act = 0.5f * sum * (1.0f + tanhf(0.7978845608f * (sum + 0.044715f * sum * sum * sum)));
          break;
        default: act = sum;
      }
      output[b * output_size + o] = act;
    }
  }
}

/* Same operation with the dot product in float64 (bias and activation too):
 * the error reference for the tolerance check of the fused path. */
void oracle_fused_linear_activation_f64(const float *input, const float *weight, const float *bias,
                                        double *output, long batch_size, long input_size,
                                        long output_size, int activation_type,
                                        float activation_param) {
  for (long b = 0; b < batch_size; b++) {
    for (long o = 0; o < output_size; o++) {
      double sum = 0.0;
      for (long i = 0; i < input_size; i++)
        sum += (double)input[b * input_size + i] * (double)weight[i * output_size + o];
      if (bias) sum += (double)bias[o];
      double act;
      switch (activation_type) {
        case 0: act = sum > 0.0 ? sum : 0.0; break;
        case 1: act = sum > 0 ? sum : sum * (double)activation_param; break;
        case 2: act = 1.0 / (1.0 + exp(-sum)); break;
        case 3: act = tanh(sum); break;
        case 4:
          act = 0.5 * sum * (1.0 + tanh(0.7978845608 * (sum + 0.044715 * sum * sum * sum)));
          break;
        default: act = sum;
      }
      output[b * output_size + o] = act;
    }
  }
}

/* internal/cgo/metal_bridge_kernels.m:28-82, kernel optimized_gemm:
 * C = alpha * (A.B) + beta * C with a float32 running sum in k order. */
void oracle_gemm_alpha_beta(const float *A, const float *B, float *C, long M, long N, long K,
                            float alpha, float beta) {
  for (long i = 0; i < M; i++)
    for (long j = 0; j < N; j++) {
      float sum = 0.0f;
      for (long k = 0; k < K; k++) sum += A[i * K + k] * B[k * N + j];
      C[i * N + j] = alpha * sum + beta * C[i * N + j];
    }
}

/* internal/cgo/metal_bridge_matrix.m:273-317: the four broadcast patterns;
 * -2 for any other shape combination. */
int oracle_add_broadcast(const float *a, long aRows, long aCols, const float *b, long bRows,
                         long bCols, float *r, long rRows, long rCols) {
  if (aRows == rRows && aCols == rCols && bRows == 1 && bCols == rCols) {
    for (long i = 0; i < rRows; i++)
      for (long j = 0; j < rCols; j++) r[i * rCols + j] = a[i * aCols + j] + b[j];
  } else if (bRows == rRows && bCols == rCols && aRows == 1 && aCols == rCols) {
    for (long i = 0; i < rRows; i++)
      for (long j = 0; j < rCols; j++) r[i * rCols + j] = a[j] + b[i * bCols + j];
  } else if (aRows == rRows && aCols == rCols && bRows == rRows && bCols == 1) {
    for (long i = 0; i < rRows; i++)
      for (long j = 0; j < rCols; j++) r[i * rCols + j] = a[i * aCols + j] + b[i];
  } else if (bRows == rRows && bCols == rCols && aRows == rRows && aCols == 1) {
    for (long i = 0; i < rRows; i++)
      for (long j = 0; j < rCols; j++) r[i * rCols + j] = a[i] + b[i * bCols + j];
  } else {
    return -2;
  }
  return 0;
}

/* internal/cgo/metal_bridge_activation.m:44-47 */
void oracle_relu_forward(const float *in, float *out, long size) {
  for (long i = 0; i < size; i++) out[i] = fmaxf(0.0f, in[i]);
}

/* internal/cgo/metal_bridge_activation.m:74-77 */
void oracle_relu_backward(const float *grad_out, const float *act_out, float *grad_in, long size) {
  for (long i = 0; i < size; i++) grad_in[i] = (act_out[i] > 0.0f) ? grad_out[i] : 0.0f;
}

/* gpu/matrix/layers.go:281-294, sumAlongAxis(axis 0): column sums in row order. */
void oracle_column_sum(const float *in, long rows, long cols, float *out) {
  for (long j = 0; j < cols; j++) out[j] = 0.0f;
  for (long i = 0; i < rows; i++)
    for (long j = 0; j < cols; j++) out[j] += in[i * cols + j];
}

/* gpu/matrix/mixed-precision.go:106-151, Float32ToFloatMP16: truncating
 * float32 -> float16 bit conversion. */
uint16_t oracle_f32_to_f16_trunc(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  uint32_t sign = (bits >> 31) & 0x1;
  uint32_t exp = (bits >> 23) & 0xFF;
  uint32_t mantissa = bits & 0x7FFFFF;
  if (exp == 0) return (uint16_t)(sign << 15);
  if (exp == 0xFF) {
    if (mantissa == 0) return (uint16_t)((sign << 15) | 0x7C00);
    return (uint16_t)((sign << 15) | 0x7C00 | (mantissa >> 13));
  }
  int32_t expAdjusted = (int32_t)exp - 127 + 15;
  if (expAdjusted >= 31) return (uint16_t)((sign << 15) | 0x7C00);
  if (expAdjusted <= 0) {
    if (expAdjusted < -10) return (uint16_t)(sign << 15);
    int32_t shiftAmount = 1 - expAdjusted;
    if (shiftAmount > 0) mantissa = (mantissa | 0x800000) >> (uint32_t)shiftAmount;
    return (uint16_t)((sign << 15) | (mantissa >> 13));
  }
  return (uint16_t)((sign << 15) | ((uint32_t)expAdjusted << 10) | (mantissa >> 13));
}

/* gpu/matrix/mixed-precision.go:154-189, FloatMP16ToFloat32.  The reference
 * does its subnormal exponent arithmetic in uint32 with wrap-around; the
 * expression below is the same arithmetic. */
float oracle_f16_to_f32(uint16_t h) {
  uint32_t bits = h;
  uint32_t sign = (bits >> 15) & 0x1;
  uint32_t exp = (bits >> 10) & 0x1F;
  uint32_t mantissa = bits & 0x3FF;
  uint32_t result;
  if (exp == 0) {
    if (mantissa == 0) {
      result = sign << 31;
    } else {
      while ((mantissa & 0x400) == 0) {
        mantissa <<= 1;
        exp--;
      }
      mantissa &= 0x3FF;
      exp = exp - 15 + 127 + 1;
      result = (sign << 31) | (exp << 23) | (mantissa << 13);
    }
  } else if (exp == 31) {
    result = (sign << 31) | 0x7F800000u | (mantissa << 13);
  } else {
    exp = exp - 15 + 127;
    result = (sign << 31) | (exp << 23) | (mantissa << 13);
  }
  float f;
  memcpy(&f, &result, 4);
  return f;
}

/* gpu/matrix/mixed-precision.go:192-210, ConvertTensorToFloat16: float16
 * precision held in float32 storage. */
void oracle_convert_tensor_f16(const float *src, float *dst, long n) {
  for (long i = 0; i < n; i++) dst[i] = oracle_f16_to_f32(oracle_f32_to_f16_trunc(src[i]));
}

/* ---- element-wise family --------------------------------------------------------
 * internal/cgo/metal_bridge_matrix.m:172-249 (add), :322-392 (subtract),
 * :394-439 (multiply), :441-484 (divide), :486-543 (scalar add / multiply).
 * op: 0 add, 1 subtract, 2 multiply, 3 divide.  The divide stops at the first
 * zero divisor: earlier elements are written, the rest are not, and it returns
 * -4 with that index in *zero_index (metal_bridge_matrix.m:470-479). */
int oracle_elementwise(int op, const float *a, const float *b, float *r, long n, long *zero_index) {
  for (long i = 0; i < n; i++) {
    switch (op) {
      case 0: r[i] = a[i] + b[i]; break;
      case 1: r[i] = a[i] - b[i]; break;
      case 2: r[i] = a[i] * b[i]; break;
      default:
        if (b[i] == 0.0f) {
          if (zero_index) *zero_index = i;
          return -4;
        }
        r[i] = a[i] / b[i];
    }
  }
  return 0;
}

void oracle_scalar_op(int multiply, const float *in, float scalar, float *out, long n) {
  for (long i = 0; i < n; i++) out[i] = multiply ? in[i] * scalar : in[i] + scalar;
}

/* internal/cgo/metal_bridge_activation.m:83-170 (sigmoid, tanh: input clamped
 * to [-88, 88]; derivatives from the activation output), :372-430 (leaky ReLU).
 * kind: 0 sigmoid, 1 tanh, 2 leaky ReLU. */
void oracle_activation_forward(int kind, const float *in, float *out, long n, float alpha) {
  for (long i = 0; i < n; i++) {
    if (kind == 0) {
      float x = fmaxf(-88.0f, fminf(88.0f, in[i]));
      out[i] = 1.0f / (1.0f + expf(-x));
    } else if (kind == 1) {
      float x = fmaxf(-88.0f, fminf(88.0f, in[i]));
      out[i] = tanhf(x);
    } else {
      float x = in[i];
      out[i] = (x > 0.0f) ? x : alpha * x;
    }
  }
}

void oracle_activation_backward(int kind, const float *grad_out, const float *act_out, float *grad_in,
                                long n, float alpha) {
  for (long i = 0; i < n; i++) {
    if (kind == 0) {
      float s = act_out[i];
      grad_in[i] = grad_out[i] * s * (1.0f - s);
    } else if (kind == 1) {
      float t = act_out[i];
      grad_in[i] = grad_out[i] * (1.0f - t * t);
    } else {
      float d = (act_out[i] > 0.0f) ? 1.0f : alpha;
      grad_in[i] = grad_out[i] * d;
    }
  }
}

/* internal/cgo/metal_bridge_activation.m:435-703: ELU, Swish, tanh-GELU.
 * kind: 3 ELU, 4 Swish, 5 GELU.  The backward forms take the activation
 * output; Swish and GELU recover the input with three Newton steps. */
static float clamp88(float x) { return fmaxf(-88.0f, fminf(88.0f, x)); }

void oracle_activation2_forward(int kind, const float *in, float *out, long n, float alpha) {
  const float k = 0.7978845608028654f, c3 = 0.044715f;
  for (long i = 0; i < n; i++) {
    float x = in[i];
    if (kind == 3) {
      out[i] = (x > 0.0f) ? x : alpha * (expf(fmaxf(-88.0f, x)) - 1.0f);
    } else if (kind == 4) {
      x = clamp88(x);
      out[i] = x * (1.0f / (1.0f + expf(-x)));
    } else {
      float inner = clamp88(k * (x + c3 * (x * x * x)));
      out[i] = 0.5f * x * (1.0f + tanhf(inner));
    }
  }
}

void oracle_activation2_backward(int kind, const float *grad_out, const float *act_out, float *grad_in,
                                 long n, float alpha) {
  const float k = 0.7978845608028654f, c3 = 0.044715f;
  for (long i = 0; i < n; i++) {
    const float y = act_out[i];
    float derivative;
    if (kind == 3) {
      derivative = (y > 0.0f) ? 1.0f : y + alpha;
    } else if (kind == 4) {
      if (fabsf(y) < 1e-8f) {
        grad_in[i] = grad_out[i] * 0.5f;
        continue;
      }
      float x = y;
      for (int it = 0; it < 3; it++) {
        float sg = 1.0f / (1.0f + expf(-x));
        float f = x * sg - y;
        float df = sg + x * sg * (1.0f - sg);
        if (fabsf(df) > 1e-8f) x = x - f / df;
      }
      float sg = 1.0f / (1.0f + expf(-x));
      derivative = sg + x * sg * (1.0f - sg);
    } else {
      float x = y;
      for (int it = 0; it < 3; it++) {
        float th = tanhf(clamp88(k * (x + c3 * (x * x * x))));
        float f = 0.5f * x * (1.0f + th) - y;
        float df = 0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * (k * (1.0f + 3.0f * c3 * x * x));
        if (fabsf(df) > 1e-8f) x = x - f / df;
      }
      float th = tanhf(clamp88(k * (x + c3 * (x * x * x))));
      derivative = 0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * (k * (1.0f + 3.0f * c3 * x * x));
    }
    grad_in[i] = grad_out[i] * derivative;
  }
}

/* internal/cgo/metal_bridge_activation.m:283-369 (the 1-D forms, :206-281, are
 * the batch == 1 case): per row, max, exp and running sum, divide; backward
 * grad_in = y * (grad_out - dot(grad_out, y)). */
void oracle_softmax_forward(const float *in, float *out, long batch, long features) {
  for (long b = 0; b < batch; b++) {
    const float *x = in + b * features;
    float *y = out + b * features;
    float m = x[0];
    for (long i = 1; i < features; i++) m = fmaxf(m, x[i]);
    float sum = 0.0f;
    for (long i = 0; i < features; i++) {
      y[i] = expf(x[i] - m);
      sum += y[i];
    }
    for (long i = 0; i < features; i++) y[i] /= sum;
  }
}

void oracle_softmax_backward(const float *grad_out, const float *act, float *grad_in, long batch,
                             long features) {
  for (long b = 0; b < batch; b++) {
    const float *g = grad_out + b * features;
    const float *y = act + b * features;
    float dot = 0.0f;
    for (long i = 0; i < features; i++) dot += g[i] * y[i];
    for (long i = 0; i < features; i++) grad_in[b * features + i] = y[i] * (g[i] - dot);
  }
}
