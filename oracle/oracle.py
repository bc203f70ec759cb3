"""Python face of the CPU oracle - TEST INFRASTRUCTURE ONLY.

Loads oracle/liboracle.so (the C restatement in oracle.c, which cites the
reference lines it follows) and adds the numpy pieces: the seeded input
generators of the five benchmark configurations, the float64 GEMM reference
(numpy/OpenBLAS, cross-checked against the C triple loop), fp16 rounding, and
the relative Frobenius error.  Only tests/, __graft_entry__.smoke() and the
CPU-baseline legs of bench.py may import this module.

Parity status: GEMM and Transpose are "parity unpinned" (the reference has no
test that asserts their output and its GEMM lives in a closed Apple library);
ReLU forward/backward are pinned by the reference's own known-answer vectors.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_l, _i, _f = ctypes.c_long, ctypes.c_int, ctypes.c_float


def build():
    """Compiles oracle.c when the shared object is missing or stale."""
    src = os.path.join(HERE, "oracle.c")
    if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        h = ctypes.CDLL(LIB_PATH)
        h.oracle_gemm_f64.argtypes = [_f32p, _f32p, _f64p, _l, _l, _l, _i, _i]
        h.oracle_gemm_f64.restype = None
        h.oracle_transpose.argtypes = [_f32p, _l, _l, _f32p, _l, _l]
        h.oracle_transpose.restype = _i
        h.oracle_fused_linear_activation.argtypes = [_f32p, _f32p, _f32p, _f32p, _l, _l, _l, _i, _f]
        h.oracle_fused_linear_activation.restype = None
        h.oracle_fused_linear_activation_f64.argtypes = [_f32p, _f32p, _f32p, _f64p, _l, _l, _l, _i, _f]
        h.oracle_fused_linear_activation_f64.restype = None
        h.oracle_gemm_alpha_beta.argtypes = [_f32p, _f32p, _f32p, _l, _l, _l, _f, _f]
        h.oracle_gemm_alpha_beta.restype = None
        h.oracle_add_broadcast.argtypes = [_f32p, _l, _l, _f32p, _l, _l, _f32p, _l, _l]
        h.oracle_add_broadcast.restype = _i
        h.oracle_relu_forward.argtypes = [_f32p, _f32p, _l]
        h.oracle_relu_forward.restype = None
        h.oracle_relu_backward.argtypes = [_f32p, _f32p, _f32p, _l]
        h.oracle_relu_backward.restype = None
        h.oracle_column_sum.argtypes = [_f32p, _l, _l, _f32p]
        h.oracle_column_sum.restype = None
        h.oracle_f32_to_f16_trunc.argtypes = [_f]
        h.oracle_f32_to_f16_trunc.restype = ctypes.c_uint16
        h.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        h.oracle_f16_to_f32.restype = _f
        h.oracle_convert_tensor_f16.argtypes = [_f32p, _f32p, _l]
        h.oracle_convert_tensor_f16.restype = None
        _lib = h
    return _lib


def _p32(a):
    return a.ctypes.data_as(_f32p)


def _c32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------- C restatement
def gemm_f64_naive(A, B, trans_a=False, trans_b=False):
    """float64 triple loop over the operands as stored (small sizes only)."""
    A, B = _c32(A), _c32(B)
    M, K = (A.shape[1], A.shape[0]) if trans_a else A.shape
    N = B.shape[0] if trans_b else B.shape[1]
    C = np.empty((M, N), dtype=np.float64)
    lib().oracle_gemm_f64(_p32(A), _p32(B), C.ctypes.data_as(_f64p), M, N, K, int(trans_a), int(trans_b))
    return C


def transpose(X):
    X = _c32(X)
    out = np.empty((X.shape[1], X.shape[0]), dtype=np.float32)
    rc = lib().oracle_transpose(_p32(X), X.shape[0], X.shape[1], _p32(out), X.shape[1], X.shape[0])
    assert rc == 0
    return out


def fused_linear_activation(X, W, bias, act, alpha=0.0):
    X, W = _c32(X), _c32(W)
    b = _c32(bias) if bias is not None else None
    out = np.empty((X.shape[0], W.shape[1]), dtype=np.float32)
    lib().oracle_fused_linear_activation(_p32(X), _p32(W), _p32(b) if b is not None else None,
                                         _p32(out), X.shape[0], X.shape[1], W.shape[1], act, alpha)
    return out


def fused_linear_activation_f64(X, W, bias, act, alpha=0.0):
    X, W = _c32(X), _c32(W)
    b = _c32(bias) if bias is not None else None
    out = np.empty((X.shape[0], W.shape[1]), dtype=np.float64)
    lib().oracle_fused_linear_activation_f64(_p32(X), _p32(W), _p32(b) if b is not None else None,
                                             out.ctypes.data_as(_f64p), X.shape[0], X.shape[1],
                                             W.shape[1], act, alpha)
    return out


def gemm_alpha_beta(A, B, C, alpha, beta):
    A, B = _c32(A), _c32(B)
    out = _c32(C).copy()
    lib().oracle_gemm_alpha_beta(_p32(A), _p32(B), _p32(out), A.shape[0], B.shape[1], A.shape[1], alpha, beta)
    return out


def add_broadcast(a, b, out_shape):
    a, b = _c32(a), _c32(b)
    out = np.empty(out_shape, dtype=np.float32)
    rc = lib().oracle_add_broadcast(_p32(a), a.shape[0], a.shape[1], _p32(b), b.shape[0], b.shape[1],
                                    _p32(out), out_shape[0], out_shape[1])
    return rc, out


def relu_forward(x):
    x = _c32(x)
    out = np.empty_like(x)
    lib().oracle_relu_forward(_p32(x), _p32(out), x.size)
    return out


def relu_backward(grad_out, act_out):
    g, a = _c32(grad_out), _c32(act_out)
    out = np.empty_like(g)
    lib().oracle_relu_backward(_p32(g), _p32(a), _p32(out), g.size)
    return out


def column_sum(x):
    x = _c32(x)
    out = np.empty(x.shape[1], dtype=np.float32)
    lib().oracle_column_sum(_p32(x), x.shape[0], x.shape[1], _p32(out))
    return out


def f16_trunc(x):
    """The reference's truncating fp32->fp16->fp32 round trip (fp16 values in fp32 storage)."""
    x = _c32(x)
    out = np.empty_like(x)
    lib().oracle_convert_tensor_f16(_p32(x), _p32(out), x.size)
    return out


def f16_trunc_numpy(x):
    """Vectorised restatement of the same bit recipe, for full-size inputs."""
    x = _c32(x)
    bits = x.view(np.uint32)
    sign = (bits >> 31).astype(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64)
    mant = (bits & 0x7FFFFF).astype(np.uint32)
    e = exp - 127 + 15
    h = np.zeros(x.shape, dtype=np.uint32)
    normal = (exp != 0) & (exp != 0xFF) & (e > 0) & (e < 31)
    h[normal] = (e[normal].astype(np.uint32) << 10) | (mant[normal] >> 13)
    over = (exp != 0) & (exp != 0xFF) & (e >= 31)
    h[over] = 0x7C00
    sub = (exp != 0) & (exp != 0xFF) & (e <= 0) & (e >= -10)
    shift = (1 - e[sub]).astype(np.uint32)
    h[sub] = ((mant[sub] | 0x800000) >> shift) >> 13
    special = exp == 0xFF
    h[special] = 0x7C00 | (mant[special] >> 13)
    h |= sign << 15
    return h.astype(np.uint16).view(np.float16).astype(np.float32)


def f16_rn(x):
    """IEEE round-to-nearest-even fp32->fp16->fp32."""
    return _c32(x).astype(np.float16).astype(np.float32)


# ---------------------------------------------------------------- numpy pieces
def gemm_f64(A, B, trans_a=False, trans_b=False):
    """float64 reference product of float32 operands as stored (numpy / OpenBLAS)."""
    A64 = np.asarray(A, dtype=np.float64)
    B64 = np.asarray(B, dtype=np.float64)
    return (A64.T if trans_a else A64) @ (B64.T if trans_b else B64)


def rel_frobenius(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    d = np.asarray(got, dtype=np.float64) - ref
    return float(np.linalg.norm(d) / max(np.linalg.norm(ref), 1e-300))


def apply_act_f64(z, act, alpha=0.0):
    z = np.asarray(z, dtype=np.float64)
    if act == 0:
        return np.maximum(z, 0.0)
    if act == 1:
        return np.where(z > 0, z, z * alpha)
    if act == 2:
        return 1.0 / (1.0 + np.exp(-z))
    if act == 3:
        return np.tanh(z)
    if act == 4:
        return 0.5 * z * (1.0 + np.tanh(0.7978845608 * (z + 0.044715 * z ** 3)))
    return z


# ---------------------------------------------------------------- model of the fp32-accuracy splits
# The CUDA fp32 path multiplies splits of its operands on the tensor cores.  These functions
# restate the splits (not the tensor cores: products and sums are exact here), so that a test
# can bound what the splits alone cost and show that small integers pass through unchanged.
def _round_mantissa(x, keep, ties_away):
    """float32 -> float32 with `keep` explicit mantissa bits (exponent range unchanged):
    ties away from zero (cvt.rna.tf32) or to even (cvt.rn.bf16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    drop = np.uint64(23 - keep)
    half = np.uint64(1) << (drop - np.uint64(1))
    if ties_away:
        u = u + half
    else:
        u = u + (half - np.uint64(1)) + ((u >> drop) & np.uint64(1))
    u = (u >> drop) << drop
    return u.astype(np.uint32).view(np.float32)


def split_tf32(x):
    """(hi, lo): hi = rna_tf32(x), lo = rna_tf32(x - hi), as the pre-pass of the single-CTA kernel."""
    hi = _round_mantissa(x, 10, True)
    return hi, _round_mantissa((np.asarray(x, np.float32) - hi).astype(np.float32), 10, True)


def split_tf32_bf16(x):
    """(hi, bf16(hi), bf16(x - hi)) as the pre-pass of the CTA-pair kernel."""
    hi = _round_mantissa(x, 10, True)
    return hi, _round_mantissa(hi, 7, False), _round_mantissa((np.asarray(x, np.float32) - hi).astype(np.float32), 7, False)


def gemm_split_model(A, B, bf16_corrections):
    """A.B from the splits with exact arithmetic: hi.hi + hi.lo + lo.hi (lo.lo is dropped), the
    two correction products from tf32 or from bf16 planes."""
    f = lambda X, Y: X.astype(np.float64) @ Y.astype(np.float64)  # noqa: E731
    if bf16_corrections:
        ah, ahb, alb = split_tf32_bf16(A)
        bh, bhb, blb = split_tf32_bf16(B)
        return f(ah, bh) + f(ahb, blb) + f(alb, bhb)
    ah, al = split_tf32(A)
    bh, bl = split_tf32(B)
    return f(ah, bh) + f(ah, bl) + f(al, bh)


# Seeded inputs of the benchmark configurations: numpy PCG64, drawn in float64
# in the order listed, cast to float32, row-major.
def config1(n=1024):
    rng = np.random.default_rng(0)
    return (rng.uniform(-1, 1, (n, n)).astype(np.float32), rng.uniform(-1, 1, (n, n)).astype(np.float32))


def config2(n=4096):
    rng = np.random.default_rng(1)
    s = 1.0 / np.sqrt(n)
    return ((rng.standard_normal((n, n)) * s).astype(np.float32),
            (rng.standard_normal((n, n)) * s).astype(np.float32))


def config3(batch=512, dims=(784, 1024, 1024, 10)):
    rng = np.random.default_rng(2)
    X = rng.uniform(0, 1, (batch, dims[0])).astype(np.float32)
    Ws = [(rng.standard_normal((dims[i], dims[i + 1])) * np.sqrt(2.0 / dims[i])).astype(np.float32)
          for i in range(3)]
    bs = [np.zeros(dims[i + 1], dtype=np.float32) for i in range(3)]
    dYs = [(rng.standard_normal((batch, dims[i + 1])) * 1e-2).astype(np.float32) for i in range(3)]
    return X, Ws, bs, dYs


def config4(n=8192):
    rng = np.random.default_rng(3)
    s = 1.0 / np.sqrt(n)
    return ((rng.standard_normal((n, n)) * s).astype(np.float32),
            (rng.standard_normal((n, n)) * s).astype(np.float32))


def config5(m=131072, k=4096, n=4096):
    rng = np.random.default_rng(4)
    s = 1.0 / np.sqrt(k)
    A = np.empty((m, k), dtype=np.float32)
    step = 8192
    for r in range(0, m, step):  # blockwise to bound float64 temporaries
        A[r:r + step] = rng.standard_normal((min(step, m - r), k)) * s
    B = (rng.standard_normal((k, n)) * s).astype(np.float32)
    return A, B


# ---------------------------------------------------------------- element-wise family
def elementwise(op, a, b, out=None):
    """op: 0 add, 1 subtract, 2 multiply, 3 divide.  Returns (code, result, zero_index);
    `out` gives the previous contents of the result (the divide may leave a tail untouched)."""
    h = lib()
    h.oracle_elementwise.argtypes = [_i, _f32p, _f32p, _f32p, _l, ctypes.POINTER(_l)]
    h.oracle_elementwise.restype = _i
    a, b = _c32(a), _c32(b)
    r = _c32(out).copy() if out is not None else np.zeros_like(a)
    z = _l(-1)
    rc = h.oracle_elementwise(op, _p32(a), _p32(b), _p32(r), a.size, ctypes.byref(z))
    return rc, r, z.value


def scalar_op(multiply, x, scalar):
    h = lib()
    h.oracle_scalar_op.argtypes = [_i, _f32p, _f, _f32p, _l]
    h.oracle_scalar_op.restype = None
    x = _c32(x)
    out = np.empty_like(x)
    h.oracle_scalar_op(int(multiply), _p32(x), scalar, _p32(out), x.size)
    return out


def activation_forward(kind, x, alpha=0.0):
    """kind: 0 sigmoid, 1 tanh, 2 leaky ReLU, 3 ELU, 4 Swish, 5 GELU."""
    h = lib()
    fn = h.oracle_activation_forward if kind < 3 else h.oracle_activation2_forward
    fn.argtypes = [_i, _f32p, _f32p, _l, _f]
    fn.restype = None
    x = _c32(x)
    out = np.empty_like(x)
    fn(kind, _p32(x), _p32(out), x.size, alpha)
    return out


def activation_backward(kind, grad_out, act_out, alpha=0.0):
    h = lib()
    fn = h.oracle_activation_backward if kind < 3 else h.oracle_activation2_backward
    fn.argtypes = [_i, _f32p, _f32p, _f32p, _l, _f]
    fn.restype = None
    g, a = _c32(grad_out), _c32(act_out)
    out = np.empty_like(g)
    fn(kind, _p32(g), _p32(a), _p32(out), g.size, alpha)
    return out


def softmax_forward(x):
    """Row softmax of a [batch, features] array (a vector counts as one row)."""
    h = lib()
    h.oracle_softmax_forward.argtypes = [_f32p, _f32p, _l, _l]
    h.oracle_softmax_forward.restype = None
    x = _c32(x)
    x2 = x.reshape(1, -1) if x.ndim == 1 else x
    out = np.empty_like(x2)
    h.oracle_softmax_forward(_p32(x2), _p32(out), x2.shape[0], x2.shape[1])
    return out.reshape(x.shape)


def softmax_backward(grad_out, act):
    h = lib()
    h.oracle_softmax_backward.argtypes = [_f32p, _f32p, _f32p, _l, _l]
    h.oracle_softmax_backward.restype = None
    g, a = _c32(grad_out), _c32(act)
    g2 = g.reshape(1, -1) if g.ndim == 1 else g
    out = np.empty_like(g2)
    h.oracle_softmax_backward(_p32(g2), _p32(a), _p32(out), g2.shape[0], g2.shape[1])
    return out.reshape(g.shape)
