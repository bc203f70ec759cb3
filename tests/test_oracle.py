"""CPU tests of the oracle itself: against the reference's own known-answer
vectors, against the committed golden file, and against independent numpy
restatements."""
import numpy as np
import pytest

from oracle import oracle


def test_relu_kats_from_reference(golden):
    ref, _ = golden
    k = ref["relu_forward"]
    got = oracle.relu_forward(np.array(k["input"], np.float32))
    assert np.allclose(got, k["expected"], atol=1e-6)
    k = ref["relu_backward"]
    got = oracle.relu_backward(np.array(k["grad_output"], np.float32),
                               np.array(k["activation_output"], np.float32))
    assert np.allclose(got, k["expected"], atol=1e-6)


def test_activation_kats_through_fused_oracle(golden):
    """The reference's activation tests, driven through the fused-linear oracle
    with an identity weight so that the pre-activation equals the input."""
    ref, _ = golden
    eye = np.eye(4, dtype=np.float32)
    k = ref["leaky_relu_forward"]
    got = oracle.fused_linear_activation(np.array([k["input"]], np.float32), eye, None, 1, k["alpha"])
    assert np.allclose(got[0], k["expected"], atol=1e-6)
    for name, code in (("sigmoid_forward", 2), ("tanh_forward", 3)):
        k = ref[name]
        got = oracle.fused_linear_activation(np.array([k["input"]], np.float32), eye, None, code, 0.0)[0]
        assert abs(got[k["index_of_zero"]] - k["expected_at_zero"]) <= 1e-6
        assert (got >= k["range"][0]).all() and (got <= k["range"][1]).all()


def test_oracle_matches_committed_golden(golden):
    _, g = golden
    for name in ("int_a", "int_b", "int_c"):
        C = oracle.gemm_f64_naive(g[f"{name}_A"], g[f"{name}_B"])
        assert np.array_equal(C.astype(np.float32), g[f"{name}_C"])
    assert np.array_equal(oracle.gemm_f64_naive(g["perm_P"], g["perm_V"]).astype(np.float32), g["perm_C"])
    assert np.array_equal(oracle.transpose(g["tr_in"]).view(np.uint32), g["tr_out"].view(np.uint32))
    assert np.array_equal(oracle.f16_trunc(g["f16_in"]).view(np.uint32), g["f16_trunc_out"].view(np.uint32))
    for act in (0, 1, 2, 3, 4, 9):
        got = oracle.fused_linear_activation(g["fl_X"], g["fl_W"], g["fl_b"], act, 0.25)
        assert np.allclose(got, g[f"fl_act{act}_f32"], rtol=0, atol=1e-6)
        assert oracle.rel_frobenius(got, g[f"fl_act{act}_f64"]) < 1e-6
    assert np.array_equal(oracle.gemm_alpha_beta(g["ab_A"], g["ab_B"], g["ab_C0"], 0.5, -2.0), g["ab_out"])
    assert np.array_equal(oracle.add_broadcast(g["bc_M"], g["bc_row"], (6, 11))[1], g["bc_m_row"])
    assert np.array_equal(oracle.add_broadcast(g["bc_col"], g["bc_M"], (6, 11))[1], g["bc_col_m"])
    assert np.array_equal(oracle.column_sum(g["colsum_in"]), g["colsum_out"])


def test_naive_c_gemm_agrees_with_numpy_float64():
    rng = np.random.default_rng(5)
    for (m, n, k) in [(1, 1, 1), (33, 17, 129), (128, 96, 200)]:
        A = rng.standard_normal((m, k)).astype(np.float32)
        B = rng.standard_normal((k, n)).astype(np.float32)
        ref = oracle.gemm_f64(A, B)
        assert oracle.rel_frobenius(oracle.gemm_f64_naive(A, B), ref) < 1e-14
        assert oracle.rel_frobenius(oracle.gemm_f64_naive(np.ascontiguousarray(A.T), B, True, False), ref) < 1e-14
        assert oracle.rel_frobenius(oracle.gemm_f64_naive(A, np.ascontiguousarray(B.T), False, True), ref) < 1e-14


def test_transpose_index_formula():
    X = np.arange(12, dtype=np.float32).reshape(3, 4)
    assert np.array_equal(oracle.transpose(X), X.T)
    assert oracle.lib().oracle_transpose(None, 3, 4, None, 3, 4) == -2  # dimension check comes first


def test_f16_truncation_properties():
    rng = np.random.default_rng(6)
    x = (rng.standard_normal(50000) * 10.0 ** rng.integers(-9, 6, 50000)).astype(np.float32)
    t = oracle.f16_trunc(x)
    assert np.array_equal(t.view(np.uint32), oracle.f16_trunc_numpy(x).view(np.uint32))
    # truncation never increases magnitude; results are fp16-representable
    fin = np.isfinite(t)
    assert (np.abs(t[fin]) <= np.abs(x[fin])).all()
    assert np.array_equal(t[fin].astype(np.float16).astype(np.float32), t[fin])
    # idempotent
    assert np.array_equal(oracle.f16_trunc(t).view(np.uint32), t.view(np.uint32))
    # overflow goes to infinity, tiny values flush to signed zero
    assert np.isinf(oracle.f16_trunc(np.array([70000.0], np.float32))[0])
    z = oracle.f16_trunc(np.array([-1e-9], np.float32))
    assert z[0] == 0.0 and np.signbit(z[0])


def test_add_broadcast_rejects_other_shapes():
    a = np.zeros((2, 3), np.float32)
    rc, _ = oracle.add_broadcast(a, np.zeros((2, 2), np.float32), (2, 3))
    assert rc == -2


def test_config_generators_are_seeded_and_shaped():
    A, B = oracle.config1(64)
    A2, B2 = oracle.config1(64)
    assert np.array_equal(A, A2) and np.array_equal(B, B2)
    assert A.dtype == np.float32 and A.min() >= -1 and A.max() < 1
    X, Ws, bs, dYs = oracle.config3(8)
    assert X.shape == (8, 784) and [w.shape for w in Ws] == [(784, 1024), (1024, 1024), (1024, 10)]
    assert all((b == 0).all() for b in bs) and [d.shape for d in dYs] == [(8, 1024), (8, 1024), (8, 10)]
    A, B = oracle.config5(256, 64, 32)
    assert A.shape == (256, 64) and B.shape == (64, 32)
    assert abs(A.std() - 1 / 8) < 0.01


def test_elementwise_family_against_reference_kats_and_numpy(golden):
    ref, _ = golden
    k = ref["leaky_relu_forward"]
    assert np.allclose(oracle.activation_forward(2, np.array(k["input"], np.float32), k["alpha"]), k["expected"], atol=1e-6)
    k = ref["sigmoid_forward"]
    s = oracle.activation_forward(0, np.array(k["input"], np.float32))
    assert abs(s[k["index_of_zero"]] - 0.5) <= 1e-6 and (s >= 0).all() and (s <= 1).all()
    k = ref["tanh_forward"]
    t = oracle.activation_forward(1, np.array(k["input"], np.float32))
    assert abs(t[k["index_of_zero"]]) <= 1e-6 and (np.abs(t) <= 1).all()
    rng = np.random.default_rng(3)
    a, b = rng.standard_normal(1000).astype(np.float32), rng.standard_normal(1000).astype(np.float32)
    for op, fn in ((0, np.add), (1, np.subtract), (2, np.multiply), (3, np.divide)):
        rc, r, _ = oracle.elementwise(op, a, b)
        assert rc == 0 and np.array_equal(r, fn(a, b))
    b[17] = 0.0
    b[500] = -0.0
    rc, r, z = oracle.elementwise(3, a, b, out=np.full(1000, 7.0, np.float32))
    assert rc == -4 and z == 17 and np.array_equal(r[:17], a[:17] / b[:17]) and (r[17:] == 7.0).all()
    assert np.array_equal(oracle.scalar_op(False, a, 1.5), a + np.float32(1.5))
    assert np.array_equal(oracle.scalar_op(True, a, 1.5), a * np.float32(1.5))
    # clamping: huge inputs neither overflow nor produce NaN
    big = np.array([-1e30, -100, 100, 1e30], np.float32)
    assert np.isfinite(oracle.activation_forward(0, big)).all() and np.isfinite(oracle.activation_forward(1, big)).all()


def test_softmax_elu_swish_gelu_against_reference_properties(golden):
    ref, _ = golden
    k = ref["softmax_forward"]
    s = oracle.softmax_forward(np.array(k["input"], np.float32))
    assert abs(float(s.sum(dtype=np.float32)) - 1.0) <= 1e-6 and (s > 0).all()
    k = ref["softmax_2d_forward"]
    s = oracle.softmax_forward(np.array(k["input"], np.float32).reshape(k["shape"]))
    assert (np.abs(s.sum(axis=1, dtype=np.float32) - 1.0) <= 1e-6).all()
    k = ref["elu_forward"]
    e = oracle.activation_forward(3, np.array(k["input"], np.float32), k["alpha"])
    assert abs(e[k["index_of_one"]] - 1.0) <= 1e-6 and e[0] < 0 and e[1] < 0
    for kind, key in ((4, "swish_forward"), (5, "gelu_forward")):
        k = ref[key]
        y = oracle.activation_forward(kind, np.array(k["input"], np.float32))
        assert abs(y[k["index_of_zero"]]) <= 1e-6
    # independent float64 statement of the same functions
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(2000) * 3).astype(np.float32)
    x64 = x.astype(np.float64)
    assert np.allclose(oracle.activation_forward(3, x, 0.7), np.where(x64 > 0, x64, 0.7 * np.expm1(x64)), atol=1e-6)
    assert np.allclose(oracle.activation_forward(4, x), x64 / (1 + np.exp(-x64)), atol=1e-6)
    g = 0.5 * x64 * (1 + np.tanh(0.7978845608028654 * (x64 + 0.044715 * x64 ** 3)))
    assert np.allclose(oracle.activation_forward(5, x), g, atol=1e-6)
    X = rng.standard_normal((7, 33)).astype(np.float32)
    e = np.exp(X.astype(np.float64) - X.max(axis=1, keepdims=True))
    sm = e / e.sum(axis=1, keepdims=True)
    assert np.allclose(oracle.softmax_forward(X), sm, atol=1e-6)
    G = rng.standard_normal((7, 33)).astype(np.float32)
    assert np.allclose(oracle.softmax_backward(G, sm.astype(np.float32)),
                       sm * (G - (G * sm).sum(axis=1, keepdims=True)), atol=1e-6)


# ---------------------------------------------------------------- the fp32-accuracy splits
@pytest.mark.parametrize("bf16", [False, True])
def test_split_model_stays_far_below_the_fp32_tolerance(bf16):
    """What the operand splits of the CUDA fp32 path cost by themselves (exact products and
    sums): below 1e-6 relative Frobenius error for both kinds of correction planes, on
    benchmark-like data, on all-positive data and on elements spread over twelve decades; the
    stated tolerance of the path is 1e-5."""
    rng = np.random.default_rng(11)
    k = 1024
    cases = {
        "normal": ((rng.standard_normal((96, k)) / np.sqrt(k)), (rng.standard_normal((k, 80)) / np.sqrt(k))),
        "uniform": (rng.random((96, k)), rng.random((k, 80))),
        "decades": (rng.standard_normal((96, k)) * 10.0 ** rng.integers(-6, 7, (96, k)),
                    rng.standard_normal((k, 80)) * 10.0 ** rng.integers(-6, 7, (k, 80))),
    }
    for name, (A, B) in cases.items():
        A, B = A.astype(np.float32), B.astype(np.float32)
        err = oracle.rel_frobenius(oracle.gemm_split_model(A, B, bf16), oracle.gemm_f64(A, B))
        assert err <= (1e-6 if bf16 else 2e-7), (name, err)


def test_split_model_is_exact_on_small_integers_and_splits_add_up():
    rng = np.random.default_rng(12)
    A = rng.integers(-8, 9, (40, 300)).astype(np.float32)
    B = rng.integers(-8, 9, (300, 24)).astype(np.float32)
    for bf16 in (False, True):
        assert np.array_equal(oracle.gemm_split_model(A, B, bf16), oracle.gemm_f64(A, B))
    x = (rng.standard_normal(4096) * 10.0 ** rng.integers(-20, 20, 4096)).astype(np.float32)
    hi, lo = oracle.split_tf32(x)
    assert np.all(np.abs(x.astype(np.float64) - hi.astype(np.float64) - lo.astype(np.float64))
                  <= np.abs(x.astype(np.float64)) * 2.0 ** -21)
    assert np.all((hi.view(np.uint32) & 0x1FFF) == 0) and np.all((lo.view(np.uint32) & 0x1FFF) == 0)
    hi2, hb, lb = oracle.split_tf32_bf16(x)
    assert np.array_equal(hi, hi2)
    assert np.all((hb.view(np.uint32) & 0xFFFF) == 0) and np.all((lb.view(np.uint32) & 0xFFFF) == 0)
    # bf16(hi) is hi to 2^-9, bf16(lo) is x - hi to 2^-9 of itself
    assert np.all(np.abs(hb.astype(np.float64) - hi) <= np.abs(hi.astype(np.float64)) * 2.0 ** -8)
    assert np.all(np.abs(lb.astype(np.float64) - (x.astype(np.float64) - hi)) <= np.abs(x.astype(np.float64) - hi) * 2.0 ** -8 + 1e-45)
