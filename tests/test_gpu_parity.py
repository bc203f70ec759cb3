"""Parity of the CUDA path against the CPU oracle, through the C ABI.

Tolerances (stated by the benchmark contract): fp32 path relative Frobenius
error <= 1e-5 against the float64 reference; fp16 path <= 1e-2; Transpose and
the other element-moving / exact-integer cases bit-exact.
"""
import ctypes

import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
FP16_TOL = 1e-2


def run_matmul(g, A, B, trans_a=False, trans_b=False, precision=0, alpha=1.0, beta=0.0, C0=None,
               bias=None, act=-1, act_param=0.0, entry="ex"):
    """A and B are given as STORED; returns the float32 result."""
    M = A.shape[1] if trans_a else A.shape[0]
    N = B.shape[0] if trans_b else B.shape[1]
    a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
    c = g.Buffer.from_host(C0 if C0 is not None else np.full((M, N), np.float32(-123.0), np.float32))
    bb = g.Buffer.from_host(bias) if bias is not None else None
    try:
        if entry == "mps":
            g.matmul(a, A.shape, b, B.shape, c, (M, N))
        else:
            g.matmul_ex(a, A.shape, trans_a, b, B.shape, trans_b, c, (M, N), precision=precision,
                        alpha=alpha, beta=beta, bias=bb, act=act, act_param=act_param)
        return c.retrieve((M, N))
    finally:
        for x in (a, b, c, bb):
            if x is not None:
                x.release()


# ------------------------------------------------------------------ known answers
def test_golden_integer_and_permutation_gemms_are_exact(gpu, golden):
    _, k = golden
    for name in ("int_a", "int_b", "int_c"):
        for prec in (gpu.FP32_3XTF32, gpu.FP16_RN, gpu.FP16_TRUNC):
            C = run_matmul(gpu, k[f"{name}_A"], k[f"{name}_B"], precision=prec)
            assert np.array_equal(C, k[f"{name}_C"]), (name, prec)
    C = run_matmul(gpu, k["perm_P"], k["perm_V"], entry="mps")
    assert np.array_equal(C, k["perm_C"])
    # the same products with transposed storage (no materialised transpose inside)
    A, B = k["int_b_A"], k["int_b_B"]
    for ta in (False, True):
        for tb in (False, True):
            for prec in (gpu.FP32_3XTF32, gpu.FP16_RN):
                As = np.ascontiguousarray(A.T) if ta else A
                Bs = np.ascontiguousarray(B.T) if tb else B
                assert np.array_equal(run_matmul(gpu, As, Bs, ta, tb, precision=prec), k["int_b_C"])


def test_reference_activation_kats(gpu, golden):
    ref, _ = golden
    k = ref["relu_forward"]
    x = np.array(k["input"], np.float32)
    i, o = gpu.Buffer.from_host(x), gpu.Buffer.empty(x.nbytes)
    gpu.relu_forward(i, x.size, o)
    assert np.allclose(o.retrieve(x.shape), k["expected"], atol=1e-6)
    k = ref["relu_backward"]
    go = gpu.Buffer.from_host(np.array(k["grad_output"], np.float32))
    ao = gpu.Buffer.from_host(np.array(k["activation_output"], np.float32))
    gi = gpu.Buffer.empty(24)
    gpu.relu_backward(go, ao, 6, gi)
    assert np.allclose(gi.retrieve((6,)), k["expected"], atol=1e-6)
    # the other activation vectors go through the fused epilogue with W = I
    eye = np.eye(4, dtype=np.float32)
    k = ref["leaky_relu_forward"]
    got = run_matmul(gpu, np.array([k["input"]], np.float32), eye, act=1, act_param=k["alpha"])
    assert np.allclose(got[0], k["expected"], atol=1e-6)
    for name, code in (("sigmoid_forward", 2), ("tanh_forward", 3)):
        k = ref[name]
        got = run_matmul(gpu, np.array([k["input"]], np.float32), eye, act=code)[0]
        assert abs(got[k["index_of_zero"]] - k["expected_at_zero"]) <= 1e-6
        assert (got >= k["range"][0]).all() and (got <= k["range"][1]).all()


# ------------------------------------------------------------------ seeded parity
@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 3, 4), (31, 33, 35), (128, 128, 128), (129, 257, 65),
                                   (200, 300, 136), (257, 10, 784), (512, 1024, 784), (1000, 1000, 1000),
                                   (64, 2048, 96), (3000, 40, 520)])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_fp32_path_matches_float64_reference(gpu, shape, layout):
    m, n, k = shape
    rng = np.random.default_rng(m * 1000003 + n * 1009 + k)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    ta, tb = layout[0] == "t", layout[1] == "t"
    As = np.ascontiguousarray(A.T) if ta else A
    Bs = np.ascontiguousarray(B.T) if tb else B
    C = run_matmul(gpu, As, Bs, ta, tb, precision=gpu.FP32_3XTF32)
    ref = oracle.gemm_f64(As, Bs, ta, tb)
    assert oracle.rel_frobenius(C, ref) <= FP32_TOL


@pytest.mark.parametrize("shape", [(1, 1, 1), (5, 7, 3), (128, 64, 64), (129, 257, 65), (200, 300, 136),
                                   (257, 10, 784), (1024, 1024, 1024), (96, 4096, 160)])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
@pytest.mark.parametrize("mode", ["rn", "trunc"])
def test_fp16_path_matches_float64_reference(gpu, shape, layout, mode):
    m, n, k = shape
    rng = np.random.default_rng(m * 7919 + n * 104729 + k)
    A = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
    B = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    ta, tb = layout[0] == "t", layout[1] == "t"
    As = np.ascontiguousarray(A.T) if ta else A
    Bs = np.ascontiguousarray(B.T) if tb else B
    prec = gpu.FP16_RN if mode == "rn" else gpu.FP16_TRUNC
    C = run_matmul(gpu, As, Bs, ta, tb, precision=prec)
    rnd = oracle.f16_rn if mode == "rn" else oracle.f16_trunc
    # against the float64 product of the fp16-rounded inputs the only error left is
    # the fp32 accumulation; against the unrounded inputs it is the fp16 tolerance
    assert oracle.rel_frobenius(C, oracle.gemm_f64(rnd(As), rnd(Bs), ta, tb)) <= 2e-5
    assert oracle.rel_frobenius(C, oracle.gemm_f64(As, Bs, ta, tb)) <= FP16_TOL


def test_every_small_shape_fp32_and_fp16(gpu):
    """All M, N, K in a ragged set: tile edges, K tails, single rows/columns."""
    sizes = [1, 2, 3, 7, 8, 15, 16, 17, 31, 33, 63, 64, 65, 127, 129]
    rng = np.random.default_rng(11)
    bad = []
    for m in sizes:
        for n in sizes:
            for k in (1, 5, 8, 31, 32, 33, 64, 65, 130):
                A = rng.integers(-3, 4, (m, k)).astype(np.float32)
                B = rng.integers(-3, 4, (k, n)).astype(np.float32)
                ref = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)
                prec = gpu.FP32_3XTF32 if (m + n + k) % 2 else gpu.FP16_RN
                if not np.array_equal(run_matmul(gpu, A, B, precision=prec), ref):
                    bad.append((m, n, k, prec))
    assert not bad, bad[:10]


def test_tile_overrides_agree(gpu):
    rng = np.random.default_rng(12)
    A = rng.standard_normal((300, 200)).astype(np.float32)
    B = rng.standard_normal((200, 700)).astype(np.float32)
    ref = oracle.gemm_f64(A, B)
    try:
        for bn in (32, 64, 128, 256):
            assert gpu.lib().gonngpu_set_gemm_tuning(bn, 0) == 0
            assert oracle.rel_frobenius(run_matmul(gpu, A, B, precision=gpu.FP32_3XTF32), ref) <= FP32_TOL
            assert oracle.rel_frobenius(run_matmul(gpu, A, B, precision=gpu.FP16_RN),
                                        oracle.gemm_f64(oracle.f16_rn(A), oracle.f16_rn(B))) <= 2e-5
        # fewer CTAs than tiles: every CTA walks several tiles (persistent loop, both accumulators)
        assert gpu.lib().gonngpu_set_gemm_tuning(64, 3) == 0
        assert oracle.rel_frobenius(run_matmul(gpu, A, B, precision=gpu.FP32_3XTF32), ref) <= FP32_TOL
    finally:
        gpu.lib().gonngpu_set_gemm_tuning(0, 0)


# ------------------------------------------------------------------ epilogues
def test_fused_linear_activation_matches_oracle(gpu, golden):
    _, k = golden
    X, W, b = k["fl_X"], k["fl_W"], k["fl_b"]
    x, w, bb = gpu.Buffer.from_host(X), gpu.Buffer.from_host(W), gpu.Buffer.from_host(b)
    y = gpu.Buffer.empty(X.shape[0] * W.shape[1] * 4)
    for act in (0, 1, 2, 3, 4, 9):
        gpu.fused_linear_activation(x, X.shape[0], X.shape[1], w, W.shape[1], bb, act, 0.25, y)
        got = y.retrieve((X.shape[0], W.shape[1]))
        assert oracle.rel_frobenius(got, k[f"fl_act{act}_f64"]) <= FP32_TOL, act
        assert np.allclose(got, k[f"fl_act{act}_f32"], rtol=0, atol=2e-5), act
    # bias is optional
    gpu.fused_linear_activation(x, X.shape[0], X.shape[1], w, W.shape[1], None, 0, 0.0, y)
    ref = oracle.fused_linear_activation_f64(X, W, None, 0, 0.0)
    assert oracle.rel_frobenius(y.retrieve(ref.shape), ref) <= FP32_TOL


def test_fused_linear_seeded_ragged(gpu):
    rng = np.random.default_rng(13)
    for (bsz, fin, fout) in [(1, 1, 1), (33, 70, 10), (512, 784, 1024), (130, 257, 999)]:
        X = rng.uniform(0, 1, (bsz, fin)).astype(np.float32)
        W = (rng.standard_normal((fin, fout)) * np.sqrt(2.0 / fin)).astype(np.float32)
        b = rng.standard_normal(fout).astype(np.float32)
        for act in (0, 4):
            got = run_matmul(gpu, X, W, bias=b, act=act)
            assert oracle.rel_frobenius(got, oracle.fused_linear_activation_f64(X, W, b, act, 0.0)) <= FP32_TOL


def test_alpha_beta_gemm(gpu, golden):
    _, k = golden
    a, b = gpu.Buffer.from_host(k["ab_A"]), gpu.Buffer.from_host(k["ab_B"])
    c = gpu.Buffer.from_host(k["ab_C0"].copy())
    gpu.optimized_gemm(a, b, c, 17, 21, 12, 0.5, -2.0)
    assert np.array_equal(c.retrieve((17, 21)), k["ab_out"])  # small integers and halves: exact
    rng = np.random.default_rng(14)
    A = rng.standard_normal((150, 90)).astype(np.float32)
    B = rng.standard_normal((90, 260)).astype(np.float32)
    C0 = rng.standard_normal((150, 260)).astype(np.float32)
    got = run_matmul(gpu, A, B, alpha=1.5, beta=0.75, C0=C0.copy())
    ref = 1.5 * oracle.gemm_f64(A, B) + 0.75 * C0.astype(np.float64)
    assert oracle.rel_frobenius(got, ref) <= FP32_TOL


# ------------------------------------------------------------------ HBM-bound kernels
@pytest.mark.parametrize("shape", [(1, 1), (1, 9), (9, 1), (37, 101), (64, 64), (65, 63), (130, 260),
                                   (1000, 36), (4096, 4096), (2051, 4099)])
def test_transpose_is_bit_exact(gpu, shape):
    rng = np.random.default_rng(shape[0] * 31 + shape[1])
    X = rng.standard_normal(shape).astype(np.float32)
    flat = X.reshape(-1)
    flat[0] = np.float32("nan")
    flat[-1] = np.float32("-0.0")
    i, o = gpu.Buffer.from_host(X), gpu.Buffer.empty(X.nbytes)
    gpu.transpose(i, X.shape, o)
    got = o.retrieve((shape[1], shape[0]))
    assert np.array_equal(got.view(np.uint32), oracle.transpose(X).view(np.uint32))
    # involution: transposing back restores the input bit for bit
    o2 = gpu.Buffer.empty(X.nbytes)
    gpu.transpose(o, (shape[1], shape[0]), o2)
    assert np.array_equal(o2.retrieve(shape).view(np.uint32), X.view(np.uint32))


def test_golden_transpose_broadcast_colsum_f16(gpu, golden):
    _, k = golden
    i, o = gpu.Buffer.from_host(k["tr_in"]), gpu.Buffer.empty(k["tr_in"].nbytes)
    gpu.transpose(i, k["tr_in"].shape, o)
    assert np.array_equal(o.retrieve(k["tr_out"].shape).view(np.uint32), k["tr_out"].view(np.uint32))
    M, row, col = k["bc_M"], k["bc_row"], k["bc_col"]
    m, r, c = gpu.Buffer.from_host(M), gpu.Buffer.from_host(row), gpu.Buffer.from_host(col)
    out = gpu.Buffer.empty(M.nbytes)
    for (x, xs, y, ys, key) in [(m, M.shape, r, row.shape, "bc_m_row"), (r, row.shape, m, M.shape, "bc_row_m"),
                                (m, M.shape, c, col.shape, "bc_m_col"), (c, col.shape, m, M.shape, "bc_col_m")]:
        gpu.add_broadcast(x, xs, y, ys, out, M.shape)
        assert np.array_equal(out.retrieve(M.shape), k[key])
    with pytest.raises(gpu.GonnError) as e:
        gpu.add_broadcast(m, M.shape, m, (2, 2), out, M.shape)
    assert e.value.code == -2 and "Unsupported broadcasting pattern" in e.value.message
    cs = gpu.Buffer.empty(M.shape[1] * 4)
    gpu.column_sum(m, M.shape[0], M.shape[1], cs)
    assert np.allclose(cs.retrieve((M.shape[1],)), k["colsum_out"], rtol=1e-6, atol=1e-6)
    # the truncating fp16 conversion is exercised through a product with the identity:
    # C = trunc16(x) exactly (fp16 values times 1, fp32 accumulate)
    x = k["f16_in"][np.isfinite(k["f16_trunc_out"]) & np.isfinite(k["f16_in"])][:1024].reshape(16, 64)
    got = run_matmul(gpu, x, np.eye(64, dtype=np.float32), precision=gpu.FP16_TRUNC)
    assert np.array_equal(got, oracle.f16_trunc(x))  # float compare: -0 == +0
    got = run_matmul(gpu, x, np.eye(64, dtype=np.float32), precision=gpu.FP16_RN)
    assert np.array_equal(got, oracle.f16_rn(x))


# ------------------------------------------------------------------ the benchmark configurations
def test_config1_fp32_1024(gpu):
    A, B = oracle.config1()
    C = run_matmul(gpu, A, B, entry="mps")
    assert oracle.rel_frobenius(C, oracle.gemm_f64(A, B)) <= FP32_TOL


def test_config2_fp32_4096_all_layouts_and_transpose(gpu):
    A, B = oracle.config2()
    ref = oracle.gemm_f64(A, B)
    assert oracle.rel_frobenius(run_matmul(gpu, A, B, entry="mps"), ref) <= FP32_TOL
    At = np.ascontiguousarray(A.T)
    assert oracle.rel_frobenius(run_matmul(gpu, At, B, True, False), ref) <= FP32_TOL
    Bt = np.ascontiguousarray(B.T)
    assert oracle.rel_frobenius(run_matmul(gpu, A, Bt, False, True), ref) <= FP32_TOL
    i, o = gpu.Buffer.from_host(A), gpu.Buffer.empty(A.nbytes)
    gpu.transpose(i, A.shape, o)
    assert np.array_equal(o.retrieve(At.shape).view(np.uint32), At.view(np.uint32))


def test_config3_mlp_training_step_gemm_set(gpu):
    X, Ws, bs, dYs = oracle.config3()
    h = X
    for layer in range(3):
        act = 0 if layer < 2 else -1
        y = run_matmul(gpu, h, Ws[layer], bias=bs[layer], act=act)
        ref = oracle.apply_act_f64(oracle.gemm_f64(h, Ws[layer]) + bs[layer].astype(np.float64), act)
        assert oracle.rel_frobenius(y, ref) <= FP32_TOL, ("fwd", layer)
        # backward GEMMs on the given dY: dW = h^T . dY, dX = dY . W^T
        dW = run_matmul(gpu, h, dYs[layer], True, False)
        assert oracle.rel_frobenius(dW, oracle.gemm_f64(h, dYs[layer], True, False)) <= FP32_TOL, ("dW", layer)
        dX = run_matmul(gpu, dYs[layer], Ws[layer], False, True)
        assert oracle.rel_frobenius(dX, oracle.gemm_f64(dYs[layer], Ws[layer], False, True)) <= FP32_TOL, ("dX", layer)
        h = y


def _row_sample(m, shards=8, per_shard=24, seed=0):
    rng = np.random.default_rng(seed)
    rows = set()
    for s in range(shards):
        lo, hi = s * m // shards, (s + 1) * m // shards
        rows.update([lo, hi - 1])
        rows.update(rng.integers(lo, hi, per_shard).tolist())
    return np.array(sorted(rows))


def test_config4_fp16_8192_sampled_rows_and_checksum(gpu):
    A, B = oracle.config4()
    C = run_matmul(gpu, A, B, precision=gpu.FP16_RN)
    rows = _row_sample(A.shape[0])
    ref_rows = oracle.gemm_f64(A[rows], B)
    assert oracle.rel_frobenius(C[rows], ref_rows) <= FP16_TOL
    assert oracle.rel_frobenius(C[rows], oracle.gemm_f64(oracle.f16_rn(A[rows]), oracle.f16_rn(B))) <= 5e-5
    # full-size property: C.1 == A16.(B16.1) in float64 (a checksum over every output)
    A16, B16 = oracle.f16_rn(A).astype(np.float64), oracle.f16_rn(B).astype(np.float64)
    want = A16 @ (B16 @ np.ones(B.shape[1]))
    got = C.astype(np.float64) @ np.ones(B.shape[1])
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-4


def test_config5_full_size_from_page_locked_host_memory(gpu):
    """The benchmarked configuration at full size (M = 131072, K = N = 4096, fp16 in / fp32
    accumulate) through create_gpu_buffer -> gonngpu_matmul_ex -> retrieve with the matrices in
    page-locked host memory, which is the streamed path (upload, convert, multiply and write-back
    in row blocks): 2048-odd sampled rows, the first and last row of every eighth among them,
    against the float64 oracle on the fp16-rounded inputs, and the checksum C.1 == A16.(B16.1)
    over every output."""
    g = gpu
    m, k, n = 131072, 4096, 4096
    hA, pA = g.pinned_array((m, k))
    hB, pB = g.pinned_array((k, n))
    hC, pC = g.pinned_array((m, n))
    rng = np.random.default_rng(4)                  # the benchmark's inputs: A first, then B
    s = 1.0 / np.sqrt(k)
    for r in range(0, m, 8192):
        np.multiply(rng.standard_normal((8192, k)), s, out=hA[r:r + 8192], casting="same_kind")
    hB[...] = rng.standard_normal((k, n)) * s
    hC[...] = -123.0
    a, b, c = g.Buffer.from_host(hA), g.Buffer.from_host(hB), g.Buffer.from_host(hC)
    try:
        g.matmul_ex(a, (m, k), False, b, (k, n), False, c, (m, n), precision=g.FP16_RN)
        c.retrieve_into(hC)
    finally:
        for x in (a, b, c):
            x.release()
    rows = _row_sample(m, shards=8, per_shard=256)
    assert len(rows) >= 2048
    B16 = oracle.f16_rn(hB)
    ref = oracle.gemm_f64(oracle.f16_rn(hA[rows]), B16)
    assert oracle.rel_frobenius(hC[rows], ref) <= FP16_TOL
    assert oracle.rel_frobenius(hC[rows], ref) <= 5e-5        # exact fp16 products, fp32 accumulation
    b1 = B16.astype(np.float64) @ np.ones(n)
    worst = 0.0
    for r in range(0, m, 8192):                     # blockwise: bounds the float64 temporaries
        want = oracle.f16_rn(hA[r:r + 8192]).astype(np.float64) @ b1
        got = hC[r:r + 8192].astype(np.float64) @ np.ones(n)
        worst = max(worst, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
    assert worst <= 1e-4
    for p in (pA, pB, pC):
        g.lib().gonngpu_host_free(p)


def test_buffer_protocol(gpu):
    """Lazy upload, retrieval of an untouched buffer, size checks, release."""
    x = np.arange(12, dtype=np.float32)
    b = gpu.Buffer.from_host(x)
    assert np.array_equal(b.retrieve((12,)), x)          # never uploaded: host bytes are the contents
    with pytest.raises(gpu.GonnError) as e:
        b.retrieve((13,))
    assert e.value.code == -2 and "length mismatch" in e.value.message
    b.upload(x * 2)
    assert np.array_equal(b.retrieve((12,)), x * 2)
    before = gpu.stats()["buffers"]
    b.release()
    assert gpu.stats()["buffers"] == before - 1
    # dimension errors keep the reference's codes
    a, c = gpu.Buffer.from_host(np.zeros((2, 3), np.float32)), gpu.Buffer.empty(16)
    with pytest.raises(gpu.GonnError) as e:
        gpu.matmul(a, (2, 3), a, (2, 3), c, (2, 2))
    assert e.value.code == -3
    with pytest.raises(gpu.GonnError) as e:
        gpu.transpose(a, (2, 3), gpu.Buffer.empty(8))
    assert e.value.code == -2
    # memory from the unified-memory adapter's allocator works as a buffer
    p = gpu.lib().allocateSharedMemory(64)
    assert p
    arr = np.frombuffer((ctypes.c_char * 64).from_address(p), dtype=np.float32)
    assert (arr == 0).all()
    arr[:] = np.arange(16)
    h = gpu.lib().createGPUBufferFromSharedMemory(None, p, 64)
    assert h
    hb = gpu.Buffer(ctypes.c_void_p(h), 64)
    out = gpu.Buffer.empty(64)
    gpu.transpose(hb, (4, 4), out)
    assert np.array_equal(out.retrieve((4, 4)), np.arange(16, dtype=np.float32).reshape(4, 4).T)
    hb.release()
    gpu.lib().gonngpu_host_free(p)


# ------------------------------------------------------------------ CTA-pair (2-SM MMA) fp16 kernels
def test_released_buffers_small_and_large_come_back_from_the_cache(gpu):
    """A released block goes to the per-device cache (small ones in 512-byte classes) and the
    next buffer of that class takes it from there; gonngpu_trim_cache empties the cache."""
    import gc
    g = gpu
    gc.collect()
    g.lib().gonngpu_trim_cache()
    assert g.stats()["cached_bytes"] == 0
    for nbytes, cls in ((40, 512), (4000, 4096), (4096, 4096), (3 << 20, 3 << 20)):
        a = g.Buffer.empty(nbytes)
        held = g.stats()["hbm_bytes"]
        a.release()
        assert g.stats()["cached_bytes"] == cls and g.stats()["hbm_bytes"] == held - nbytes
        b = g.Buffer.empty(cls - 1 if cls <= 4096 else cls)      # same class: served from the cache
        assert g.stats()["cached_bytes"] == 0
        b.release()
        assert g.lib().gonngpu_trim_cache() == cls and g.stats()["cached_bytes"] == 0


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 256, 256), (1024, 512, 512), (600, 400, 136),
                                   (130, 300, 200), (257, 129, 65), (2048, 2048, 1024)])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_fp16_cta_pair_kernels(gpu, mode, shape, layout):
    """The 256-row (mode 1) and 512-row (mode 2) pair kernels, forced also for
    shapes the size heuristic would give to the single-CTA kernel."""
    m, n, k = shape
    rng = np.random.default_rng(m * 31 + n * 17 + k)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    ta, tb = layout[0] == "t", layout[1] == "t"
    As = np.ascontiguousarray(A.T) if ta else A
    Bs = np.ascontiguousarray(B.T) if tb else B
    try:
        assert gpu.lib().gonngpu_set_gemm_pair_mode(mode) == 0
        C = run_matmul(gpu, As, Bs, ta, tb, precision=gpu.FP16_RN)
    finally:
        gpu.lib().gonngpu_set_gemm_pair_mode(-1)
    assert oracle.rel_frobenius(C, oracle.gemm_f64(oracle.f16_rn(As), oracle.f16_rn(Bs), ta, tb)) <= 2e-5


@pytest.mark.parametrize("mode", [1, 2])
def test_fp16_cta_pair_persistent_loop_and_epilogue(gpu, mode):
    rng = np.random.default_rng(77 + mode)
    A = rng.integers(-3, 4, (4096, 320)).astype(np.float32)
    B = rng.integers(-3, 4, (320, 1024)).astype(np.float32)
    bias = rng.integers(-5, 6, 1024).astype(np.float32)
    C0 = rng.integers(-3, 4, (4096, 1024)).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    try:
        gpu.lib().gonngpu_set_gemm_pair_mode(mode)
        gpu.lib().gonngpu_set_gemm_tuning(0, 6)       # 3 pairs walk 32 or 64 tiles: accumulator ring, stage ring
        assert np.array_equal(run_matmul(gpu, A, B, precision=gpu.FP16_RN), ref.astype(np.float32))
        gpu.lib().gonngpu_set_gemm_tuning(0, 0)
        got = run_matmul(gpu, A, B, precision=gpu.FP16_RN, bias=bias, act=0)
        assert np.array_equal(got, np.maximum(ref + bias, 0).astype(np.float32))
        got = run_matmul(gpu, A, B, precision=gpu.FP16_RN, alpha=0.5, beta=2.0, C0=C0.copy())
        assert np.array_equal(got, (0.5 * ref + 2.0 * C0).astype(np.float32))
    finally:
        gpu.lib().gonngpu_set_gemm_tuning(0, 0)
        gpu.lib().gonngpu_set_gemm_pair_mode(-1)


def test_streamed_matmul_from_pinned_host_memory(gpu):
    """A large product whose A and C live in page-locked host memory takes the
    streamed path (upload, multiply and write-back overlapped in row blocks);
    the host copy of C is current on return and the device copies stay valid."""
    m, k, n = 20000, 256, 512                     # ragged last block (20000 = 4*4096 + 3616)
    rng = np.random.default_rng(5)
    hA, pA = gpu.pinned_array((m, k))
    hC, pC = gpu.pinned_array((m, n))
    hA[:] = (rng.standard_normal((m, k)) / 16).astype(np.float32)
    B = (rng.standard_normal((k, n)) / 16).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    hC[:] = -5.0
    a, b, c, bb = gpu.Buffer.from_host(hA), gpu.Buffer.from_host(B), gpu.Buffer.from_host(hC), gpu.Buffer.from_host(bias)
    before = gpu.stats()
    gpu.matmul_ex(a, (m, k), False, b, (k, n), False, c, (m, n), precision=gpu.FP16_RN, bias=bb, act=0)
    after = gpu.stats()
    ref = np.maximum(oracle.gemm_f64(oracle.f16_rn(hA), oracle.f16_rn(B)) + bias, 0)
    assert oracle.rel_frobenius(hC, ref) <= 2e-5            # written back without a retrieve call
    assert after["gemm_launches"] - before["gemm_launches"] == 5   # five row blocks of 4096
    assert after["d2h_bytes"] - before["d2h_bytes"] == m * n * 4
    c.retrieve_into(hC)                                      # nothing left to copy
    assert gpu.stats()["d2h_bytes"] == after["d2h_bytes"]
    other = c.retrieve((m, n))                               # a different destination still copies
    assert np.array_equal(other, hC)
    # the device copies are valid: reuse A (cached plane) and C (as an input) in ordinary calls
    c2 = gpu.Buffer.empty(m * n * 4)
    gpu.matmul_ex(a, (m, k), False, b, (k, n), False, c2, (m, n), precision=gpu.FP16_RN, bias=bb, act=0)
    assert np.array_equal(c2.retrieve((m, n)), hC)
    t = gpu.Buffer.empty(m * n * 4)
    gpu.transpose(c, (m, n), t)
    assert np.array_equal(t.retrieve((n, m)), hC.T)
    for x in (a, b, c, bb, c2, t):
        x.release()
    gpu.lib().gonngpu_host_free(pA)
    gpu.lib().gonngpu_host_free(pC)


@pytest.mark.parametrize("shape", [(256, 256, 32), (512, 256, 200), (600, 400, 136), (130, 300, 2000),
                                   (257, 129, 65), (2048, 1024, 4096)])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_fp32_cta_pair_kernel(gpu, shape, layout):
    """The fp32-accurate (3xTF32, chunk-promoted) kernel on CTA pairs, forced for
    every shape; K up to 4096 to show that the error does not grow with K."""
    m, n, k = shape
    rng = np.random.default_rng(m * 13 + n * 7 + k)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    ta, tb = layout[0] == "t", layout[1] == "t"
    As = np.ascontiguousarray(A.T) if ta else A
    Bs = np.ascontiguousarray(B.T) if tb else B
    try:
        assert gpu.lib().gonngpu_set_gemm_pair_mode(1) == 0
        C = run_matmul(gpu, As, Bs, ta, tb, precision=gpu.FP32_3XTF32)
    finally:
        gpu.lib().gonngpu_set_gemm_pair_mode(-1)
    assert oracle.rel_frobenius(C, oracle.gemm_f64(As, Bs, ta, tb)) <= 2e-6


@pytest.mark.parametrize("layout", ["nn", "tn", "nt", "tt"])
def test_fp32_cta_pair_kernel_wide_dynamic_range_and_chosen_by_size(gpu, layout):
    """The CTA-pair kernel takes its correction terms from bf16 planes: elements spread over
    twelve decades (bf16 keeps fp32's exponent range), ragged sizes, and a shape large enough
    that the library picks the kernel itself."""
    m, n, k = 2311, 2377, 805
    rng = np.random.default_rng(77 + len(layout) + ord(layout[0]) * 3 + ord(layout[1]))
    A = (rng.standard_normal((m, k)) * 10.0 ** rng.integers(-6, 7, (m, k))).astype(np.float32)
    B = (rng.standard_normal((k, n)) * 10.0 ** rng.integers(-6, 7, (k, n))).astype(np.float32)
    ta, tb = layout[0] == "t", layout[1] == "t"
    As = np.ascontiguousarray(A.T) if ta else A
    Bs = np.ascontiguousarray(B.T) if tb else B
    C = run_matmul(gpu, As, Bs, ta, tb, precision=gpu.FP32_3XTF32)   # 100 pair tiles: chosen by size
    assert oracle.rel_frobenius(C, oracle.gemm_f64(As, Bs, ta, tb)) <= 2e-6


def test_fp32_cta_pair_kernel_persistent_loop_and_epilogue(gpu):
    rng = np.random.default_rng(91)
    A = rng.integers(-3, 4, (2048, 160)).astype(np.float32)
    B = rng.integers(-3, 4, (160, 768)).astype(np.float32)
    bias = rng.integers(-5, 6, 768).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    try:
        gpu.lib().gonngpu_set_gemm_pair_mode(1)
        gpu.lib().gonngpu_set_gemm_tuning(0, 4)      # 2 pairs walk 24 tiles
        assert np.array_equal(run_matmul(gpu, A, B), ref.astype(np.float32))
        gpu.lib().gonngpu_set_gemm_tuning(0, 0)
        assert np.array_equal(run_matmul(gpu, A, B, bias=bias, act=0), np.maximum(ref + bias, 0).astype(np.float32))
    finally:
        gpu.lib().gonngpu_set_gemm_tuning(0, 0)
        gpu.lib().gonngpu_set_gemm_pair_mode(-1)


# ------------------------------------------------------------------ fused linear backward
# the last two: both products on the CTA-pair kernel; dW on it and dX (small batch) not
@pytest.mark.parametrize("shape", [(1, 1, 1), (33, 70, 10), (130, 257, 99), (512, 784, 1024),
                                   (2560, 2304, 2400), (200, 2304, 2400)])
@pytest.mark.parametrize("masked", [False, True])
def test_linear_backward_matches_unfused_oracle(gpu, shape, masked):
    """dW, dX, db of a linear layer in one call against the reference's unfused
    chain (ReLU backward, Transpose + MatMul twice, column sums) done by the oracle."""
    batch, fin, fout = shape
    rng = np.random.default_rng(batch * 3 + fin * 5 + fout * 7 + masked)
    X = rng.uniform(0, 1, (batch, fin)).astype(np.float32)
    W = (rng.standard_normal((fin, fout)) * np.sqrt(2.0 / fin)).astype(np.float32)
    dY = (rng.standard_normal((batch, fout)) * 1e-2).astype(np.float32)
    act = np.maximum(rng.standard_normal((batch, fout)), 0).astype(np.float32) if masked else None
    dAct = oracle.relu_backward(dY, act) if masked else dY
    x, w, dy = gpu.Buffer.from_host(X), gpu.Buffer.from_host(W), gpu.Buffer.from_host(dY)
    a = gpu.Buffer.from_host(act) if masked else None
    dx, dw, db = gpu.Buffer.empty(X.nbytes), gpu.Buffer.empty(W.nbytes), gpu.Buffer.empty(fout * 4)
    gpu.linear_backward(x, w, dy, a, batch, fin, fout, dx=dx, dw=dw, db=db)
    assert oracle.rel_frobenius(dw.retrieve(W.shape), oracle.gemm_f64(X, dAct, True, False)) <= FP32_TOL
    assert oracle.rel_frobenius(dx.retrieve(X.shape), oracle.gemm_f64(dAct, W, False, True)) <= FP32_TOL
    ref_db = dAct.astype(np.float64).sum(axis=0)
    assert np.allclose(db.retrieve((fout,)), ref_db, rtol=1e-5, atol=1e-6 * max(1.0, np.abs(ref_db).max()))
    # partial requests
    dw2 = gpu.Buffer.empty(W.nbytes)
    gpu.linear_backward(x, None, dy, a, batch, fin, fout, dw=dw2)
    assert np.array_equal(dw2.retrieve(W.shape), dw.retrieve(W.shape))
    with pytest.raises(gpu.GonnError) as e:
        gpu.linear_backward(None, w, dy, a, batch, fin, fout, dw=dw2)   # dW needs X
    assert e.value.code == -2


def test_config3_training_step_with_fused_calls(gpu):
    """The MLP step of configuration 3 as 3 fused forward calls and 3 fused
    backward calls (the ReLU mask of the hidden layers applied inside)."""
    X, Ws, bs, dYs = oracle.config3()
    acts = [X]
    for layer in range(3):
        acts.append(run_matmul(gpu, acts[-1], Ws[layer], bias=bs[layer], act=0 if layer < 2 else -1))
    grad = dYs[2]                                   # gradient arriving at the output layer
    for layer in (2, 1, 0):
        h_in, W = acts[layer], Ws[layer]
        mask = acts[layer + 1] if layer < 2 else None
        x, w, dy = gpu.Buffer.from_host(h_in), gpu.Buffer.from_host(W), gpu.Buffer.from_host(grad)
        m = gpu.Buffer.from_host(mask) if mask is not None else None
        dx, dw, db = gpu.Buffer.empty(h_in.nbytes), gpu.Buffer.empty(W.nbytes), gpu.Buffer.empty(W.shape[1] * 4)
        gpu.linear_backward(x, w, dy, m, h_in.shape[0], W.shape[0], W.shape[1], dx=dx, dw=dw, db=db)
        dAct = oracle.relu_backward(grad, mask) if mask is not None else grad
        assert oracle.rel_frobenius(dw.retrieve(W.shape), oracle.gemm_f64(h_in, dAct, True, False)) <= FP32_TOL
        got_dx = dx.retrieve(h_in.shape)
        assert oracle.rel_frobenius(got_dx, oracle.gemm_f64(dAct, W, False, True)) <= FP32_TOL
        grad = got_dx


# ------------------------------------------------------------------ batched product
@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (3, 5, 7, 9), (4, 128, 64, 32), (5, 130, 70, 33),
                                   (16, 200, 96, 100), (64, 64, 64, 64), (2, 512, 1024, 784)])
def test_batch_matmul_matches_per_batch_oracle(gpu, shape):
    batch, m, n, k = shape
    rng = np.random.default_rng(batch * 11 + m * 7 + n * 3 + k)
    A = rng.standard_normal((batch, m, k)).astype(np.float32)
    B = rng.standard_normal((batch, k, n)).astype(np.float32)
    # a poisoned batch must not leak into its neighbours (k blocks never straddle batches)
    if batch > 2:
        B[1] = np.float32("inf")
    a, b = gpu.Buffer.from_host(A), gpu.Buffer.from_host(B)
    c = gpu.Buffer.from_host(np.full((batch, m, n), np.float32(-9.0)))
    gpu.batch_matmul(a, b, c, batch, m, n, k)
    C = c.retrieve((batch, m, n))
    for i in range(batch):
        if batch > 2 and i == 1:
            continue
        assert oracle.rel_frobenius(C[i], oracle.gemm_f64(A[i], B[i])) <= FP32_TOL, i
    with pytest.raises(gpu.GonnError) as e:
        gpu.batch_matmul(a, b, c, batch + 1, m, n, k)
    assert e.value.code == -3


# ------------------------------------------------------------------ element-wise family
@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (37, 101), (512, 1024), (1000, 1001)])
def test_elementwise_ops_are_bit_exact(gpu, shape):
    rng = np.random.default_rng(shape[0] * 7 + shape[1])
    A = rng.standard_normal(shape).astype(np.float32)
    B = (rng.standard_normal(shape) + np.float32(3.0)).astype(np.float32)
    B[B == 0] = 1.0
    a, b, c = gpu.Buffer.from_host(A), gpu.Buffer.from_host(B), gpu.Buffer.empty(A.nbytes)
    for op, name in enumerate(["add", "subtract", "element_multiply", "element_divide"]):
        gpu.elementwise(name, a, b, c, shape)
        rc, ref, _ = oracle.elementwise(op, A, B)
        assert rc == 0
        assert np.array_equal(c.retrieve(shape).view(np.uint32), ref.reshape(shape).view(np.uint32)), name
    for mult, name in ((False, "scalar_add"), (True, "scalar_multiply")):
        gpu.scalar_op(name, a, shape, 1.375, c)
        assert np.array_equal(c.retrieve(shape), oracle.scalar_op(mult, A, 1.375).reshape(shape))
    with pytest.raises(gpu.GonnError) as e:
        lib = gpu.lib()
        err = gpu.CError()
        rc = lib.perform_mps_matrix_add(a.handle, shape[0], shape[1], b.handle, shape[0], shape[1] + 1, c.handle,
                                        shape[0], shape[1], None, ctypes.byref(err))
        gpu._check(rc, err)
    assert e.value.code == -2 and "same dimensions" in e.value.message


def test_divide_stops_at_first_zero_like_the_reference(gpu):
    rng = np.random.default_rng(8)
    n = 5000
    A = rng.standard_normal((1, n)).astype(np.float32)
    B = (rng.standard_normal((1, n)) + np.float32(4.0)).astype(np.float32)
    B[0, 1234] = 0.0
    B[0, 4000] = -0.0
    prev = np.full((1, n), 7.0, np.float32)
    a, b, c = gpu.Buffer.from_host(A), gpu.Buffer.from_host(B), gpu.Buffer.from_host(prev)
    with pytest.raises(gpu.GonnError) as e:
        gpu.elementwise("element_divide", a, b, c, (1, n))
    assert e.value.code == -4 and "Division by zero encountered at element 1234" in e.value.message
    rc, ref, z = oracle.elementwise(3, A, B, out=prev)
    assert rc == -4 and z == 1234
    assert np.array_equal(c.retrieve((1, n)).view(np.uint32), ref.reshape(1, n).view(np.uint32))


def test_activation_family_matches_oracle(gpu, golden):
    ref, _ = golden
    rng = np.random.default_rng(9)
    x = np.concatenate([rng.standard_normal(4093) * 3, [-1e30, -100.0, 0.0, -0.0, 100.0, 1e30]]).astype(np.float32)
    go = rng.standard_normal(x.size).astype(np.float32)
    xi, gi = gpu.Buffer.from_host(x), gpu.Buffer.from_host(go)
    out, gin = gpu.Buffer.empty(x.nbytes), gpu.Buffer.empty(x.nbytes)
    for kind, name, alpha in ((0, "sigmoid", None), (1, "tanh", None), (2, "leaky_relu", 0.1)):
        gpu.activation_forward(name, xi, x.size, out, alpha)
        y = out.retrieve(x.shape)
        y_ref = oracle.activation_forward(kind, x, alpha or 0.0)
        assert np.allclose(y, y_ref, rtol=2e-6, atol=1e-7), name     # expf / tanhf differ by an ulp or two
        gpu.activation_backward(name, gi, out, x.size, gin, alpha)
        assert np.allclose(gin.retrieve(x.shape), oracle.activation_backward(kind, go, y, alpha or 0.0),
                           rtol=2e-6, atol=1e-7), name
    # the reference's own vectors
    k = ref["leaky_relu_forward"]
    v = np.array(k["input"], np.float32)
    vi, vo = gpu.Buffer.from_host(v), gpu.Buffer.empty(v.nbytes)
    gpu.activation_forward("leaky_relu", vi, v.size, vo, k["alpha"])
    assert np.allclose(vo.retrieve(v.shape), k["expected"], atol=1e-6)
    gpu.activation_forward("sigmoid", vi, v.size, vo)
    assert abs(vo.retrieve(v.shape)[2] - 0.5) <= 1e-6
    gpu.activation_forward("tanh", vi, v.size, vo)
    assert abs(vo.retrieve(v.shape)[2]) <= 1e-6


def test_elu_swish_gelu_match_oracle(gpu, golden):
    ref, _ = golden
    rng = np.random.default_rng(10)
    x = np.concatenate([rng.standard_normal(8190) * 3, [-1e30, -100.0, 0.0, -0.0, 100.0, 1e30]]).astype(np.float32)
    go = rng.standard_normal(x.size).astype(np.float32)
    xi, gi = gpu.Buffer.from_host(x), gpu.Buffer.from_host(go)
    out, gin = gpu.Buffer.empty(x.nbytes), gpu.Buffer.empty(x.nbytes)
    for kind, name, alpha in ((3, "elu", 0.7), (4, "swish", None), (5, "gelu", None)):
        gpu.activation_forward(name, xi, x.size, out, alpha)
        y = out.retrieve(x.shape)
        assert np.allclose(y, oracle.activation_forward(kind, x, alpha or 0.0), rtol=3e-6, atol=1e-6), name
        # the backward form is a function of the activation OUTPUT: feed both sides the same one
        gpu.activation_backward(name, gi, out, x.size, gin, alpha)
        want = oracle.activation_backward(kind, go, y, alpha or 0.0)
        got = gin.retrieve(x.shape)
        ok = np.isfinite(want)
        # Newton on a flat stretch amplifies an ulp of expf/tanhf: tolerance 1e-4 of the gradient scale
        assert np.allclose(got[ok], want[ok], rtol=1e-4, atol=1e-4), name
        assert np.array_equal(np.isfinite(got), ok), name
    for key, name, alpha in (("elu_forward", "elu", 1.0), ("swish_forward", "swish", None), ("gelu_forward", "gelu", None)):
        k = ref[key]
        v = np.array(k["input"], np.float32)
        vi, vo = gpu.Buffer.from_host(v), gpu.Buffer.empty(v.nbytes)
        gpu.activation_forward(name, vi, v.size, vo, alpha)
        r = vo.retrieve(v.shape)
        if "index_of_zero" in k:
            assert abs(r[k["index_of_zero"]]) <= 1e-6
        else:
            assert abs(r[k["index_of_one"]] - 1.0) <= 1e-6 and r[0] < 0 and r[1] < 0


@pytest.mark.parametrize("shape", [(1, 4), (2, 3), (1, 1), (9, 10), (512, 10), (33, 512), (5, 513), (3, 5000),
                                   (1, 100000), (1001, 3), (777, 8), (130, 20), (67, 100), (19, 300), (7, 1000),
                                   (9, 2048), (5, 3000), (3, 4095), (300, 8192), (2, 9000), (2, 9001), (1003, 4), (517, 16),
                                   (99, 28), (50, 128), (21, 260), (11, 512)])
def test_softmax_rows_match_oracle(gpu, golden, shape):
    ref, _ = golden
    rng = np.random.default_rng(shape[0] + shape[1])
    X = (rng.standard_normal(shape) * 4).astype(np.float32)
    if shape == (1, 4):
        X = np.array(ref["softmax_forward"]["input"], np.float32).reshape(shape)
    if shape == (2, 3):
        X = np.array(ref["softmax_2d_forward"]["input"], np.float32).reshape(shape)
    G = rng.standard_normal(shape).astype(np.float32)
    xi, gi = gpu.Buffer.from_host(X), gpu.Buffer.from_host(G)
    out, gin = gpu.Buffer.empty(X.nbytes), gpu.Buffer.empty(X.nbytes)
    gpu.softmax_2d(xi, shape[0], shape[1], out)
    Y = out.retrieve(shape)
    want = oracle.softmax_forward(X)
    # the reference's running float32 sum drifts with the row length; the tree sum here does not
    # (1.9e-4 at 100000 features, measured against float64), so the band widens with the length
    assert np.allclose(Y, want, rtol=1e-5 + 3e-9 * shape[1], atol=1e-9)
    e = np.exp(X.astype(np.float64) - X.max(axis=1, keepdims=True))
    assert np.allclose(Y, e / e.sum(axis=1, keepdims=True), rtol=5e-6, atol=1e-12)
    assert (np.abs(Y.sum(axis=1, dtype=np.float64) - 1.0) <= 1e-6).all() and (Y >= 0).all()
    gpu.softmax_2d_backward(gi, out, shape[0], shape[1], gin)
    # g - dot cancels, and the reference's running float32 dot drifts with the row length
    GI = gin.retrieve(shape)
    assert np.allclose(GI, oracle.softmax_backward(G, Y), rtol=1e-5, atol=1e-6 + 2e-9 * shape[1])
    Y64, G64 = Y.astype(np.float64), G.astype(np.float64)
    assert np.allclose(GI, Y64 * (G64 - (G64 * Y64).sum(axis=1, keepdims=True)), rtol=1e-5, atol=3e-7)
    if shape[0] == 1:
        gpu.activation_forward("softmax_1d", xi, shape[1], out)
        assert np.array_equal(out.retrieve(shape), Y)
        gpu.activation_backward("softmax_1d", gi, out, shape[1], gin)
        assert np.array_equal(gin.retrieve(shape), GI)


# ------------------------------------------------------------------ float64 facade data
@pytest.mark.parametrize("n", [0, 1, 3, 4, 1023, 4097, 1 << 20])
def test_float64_upload_and_retrieve_are_bit_exact(gpu, n):
    rng = np.random.default_rng(n + 17)
    x = rng.standard_normal(n) * 10.0 ** rng.integers(-30, 30, n)
    if n >= 1023:
        x[:8] = [0.0, -0.0, np.inf, -np.inf, 1e39, -1e39, 1e-46, np.float64(np.float32(1.0)) + 2.0 ** -24]
        x[8] = np.nan
    buf = gpu.Buffer.empty(max(n, 1) * 4)
    buf.upload_f64(x)
    want = x.astype(np.float32)                    # IEEE round-to-nearest-even, like Go's float32(v)
    got = buf.retrieve((n,))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    back = buf.retrieve_f64((n,))
    assert np.array_equal(back.view(np.uint64), want.astype(np.float64).view(np.uint64))
    # a partial upload keeps the tail
    if n >= 4:
        buf.upload_f64(np.full(n // 2, 2.5))
        got = buf.retrieve((n,))
        assert (got[: n // 2] == 2.5).all() and np.array_equal(got[n // 2:].view(np.uint32), want[n // 2:].view(np.uint32))
    with pytest.raises(gpu.GonnError) as e:
        buf.upload_f64(np.zeros(max(n, 1) + 1))
    assert e.value.code == -2


def test_float64_facade_feeds_the_gemm(gpu):
    rng = np.random.default_rng(23)
    A, B = rng.standard_normal((300, 200)), rng.standard_normal((200, 150))
    a, b, c = gpu.Buffer.empty(A.size * 4), gpu.Buffer.empty(B.size * 4), gpu.Buffer.empty(300 * 150 * 4)
    a.upload_f64(A)
    b.upload_f64(B)
    gpu.matmul(a, A.shape, b, B.shape, c, (300, 150))
    C = c.retrieve_f64((300, 150))
    ref = oracle.gemm_f64(A.astype(np.float32), B.astype(np.float32))
    assert C.dtype == np.float64 and oracle.rel_frobenius(C, ref) <= FP32_TOL


# ------------------------------------------------------------------ split-K (fp32, few tiles)
@pytest.mark.parametrize("shape", [(128, 128, 1024), (512, 1024, 784), (1024, 1024, 1024), (300, 200, 2000),
                                   (64, 10, 4096), (257, 129, 520)])
@pytest.mark.parametrize("splits", [2, 3, 4, 8])
def test_split_k_matches_float64_reference_and_is_deterministic(gpu, shape, splits):
    m, n, k = shape
    rng = np.random.default_rng(m + 3 * n + 7 * k + splits)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    C0 = rng.standard_normal((m, n)).astype(np.float32)
    ref = np.maximum(0.5 * oracle.gemm_f64(A, B) + 0.25 * C0 + bias, 0)
    L = gpu.lib()
    try:
        assert L.gonngpu_set_gemm_pair_mode(0) == 0          # keep the product on the single-CTA kernel
        assert L.gonngpu_set_gemm_split_k(splits) == 0
        kw = dict(precision=gpu.FP32_3XTF32, alpha=0.5, beta=0.25, C0=C0, bias=bias, act=0)
        first = run_matmul(gpu, A, B, **kw)
        again = run_matmul(gpu, A, B, **kw)
        assert oracle.rel_frobenius(first, ref) <= FP32_TOL
        assert np.array_equal(first.view(np.uint32), again.view(np.uint32))
        # transposed storage takes the same route
        got = run_matmul(gpu, np.ascontiguousarray(A.T), np.ascontiguousarray(B.T), True, True, **kw)
        assert oracle.rel_frobenius(got, ref) <= FP32_TOL
        # the counters are back at zero: an unsplit product and another split one follow cleanly
        assert L.gonngpu_set_gemm_split_k(1) == 0
        plain = run_matmul(gpu, A, B, **kw)
        assert oracle.rel_frobenius(plain, ref) <= FP32_TOL
        assert L.gonngpu_set_gemm_split_k(0) == 0            # chosen by size
        auto = run_matmul(gpu, A, B, **kw)
        assert oracle.rel_frobenius(auto, ref) <= FP32_TOL
    finally:
        L.gonngpu_set_gemm_split_k(0)
        L.gonngpu_set_gemm_pair_mode(-1)


def test_split_k_with_more_units_than_sms_and_in_batches(gpu):
    rng = np.random.default_rng(77)
    L = gpu.lib()
    try:
        assert L.gonngpu_set_gemm_pair_mode(0) == 0
        assert L.gonngpu_set_gemm_split_k(4) == 0
        A = rng.standard_normal((1500, 600)).astype(np.float32)     # 12 x 5 tiles x 4 splits > 148 CTAs
        B = rng.standard_normal((600, 600)).astype(np.float32)
        assert oracle.rel_frobenius(run_matmul(gpu, A, B, precision=gpu.FP32_3XTF32), oracle.gemm_f64(A, B)) <= FP32_TOL
        nb, bm, bk, bn = 5, 70, 400, 90
        bA = rng.standard_normal((nb, bm, bk)).astype(np.float32)
        bB = rng.standard_normal((nb, bk, bn)).astype(np.float32)
        a, b, c = gpu.Buffer.from_host(bA), gpu.Buffer.from_host(bB), gpu.Buffer.empty(nb * bm * bn * 4)
        gpu.batch_matmul(a, b, c, nb, bm, bn, bk)
        got = c.retrieve((nb, bm, bn))
        for i in range(nb):
            assert oracle.rel_frobenius(got[i], oracle.gemm_f64(bA[i], bB[i])) <= FP32_TOL
    finally:
        L.gonngpu_set_gemm_split_k(0)
        L.gonngpu_set_gemm_pair_mode(-1)


# ------------------------------------------------------------------ seeded random sweep
def test_random_shapes_layouts_and_epilogues(gpu):
    """120 seeded random products (ragged sizes, all four layouts, both precisions, random
    alpha / beta / bias / activation) against the float64 oracle: the tile chooser, split-K,
    3-D operand boxes and both epilogue store paths all get hit by the mix."""
    rng = np.random.default_rng(2024)
    acts = [-1, 0, 1, 2, 3, 4]
    bad = []
    for case in range(120):
        m = int(rng.integers(1, 700))
        n = int(rng.integers(1, 700))
        k = int(rng.integers(1, 1500)) if case % 3 else int(rng.integers(1, 5000))
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        prec = gpu.FP32_3XTF32 if case % 2 else gpu.FP16_RN
        A = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
        B = rng.standard_normal((k, n)).astype(np.float32)
        alpha = float(rng.choice([1.0, 0.5, -2.0]))
        beta = float(rng.choice([0.0, 0.0, 0.75]))
        bias = rng.standard_normal(n).astype(np.float32) if rng.integers(0, 2) else None
        act = int(rng.choice(acts))
        C0 = rng.standard_normal((m, n)).astype(np.float32)
        As = np.ascontiguousarray(A.T) if ta else A
        Bs = np.ascontiguousarray(B.T) if tb else B
        got = run_matmul(gpu, As, Bs, ta, tb, precision=prec, alpha=alpha, beta=beta, C0=C0, bias=bias,
                         act=act, act_param=0.1)
        Ar, Br = (oracle.f16_rn(A), oracle.f16_rn(B)) if prec == gpu.FP16_RN else (A, B)
        z = alpha * oracle.gemm_f64(Ar, Br) + beta * C0.astype(np.float64)
        if bias is not None:
            z = z + bias
        ref = oracle.apply_act_f64(z, act, 0.1)
        tol = 3e-5 if prec == gpu.FP16_RN else FP32_TOL   # fp16: fp32 accumulation error only
        err = oracle.rel_frobenius(got, ref)
        if not err <= tol:
            bad.append((case, m, n, k, ta, tb, prec, alpha, beta, bias is not None, act, err))
    assert not bad, bad[:5]


@pytest.mark.parametrize("shape", [(1, 1), (7, 5), (127, 33), (128, 64), (512, 1024), (513, 10), (5000, 100),
                                   (70000, 40), (300, 5000)])
def test_column_sum_shapes_and_determinism(gpu, shape):
    """Bias gradient: one row chunk or several (partials through the workspace), integer data exact,
    random data within float32 summation error of float64, and the same bits on every run."""
    rows, cols = shape
    rng = np.random.default_rng(rows * 31 + cols)
    Xi = rng.integers(-8, 9, shape).astype(np.float32)
    x, o = gpu.Buffer.from_host(Xi), gpu.Buffer.empty(cols * 4)
    gpu.column_sum(x, rows, cols, o)
    assert np.array_equal(o.retrieve((cols,)), Xi.sum(axis=0, dtype=np.float64).astype(np.float32))
    X = rng.standard_normal(shape).astype(np.float32)
    x.upload(X)
    gpu.column_sum(x, rows, cols, o)
    first = o.retrieve((cols,))
    ref = X.sum(axis=0, dtype=np.float64)
    assert np.allclose(first, ref, rtol=1e-5, atol=1e-5 * np.sqrt(rows))
    gpu.column_sum(x, rows, cols, o)
    assert np.array_equal(first.view(np.uint32), o.retrieve((cols,)).view(np.uint32))
    # a split fp32 product right after it finds the shared counters at zero
    A = rng.standard_normal((128, 1024)).astype(np.float32)
    B = rng.standard_normal((1024, 128)).astype(np.float32)
    assert oracle.rel_frobenius(run_matmul(gpu, A, B, precision=gpu.FP32_3XTF32), oracle.gemm_f64(A, B)) <= FP32_TOL
