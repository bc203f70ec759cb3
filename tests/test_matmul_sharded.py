"""gonngpu_matmul_sharded: the row-sharded MatMul as one call with host matrices.

On a one-GPU box the call runs with one device (plan, streaming in row blocks,
write-back into the caller's C); with more GPUs visible it is run over all of
them and over two, and every variant is compared with the float64 oracle on the
fp16-rounded inputs.  Argument errors answer without touching a GPU."""
import numpy as np
import pytest


def _inputs(g, m, k, n, pinned, seed=31):
    rng = np.random.default_rng(seed)
    A = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
    B = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    if not pinned:
        return A, B, np.zeros((m, n), np.float32), []
    hA, pA = g.pinned_array((m, k))
    hB, pB = g.pinned_array((k, n))
    hC, pC = g.pinned_array((m, n))
    hA[...] = A
    hB[...] = B
    return hA, hB, hC, [pA, pB, pC]


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n,pinned,precision", [(9000, 300, 520, True, "rn"), (9000, 300, 520, False, "rn"),
                                                    (700, 64, 8, True, "trunc"), (20000, 1024, 1024, True, "rn")])
def test_sharded_matmul_from_host_memory(gpu, m, k, n, pinned, precision):
    from oracle import oracle
    g = gpu
    g.lib().gonngpu_set_blocking(1)
    A, B, C, pins = _inputs(g, m, k, n, pinned)
    prec = g.FP16_RN if precision == "rn" else g.FP16_TRUNC
    rnd = oracle.f16_rn if precision == "rn" else oracle.f16_trunc
    ref = oracle.gemm_f64(rnd(np.asarray(A)), rnd(np.asarray(B)))
    visible = g.lib().gonngpu_device_count()
    for n_dev in sorted({1, min(2, visible), visible}):
        C[...] = -1.0
        g.matmul_sharded(A, B, C, precision=prec, n_devices=n_dev)
        assert oracle.rel_frobenius(np.asarray(C), ref) <= 1e-2, n_dev      # fp16-path tolerance
        assert oracle.rel_frobenius(np.asarray(C), ref) <= 1e-5, n_dev      # exact fp16 products, fp32 sums
        # every row was written, the first and last row of every shard among them
        for d in range(n_dev):
            lo, hi = g.shard_plan(m, n_dev, d)
            for r in {lo, hi - 1} if hi > lo else set():
                assert oracle.rel_frobenius(np.asarray(C[r:r + 1]), ref[r:r + 1]) <= 1e-4
    # the library's current device is what it was, and ordinary calls still work
    assert g.lib().gonngpu_get_device() == 0
    a, b = g.Buffer.from_host(np.asarray(A[:64])), g.Buffer.from_host(np.asarray(B))
    c = g.Buffer.empty(64 * n * 4)
    g.matmul(a, (64, k), b, (k, n), c, (64, n))
    assert oracle.rel_frobenius(c.retrieve((64, n)), oracle.gemm_f64(np.asarray(A[:64]), np.asarray(B))) <= 1e-5
    for x in (a, b, c):
        x.release()
    for p in pins:
        g.lib().gonngpu_host_free(p)


def test_sharded_matmul_argument_errors(built_lib):
    g = built_lib
    A = np.zeros((4, 6), np.float32)
    B = np.zeros((6, 8), np.float32)
    C = np.zeros((4, 8), np.float32)
    with pytest.raises(g.GonnError) as e:
        g.matmul_sharded(A, np.zeros((5, 8), np.float32), C)
    assert e.value.code == -3 and "incompatible dimensions" in e.value.message
    with pytest.raises(g.GonnError) as e:
        g.matmul_sharded(A, B, C, precision=g.FP32_3XTF32)
    assert e.value.code == -3
    with pytest.raises(g.GonnError) as e:
        g.matmul_sharded(A, B, C, n_devices=1000)
    assert e.value.code == -1 and "devices asked for" in e.value.message
    import ctypes
    err = g.CError()
    assert g.lib().gonngpu_matmul_sharded(None, 4, 6, B.ctypes.data, 6, 8, C.ctypes.data, g.FP16_RN, 1,
                                          ctypes.byref(err)) == -2
    g.lib().free_c_error_message(err.message)
    assert g.shard_plan(131072, 8, 3) == (3 * 16384, 4 * 16384)
    assert g.shard_plan(1000, 3, 1) == (512, 1000) and g.shard_plan(1000, 3, 2) == (1000, 1000)
    with pytest.raises(g.GonnError):
        g.shard_plan(10, 2, 2)
