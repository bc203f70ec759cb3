"""The allocation-free MatMul entry point (gonngpu_matmul_f16_static_scratch).

It serves callers that cannot call cudaMalloc while they compute - a process
that reserved all of HBM for its own arena, or a latency-critical loop - by
keeping the fp16 operand planes in a fixed array inside the library.  The test
drives it through the C ABI twice in a row (the second call reuses the array
with other shapes, so stale contents would show) and compares each result with
the ordinary allocating entry point on the same inputs and with the float64
oracle; the device's free memory, as the driver reports it, must not shrink
across the two calls (after one warm-up call, which is when CUDA loads the
kernels).  This file sorts last so that a failure here cannot hide the other
tests' results.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_bytes():
    """Free device memory as the driver reports it (cudaMemGetInfo)."""
    try:
        from cuda.bindings import runtime as rt
    except ImportError:
        from cuda import cudart as rt
    err, free, _total = rt.cudaMemGetInfo()
    assert int(err) == 0, err
    return int(free)


def _ordinary(gpu, A, B):
    a, b = gpu.Buffer.from_host(A), gpu.Buffer.from_host(B)
    c = gpu.Buffer.empty(A.shape[0] * B.shape[1] * 4)
    gpu.matmul_ex(a, A.shape, False, b, B.shape, False, c, (A.shape[0], B.shape[1]), precision=gpu.FP16_RN)
    out = c.retrieve((A.shape[0], B.shape[1]))
    for x in (a, b, c):
        x.release()
    return out


def test_static_scratch_matmul_matches_allocating_entry_twice(gpu):
    from oracle import oracle
    rng = np.random.default_rng(99)
    # inputs and outputs are allocated up front, outside the calls under test
    shapes = [((700, 520), (520, 900)), ((129, 65), (65, 257))]
    bufs = []
    for (sa, sb) in shapes:
        A = (rng.standard_normal(sa) / np.sqrt(sa[1])).astype(np.float32)
        B = (rng.standard_normal(sb) / np.sqrt(sa[1])).astype(np.float32)
        a, b = gpu.Buffer.from_host(A), gpu.Buffer.from_host(B)
        c = gpu.Buffer.empty(sa[0] * sb[1] * 4)
        bufs.append((A, B, a, b, c, a.device_address(), b.device_address(), c.device_address()))
    # the warm-up a caller makes once per device (set-up; CUDA loads each kernel at its first use)
    for (A, B, a, b, c, pa, pb, pc) in bufs:
        gpu.matmul_f16_static_scratch(pa, A.shape, pb, B.shape, pc)
        c.upload(np.zeros((A.shape[0], B.shape[1]), np.float32))   # the checked results come from the calls below
    import gc
    gc.collect()                                       # buffers of earlier tests are released now, not mid-measurement
    hbm_before = gpu.stats()["hbm_bytes"]
    free_before = _free_bytes()
    for (A, B, a, b, c, pa, pb, pc) in bufs:           # two calls in a row
        gpu.matmul_f16_static_scratch(pa, A.shape, pb, B.shape, pc)
    assert _free_bytes() >= free_before                # nothing was taken from the device
    assert gpu.stats()["hbm_bytes"] == hbm_before      # nor through the library's own allocator
    for (A, B, a, b, c, *_) in bufs:
        C = c.retrieve((A.shape[0], B.shape[1]))
        ref = _ordinary(gpu, A, B)
        err = np.linalg.norm(C.astype(np.float64) - ref) / np.linalg.norm(ref.astype(np.float64))
        assert err <= 2e-5, err                         # against the existing entry point
        exact = oracle.gemm_f64(A.astype(np.float16).astype(np.float32), B.astype(np.float16).astype(np.float32))
        assert oracle.rel_frobenius(C, exact) <= 1e-2   # fp16-path tolerance against the oracle
        assert oracle.rel_frobenius(C, exact) <= 1e-5   # (fp32 accumulation of exact fp16 products)
    for (_, _, a, b, c, *_) in bufs:
        for x in (a, b, c):
            x.release()


def test_static_scratch_refuses_oversized_operands(gpu):
    a = gpu.Buffer.empty(16)
    p = a.device_address()
    with pytest.raises(gpu.GonnError) as e:
        gpu.matmul_f16_static_scratch(p, (8192, 8192), p, (8192, 8192), p)
    assert e.value.code == -3 and "built-in scratch holds" in e.value.message
    with pytest.raises(gpu.GonnError) as e:
        gpu.matmul_f16_static_scratch(p, (4, 5), p, (6, 4), p)
    assert e.value.code == -3
    a.release()
