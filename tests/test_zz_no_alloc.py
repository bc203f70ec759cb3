"""The allocation-free MatMul entry point (gonngpu_matmul_f16_static_scratch).

It serves callers that cannot call cudaMalloc while they compute - a process
that reserved all of HBM for its own arena, or a latency-critical loop - by
keeping the fp16 operand planes in a fixed array inside the library.  The test
drives it through the C ABI twice in a row (the second call reuses the array
with other shapes, so stale contents would show) and compares each result with
the ordinary allocating entry point on the same inputs.  This file sorts last
so that a failure here cannot hide the other tests' results.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ordinary(gpu, A, B):
    a, b = gpu.Buffer.from_host(A), gpu.Buffer.from_host(B)
    c = gpu.Buffer.empty(A.shape[0] * B.shape[1] * 4)
    gpu.matmul_ex(a, A.shape, False, b, B.shape, False, c, (A.shape[0], B.shape[1]), precision=gpu.FP16_RN)
    out = c.retrieve((A.shape[0], B.shape[1]))
    for x in (a, b, c):
        x.release()
    return out


def test_static_scratch_matmul_matches_allocating_entry_twice(gpu):
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
    hbm_before = gpu.stats()["hbm_bytes"]
    got = []
    for (A, B, a, b, c, pa, pb, pc) in bufs:           # two calls in a row
        gpu.matmul_f16_static_scratch(pa, A.shape, pb, B.shape, pc)
        got.append(c.retrieve((A.shape[0], B.shape[1])))
    assert gpu.stats()["hbm_bytes"] == hbm_before      # the library's allocator was not used
    for (A, B, *_), C in zip(bufs, got):
        ref = _ordinary(gpu, A, B)
        err = np.linalg.norm(C.astype(np.float64) - ref) / np.linalg.norm(ref.astype(np.float64))
        assert err <= 2e-5, err                         # same tolerance as the fp16-path tests
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
