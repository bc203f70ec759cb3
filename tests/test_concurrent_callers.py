"""Calls from several threads at once, as goroutines of the reference's callers make them
(the reference wraps each call in LockOSThread and shares no lock between them).  Every
thread owns its buffers; the library orders the calls and releases its lock while one of them
waits for the GPU.  Results are checked against the float64 oracle."""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_concurrent_matmuls_transposes_and_retrievals(gpu):
    from oracle import oracle
    g = gpu
    g.lib().gonngpu_set_blocking(1)
    errors = []

    def worker(seed):
        try:
            rng = np.random.default_rng(seed)
            for it in range(12):
                m, k, n = (int(x) for x in rng.integers(40, 400, 3))
                A = rng.standard_normal((m, k)).astype(np.float32)
                B = rng.standard_normal((k, n)).astype(np.float32)
                a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
                c = g.Buffer.empty(m * n * 4)
                if it % 3 == 2:
                    g.matmul_ex(a, A.shape, False, b, B.shape, False, c, (m, n), precision=g.FP16_RN)
                    ref = oracle.gemm_f64(oracle.f16_rn(A), oracle.f16_rn(B))
                else:
                    g.matmul(a, A.shape, b, B.shape, c, (m, n))
                    ref = oracle.gemm_f64(A, B)
                got = c.retrieve((m, n))
                if oracle.rel_frobenius(got, ref) > 1e-5:
                    errors.append((seed, it, "product"))
                t = g.Buffer.empty(A.nbytes)
                g.transpose(a, A.shape, t)
                if not np.array_equal(t.retrieve((k, m)), A.T):
                    errors.append((seed, it, "transpose"))
                for x in (a, b, c, t):
                    x.release()
        except Exception as e:  # noqa: BLE001
            errors.append((seed, repr(e)))

    before = g.stats()["buffers"]
    threads = [threading.Thread(target=worker, args=(100 + i,)) for i in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:5]
    assert g.stats()["buffers"] == before
