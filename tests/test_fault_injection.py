"""Error paths of the bridge under host-side fault injection (gonngpu_inject_fault).

The injected failure is reported on the host, before the device is asked for
anything: no GPU is made to fault.  Each case checks the documented return
code and message of the entry point that hit it, that the library's
bookkeeping (live buffers, held memory) is what it was, and that the same call
succeeds right afterwards."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _inject(g, kind, nth):
    assert g.lib().gonngpu_inject_fault(kind.encode(), nth) == 0


@pytest.fixture()
def mats():
    rng = np.random.default_rng(41)
    A = rng.standard_normal((200, 96)).astype(np.float32)
    B = rng.standard_normal((96, 136)).astype(np.float32)
    return A, B


def test_unknown_kind_is_refused(gpu):
    assert gpu.lib().gonngpu_inject_fault(b"launch", 1) == -3
    assert gpu.lib().gonngpu_inject_fault(None, 1) == -3
    assert gpu.lib().gonngpu_inject_fault(b"alloc", -1) == -3


def test_allocation_failure_in_create_gpu_buffer(gpu, mats):
    g = gpu
    g.lib().gonngpu_trim_cache()                      # so that the buffer cannot come from the cache
    before = g.stats()
    _inject(g, "alloc", 1)
    with pytest.raises(g.GonnError) as e:
        g.Buffer.from_host(mats[0])
    assert e.value.code == -3 and "Could not allocate" in e.value.message
    after = g.stats()
    assert after["buffers"] == before["buffers"] and after["hbm_bytes"] == before["hbm_bytes"]
    a = g.Buffer.from_host(mats[0])                   # disarmed after it fired
    assert g.stats()["buffers"] == before["buffers"] + 1
    a.release()


def test_upload_failure_in_matmul(gpu, mats):
    from oracle import oracle
    g = gpu
    A, B = mats
    a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
    c = g.Buffer.empty(A.shape[0] * B.shape[1] * 4)
    before = g.stats()
    _inject(g, "h2d", 2)                              # A goes up, B's copy fails
    with pytest.raises(g.GonnError) as e:
        g.matmul(a, A.shape, b, B.shape, c, (A.shape[0], B.shape[1]))
    assert e.value.code == -6 and "host to device copy failed" in e.value.message
    assert g.stats()["buffers"] == before["buffers"]
    g.matmul(a, A.shape, b, B.shape, c, (A.shape[0], B.shape[1]))   # B is uploaded now
    assert oracle.rel_frobenius(c.retrieve((A.shape[0], B.shape[1])), oracle.gemm_f64(A, B)) <= 1e-5
    for x in (a, b, c):
        x.release()


@pytest.mark.parametrize("nth", [1, 2, 3, 4])           # hi / lo plane of A, hi / lo plane of B
def test_operand_plane_allocation_failure_in_matmul(gpu, mats, nth):
    from oracle import oracle
    g = gpu
    A, B = mats
    g.lib().gonngpu_trim_cache()
    before = g.stats()
    a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
    c = g.Buffer.empty(A.shape[0] * B.shape[1] * 4)
    g.lib().gonngpu_trim_cache()
    _inject(g, "alloc", nth)
    with pytest.raises(g.GonnError) as e:
        g.matmul(a, A.shape, b, B.shape, c, (A.shape[0], B.shape[1]))
    assert e.value.code == -5 and "could not allocate operand planes" in e.value.message
    assert g.stats()["buffers"] == before["buffers"] + 3
    g.matmul(a, A.shape, b, B.shape, c, (A.shape[0], B.shape[1]))   # the same call, nothing armed
    assert oracle.rel_frobenius(c.retrieve((A.shape[0], B.shape[1])), oracle.gemm_f64(A, B)) <= 1e-5
    for x in (a, b, c):
        x.release()
    g.lib().gonngpu_trim_cache()
    after = g.stats()
    # nothing leaked: buffers, held memory and operand planes are back where they were
    assert (after["buffers"], after["hbm_bytes"], after["plane_bytes"]) == \
        (before["buffers"], before["hbm_bytes"], before["plane_bytes"])


def test_download_failure_in_retrieve(gpu, mats):
    g = gpu
    A, _ = mats
    a = g.Buffer.from_host(A)
    t = g.Buffer.empty(A.nbytes)
    g.transpose(a, A.shape, t)
    _inject(g, "d2h", 1)
    with pytest.raises(g.GonnError) as e:
        t.retrieve((A.shape[1], A.shape[0]))
    assert e.value.code == -3 and "Device to host copy failed" in e.value.message
    assert np.array_equal(t.retrieve((A.shape[1], A.shape[0])), A.T)
    a.release()
    t.release()


def test_allocation_failure_in_sharded_matmul(gpu):
    from oracle import oracle
    g = gpu
    rng = np.random.default_rng(42)
    A = (rng.standard_normal((600, 128)) / 11).astype(np.float32)
    B = (rng.standard_normal((128, 64)) / 11).astype(np.float32)
    C = np.zeros((600, 64), np.float32)
    g.lib().gonngpu_trim_cache()
    before = g.stats()
    _inject(g, "alloc", 3)
    with pytest.raises(g.GonnError) as e:
        g.matmul_sharded(A, B, C, n_devices=1)
    assert e.value.code == -5 and "could not allocate device memory" in e.value.message
    assert g.stats()["buffers"] == before["buffers"] and g.stats()["hbm_bytes"] == before["hbm_bytes"]
    g.matmul_sharded(A, B, C, n_devices=1)
    assert oracle.rel_frobenius(C, oracle.gemm_f64(oracle.f16_rn(A), oracle.f16_rn(B))) <= 1e-5
