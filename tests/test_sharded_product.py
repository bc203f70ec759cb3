"""Row-sharded product whose kernel replicates B itself (gonngpu_gemm_f16_sharded).

CPU part: the epoch / slot numbers `ShardedProduct` hands to the C-ABI call.
One-GPU part: a group of one (the owner sends to itself with plain stores, so
sender warps, arrival flags, gating, the slab-by-slab tile order and the
acknowledgement all run), B different in every epoch, against the float64
oracle and bit for bit against the ordinary fp16 product; a rank whose B never
arrives gives up after its limit and reports, without a fault, and the library
goes on working.
Two-GPU part (skipped on a one-GPU box): two processes over an NVSwitch
multicast address and over plain peer stores, B different in every epoch, the
assembled product against the float64 oracle.
"""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))
from replicate import ShardedProduct  # noqa: E402

CTRL_WORDS = 128  # 512 bytes: arrived[2][32], ack[16], sent[32], exited, gave_up, pad


class FakeBinding:
    def __init__(self):
        self.calls = []

    def gemm_f16_sharded(self, a_ptr, a_shape, a_pitch, b_src, n, local, bases, mc, world, owner, rank,
                         slots_offset, ctrl_offset, epoch, c_ptr, ldc, first_group=0):
        self.calls.append(dict(b_src=b_src, epoch=epoch, ctrl=ctrl_offset, slots=slots_offset, rank=rank,
                               shape=a_shape, n=n))


def test_sharded_product_epochs_and_slots():
    k, n = 512, 768
    fakes = [FakeBinding() for _ in range(3)]
    prods = [ShardedProduct(fakes[r], 3, r, 1, 0x1000 * (r + 1), 0x9000, 0x7000_0000, k, n) for r in range(3)]
    for e in range(1, 6):
        slots = {p.step(0xA000, 256, k, 0xC000, n, b_src_ptr=0xB000) for p in prods}
        assert slots == {e % 2}                                   # every rank reads the same slot
    for r, f in enumerate(fakes):
        assert [c["epoch"] for c in f.calls] == [1, 2, 3, 4, 5]
        assert all(c["ctrl"] == 4 * k * n and c["slots"] == 0 for c in f.calls)
        # only the owner hands over a source
        assert all((c["b_src"] == 0xB000) == (r == 1) for c in f.calls)
    with pytest.raises(ValueError):
        ShardedProduct(FakeBinding(), 2, 0, 0, 1, 2, 3, 64, 100)      # N not a multiple of 8
    p = ShardedProduct(FakeBinding(), 2, 0, 0, 1, 2, 3, 64, 64)
    with pytest.raises(ValueError):
        p.step(1, 2, 64, 3, 64)                                   # the owner must name B


class Group1:
    """A symmetric buffer for a group of one on the current GPU: two slots of B, then the
    control words; `bases` holds its address `world` times."""

    def __init__(self, g, k, n, world=1):
        self.g, self.k, self.n = g, k, n
        self.slot_bytes = 2 * k * n
        self.nbytes = 2 * self.slot_bytes + 4 * CTRL_WORDS
        self.buf = g.Buffer.from_host(np.zeros(self.nbytes // 4, np.float32))
        self.addr = g.lib().gonngpu_device_address(self.buf.handle)
        assert self.addr
        self.bases = g.Buffer.from_host(np.array([self.addr] * world, np.uint64).view(np.float32))
        self.bases_addr = g.lib().gonngpu_device_address(self.bases.handle)
        assert self.bases_addr

    def words(self):
        raw = self.buf.retrieve((self.nbytes // 4,)).view(np.uint32)
        return raw[2 * self.slot_bytes // 4:]

    def slot(self, i):
        raw = self.buf.retrieve((self.nbytes // 4,)).view(np.float16)
        return raw[i * self.k * self.n:(i + 1) * self.k * self.n].reshape(self.k, self.n)

    def set_words(self, words):
        raw = self.buf.retrieve((self.nbytes // 4,)).view(np.uint32).copy()
        raw[2 * self.slot_bytes // 4:] = words
        self.buf.upload(raw.view(np.float32))

    def release(self):
        self.buf.release()
        self.bases.release()


def f16_plane(g, x):
    """fp16 copy of a float32 matrix in device memory (dense); returns (buffer, address)."""
    src = g.Buffer.from_host(x)
    dst = g.Buffer.empty(max(x.size * 2, 16))
    g.convert_f16_device(src.device_address(), x.shape[0], x.shape[1], dst.device_address(), x.shape[1])
    src.release()
    return dst, dst.device_address()


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n,first_group", [(1000, 512, 768, 0), (300, 200, 72, 0), (5000, 264, 2056, 3),
                                               (20000, 1024, 4096, 32)])
def test_group_of_one_sends_to_itself_and_multiplies(gpu, m, k, n, first_group):
    from oracle import oracle
    g = gpu
    g.lib().gonngpu_set_blocking(1)
    grp = Group1(g, k, n)
    prod = ShardedProduct(g, 1, 0, 0, grp.addr, grp.bases_addr, None, k, n, first_group)
    rng = np.random.default_rng(21)
    A = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
    a16, a_addr = f16_plane(g, A)
    c = g.Buffer.empty(m * n * 4)
    c2 = g.Buffer.empty(m * n * 4)
    tiles_n = -(-n // 256)
    slab_tiles = -(-tiles_n // 32)
    slabs = -(-tiles_n // slab_tiles)
    pair_kernel = m >= 256 and n >= 128 and -(-m // 256) * tiles_n >= 74
    for e in range(1, 5):
        B = (rng.standard_normal((k, n)) / np.sqrt(k) * e).astype(np.float32)
        b16, b_addr = f16_plane(g, B)
        slot = prod.step(a_addr, m, k, c.device_address(), n, b_src_ptr=b_addr)
        assert slot == e % 2
        C = c.retrieve((m, n))
        # B arrived bit for bit in the slot of this epoch
        assert np.array_equal(grp.slot(slot).view(np.uint16), B.astype(np.float16).view(np.uint16))
        ref = oracle.gemm_f64(A.astype(np.float16).astype(np.float32), B.astype(np.float16).astype(np.float32))
        assert oracle.rel_frobenius(C, ref) <= 1e-2                # fp16-path tolerance
        # the same tiles and the same accumulation order as the ordinary fp16 product
        g.gemm_f16_device(a_addr, (m, k), k, False, b_addr, (k, n), n, False, c2.device_address(), n)
        if pair_kernel:                                           # both run the 256-row pair kernel
            assert np.array_equal(C.view(np.uint32), c2.retrieve((m, n)).view(np.uint32))
        else:
            assert oracle.rel_frobenius(C, c2.retrieve((m, n)).astype(np.float64)) <= 1e-5
        w = grp.words()
        assert list(w[slot * 32:slot * 32 + slabs]) == [e] * slabs     # every slab's flag raised
        assert w[64] == e                                          # acknowledged to the owner (itself)
        assert not w[80:114].any()                                 # scratch words back to zero
        b16.release()
    for x in (a16, c, c2):
        x.release()
    grp.release()


@pytest.mark.gpu
def test_rank_whose_b_never_arrives_gives_up_and_reports(gpu):
    """Failure detection without a fault: rank 0 of a group of two whose owner (rank 1) does not
    exist.  The producers' wait for the first slab runs out (1.25 s), the call returns -6 with the
    slab, tile and epoch, no acknowledgement is written, and the library goes on working.  With
    the flags set by hand (the data is then whatever lies in the slot) the same call succeeds."""
    from oracle import oracle
    g = gpu
    g.lib().gonngpu_set_blocking(1)
    m, k, n = 600, 256, 512
    grp = Group1(g, k, n, world=2)
    rng = np.random.default_rng(22)
    A = (rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32)
    B = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    a16, a_addr = f16_plane(g, A)
    c = g.Buffer.empty(m * n * 4)
    t0 = time.time()
    with pytest.raises(g.GonnError) as ei:
        g.gemm_f16_sharded(a_addr, (m, k), k, None, n, grp.addr, grp.bases_addr, None, 2, 1, 0, 0,
                           2 * grp.slot_bytes, 3, c.device_address(), n)
    dt = time.time() - t0
    assert ei.value.code == -6 and "role 6" in ei.value.message
    assert 1.0 < dt < 20.0
    st = g.last_kernel_status()
    assert st[0] == 6 and st[1] in (0, 1) and st[3] == 3            # one of the two slabs, epoch 3
    w = grp.words()
    assert not w.any()                                              # no flag, no acknowledgement, scratch zero
    # now the data "arrives": B into slot 1 (epoch 3), both slabs flagged
    raw = grp.buf.retrieve((grp.nbytes // 4,)).view(np.float16).copy()
    raw[k * n:2 * k * n] = B.astype(np.float16).ravel()
    grp.buf.upload(raw.view(np.float32))
    words = np.zeros(CTRL_WORDS, np.uint32)
    words[32:34] = 3
    grp.set_words(words)
    t0 = time.time()
    g.gemm_f16_sharded(a_addr, (m, k), k, None, n, grp.addr, grp.bases_addr, None, 2, 1, 0, 0,
                       2 * grp.slot_bytes, 3, c.device_address(), n)
    assert time.time() - t0 < 1.0
    ref = oracle.gemm_f64(A.astype(np.float16).astype(np.float32), B.astype(np.float16).astype(np.float32))
    assert oracle.rel_frobenius(c.retrieve((m, n)), ref) <= 1e-2
    w = grp.words()
    assert w[64] == 3 and w[65] == 0                                # ack[0] on the "owner" (same buffer)
    # the context is intact: an fp32 product still matches the oracle
    a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
    c32 = g.Buffer.empty(m * n * 4)
    g.matmul(a, A.shape, b, B.shape, c32, (m, n))
    assert oracle.rel_frobenius(c32.retrieve((m, n)), oracle.gemm_f64(A, B)) <= 1e-5
    # argument checks answer without touching the GPU
    ok = dict(a=a_addr, shape=(m, k), pitch=k, n=n, world=2, owner=1, rank=0, slots=0,
              ctrl=2 * grp.slot_bytes, epoch=1)
    for bad, code in [(dict(n=100), -3), (dict(world=0), -3), (dict(rank=2), -3), (dict(owner=5), -3),
                      (dict(epoch=0), -3), (dict(ctrl=8), -3), (dict(ctrl=16), -3), (dict(pitch=k + 1), -3),
                      (dict(a=0), -2), (dict(owner=0), -2)]:        # owner without a source
        kw = dict(ok)
        kw.update(bad)
        with pytest.raises(g.GonnError) as ei:
            g.gemm_f16_sharded(kw["a"], kw["shape"], kw["pitch"], None, kw["n"], grp.addr, grp.bases_addr,
                               None, kw["world"], kw["owner"], kw["rank"], kw["slots"], kw["ctrl"],
                               kw["epoch"], c.device_address(), n)
        assert ei.value.code == code, (bad, ei.value.code)
    for x in (a16, c, a, b, c32):
        x.release()
    grp.release()


@pytest.mark.gpu
def test_two_gpu_sharded_product(tmp_path, gpu):
    if gpu.lib().gonngpu_device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29300 + (os.getpid() % 300)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "sharded_worker.py"), str(tmp_path)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    from oracle import oracle
    meta = np.load(tmp_path / "inputs.npz")
    modes = (tmp_path / "modes.txt").read_text().split()
    assert "peer" in modes                                          # plain peer stores always run
    A16 = meta["A"].astype(np.float16).astype(np.float32)
    for mode in modes:
        for e in range(int(meta["epochs"])):
            C = np.concatenate([np.load(tmp_path / f"c_{mode}_{e}_{r}.npy") for r in range(2)], axis=0)
            ref = oracle.gemm_f64(A16, meta[f"B{e}"].astype(np.float16).astype(np.float32))
            assert oracle.rel_frobenius(C, ref) <= 1e-2, (mode, e)  # fp16 path tolerance
        assert (tmp_path / f"bit_exact_{mode}.txt").read_text() == "1"
