"""Replication of B over NVSwitch for the row-sharded product.

CPU part: the slot / epoch / acknowledgement numbers `Replicator` hands to the two
C-ABI calls, checked against a small model of the protocol (a slot is never
overwritten while a product that reads it may still run).
GPU part (needs two B200s with an NVSwitch multicast address, skipped on a
one-GPU box): two processes, B different in every epoch, every rank checks bit
for bit what arrived and multiplies its row shard by it; the assembled product
is compared with the float64 oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))
from replicate import Replicator  # noqa: E402


class FakeBinding:
    def __init__(self, log):
        self.log = log

    def replicate_send(self, src, dst, nbytes, bases, world, rank, ctrl, slot, epoch, ack_needed, ctas=0,
                       stream=None):
        self.log.append(("send", rank, slot, epoch, ack_needed, dst, nbytes))

    def replicate_wait(self, bases, world, owner, rank, ctrl, slot, epoch, ack_value):
        self.log.append(("wait", rank, slot, epoch, ack_value, owner))


def test_replicator_sequence_and_slot_safety():
    world, slot_bytes, mc = 4, 1 << 20, 0x7000_0000_0000
    logs = [[] for _ in range(world)]
    reps = [Replicator(FakeBinding(logs[r]), world, r, 0, 0x1000, mc, slot_bytes, 2 * slot_bytes)
            for r in range(world)]
    for _ in range(6):
        slots = {rep.replicate(0xABC0 if rep.rank == 0 else None) for rep in reps}
        assert len(slots) == 1                       # every rank reads the same slot
    sends = [x for x in logs[0] if x[0] == "send"]
    assert [s[3] for s in sends] == [1, 2, 3, 4, 5, 6]
    for _, _, slot, epoch, ack_needed, dst, nbytes in sends:
        assert slot == epoch % 2 and dst == mc + slot * slot_bytes and nbytes == slot_bytes
        # the slot was last read by the products of epoch - 2: exactly those must be acknowledged
        assert ack_needed == max(epoch - 2, 0)
    for r in range(world):
        waits = [x for x in logs[r] if x[0] == "wait"]
        assert [(w[2], w[3], w[4], w[5]) for w in waits] == [(e % 2, e, e - 1, 0) for e in range(1, 7)]
        if r != 0:
            assert not [x for x in logs[r] if x[0] == "send"]
    # model: a rank acknowledges e - 1 only after its product of epoch e - 1; the owner overwrites
    # slot s at epoch e only when every ack >= e - 2; products of e - 1 read the OTHER slot.
    for e in range(3, 7):
        assert (e - 1) % 2 != e % 2 and (e - 2) % 2 == e % 2


def test_replicator_channels_share_a_buffer():
    """Two column slabs of B: each channel has its own slots and control words."""
    slab, log = 1 << 16, []
    chans = [Replicator(FakeBinding(log), 2, 0, 0, 0x1000, 0x9000_0000, slab, 4 * slab + 128 * j,
                        data_offset=2 * slab * j, send_stream=0x55) for j in range(2)]
    for rep in chans:
        rep.send(0xAB00)
    for rep in chans:
        rep.wait()
    sends = [x for x in log if x[0] == "send"]
    assert [s[5] for s in sends] == [0x9000_0000 + slab, 0x9000_0000 + 3 * slab]   # epoch 1 -> slot 1
    assert [x[0] for x in log] == ["send", "send", "wait", "wait"]
    assert chans[1].slot_offset(0) == 2 * slab and chans[1].slot_offset(1) == 3 * slab


def test_replicator_rejects_bad_layout():
    with pytest.raises(ValueError):
        Replicator(FakeBinding([]), 2, 0, 0, 1, 2, 1000, 4096)       # slot not a multiple of 16
    with pytest.raises(ValueError):
        Replicator(FakeBinding([]), 2, 0, 0, 1, 2, 1024, 1024)       # control words inside a slot
    rep = Replicator(FakeBinding([]), 2, 0, 0, 1, 2, 1024, 2048)
    with pytest.raises(ValueError):
        rep.replicate(None)                                          # the owner must name a source


@pytest.mark.gpu
def test_wait_that_nothing_answers_runs_out_and_reports(gpu):
    """Failure detection without a fault: one GPU, a group of one, an arrival flag that nobody
    sets.  The wait kernel gives up after its limit (1.5 s), the call returns -6 with the slot,
    the epoch and the last value seen, the acknowledgement has been written, and the library
    goes on working.  Then the flag is set and the same wait returns at once."""
    import time
    g = gpu
    L = g.lib()
    L.gonngpu_set_blocking(1)
    words = np.zeros(64, np.uint32)                      # control words (first 128 bytes) + spare
    ctrl = g.Buffer.from_host(words.view(np.float32))
    ctrl_addr = L.gonngpu_device_address(ctrl.handle)
    assert ctrl_addr
    bases = g.Buffer.from_host(np.array([ctrl_addr, 0], np.uint64).view(np.float32))
    bases_addr = L.gonngpu_device_address(bases.handle)
    assert bases_addr
    t0 = time.time()
    with pytest.raises(g.GonnError) as ei:
        g.replicate_wait(bases_addr, 1, 0, 0, 0, 1, 7, 6)     # slot 1, epoch 7, acknowledge 6
    dt = time.time() - t0
    assert ei.value.code == -6 and "role 5" in ei.value.message
    assert 1.0 < dt < 20.0
    assert g.last_kernel_status() == [5, 1, 7, 0]
    seen = ctrl.retrieve((64,)).view(np.uint32)
    assert seen[16] == 6 and seen[0] == 0 and seen[1] == 0    # ack[0] written, flags untouched
    words[1] = 9                                              # a later epoch satisfies the wait too
    ctrl.upload(words.view(np.float32))
    t0 = time.time()
    g.replicate_wait(bases_addr, 1, 0, 0, 0, 1, 7, 6)
    assert time.time() - t0 < 1.0
    # the context is intact: a product still matches the oracle
    from oracle import oracle
    rng = np.random.default_rng(5)
    A = rng.standard_normal((96, 40)).astype(np.float32)
    B = rng.standard_normal((40, 24)).astype(np.float32)
    a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
    c = g.Buffer.from_host(np.zeros((96, 24), np.float32))
    g.matmul(a, A.shape, b, B.shape, c, (96, 24))
    assert oracle.rel_frobenius(c.retrieve((96, 24)), oracle.gemm_f64(A, B)) <= 1e-5
    for x in (a, b, c, ctrl, bases):
        x.release()
    # argument checks answer without touching the GPU
    for bad in [dict(world=0), dict(rank=1), dict(owner=3), dict(slot=2), dict(ctrl=8)]:
        kw = dict(world=1, owner=0, rank=0, ctrl=0, slot=0)
        kw.update(bad)
        with pytest.raises(g.GonnError) as ei:
            g.replicate_wait(1 << 20, kw["world"], kw["owner"], kw["rank"], kw["ctrl"], kw["slot"], 1, 0)
        assert ei.value.code == -3


@pytest.mark.gpu
def test_two_gpu_replication_and_sharded_product(tmp_path, gpu):
    if gpu.lib().gonngpu_device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29600 + (os.getpid() % 300)
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "replicate_worker.py"), str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    if (tmp_path / "skipped.txt").exists():
        pytest.skip((tmp_path / "skipped.txt").read_text())
    from oracle import oracle
    meta = np.load(tmp_path / "inputs.npz")
    for e in range(int(meta["epochs"])):
        C = np.concatenate([np.load(tmp_path / f"c_{e}_{r}.npy") for r in range(2)], axis=0)
        ref = oracle.gemm_f64(meta["A"].astype(np.float16).astype(np.float32),
                              meta[f"B{e}"].astype(np.float16).astype(np.float32))
        assert oracle.rel_frobenius(C, ref) <= 1e-2      # fp16 path tolerance
    assert (tmp_path / "bit_exact.txt").read_text() == "1"
