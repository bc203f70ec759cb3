"""One rank of the two-GPU replication test (started by torchrun from
tests/test_replicate.py).  Every epoch has its own B, so a slot that was read
too early or overwritten too early shows up as a wrong product or a failed
bit comparison."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))

M, K, N, EPOCHS = 1024, 512, 768, 5


def main():
    out = sys.argv[1]
    import torch
    import torch.distributed as dist
    import gonngpu as g
    from replicate import Replicator, open_symmetric
    from sharding import shard_rows
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    L = g.lib()
    assert L.gonngpu_set_device(local) == 0
    stream = torch.cuda.ExternalStream(L.gonngpu_stream(), device=dev)
    slot_bytes = 2 * K * N
    ok, why = 1, ""
    try:
        buf, hdl, ctrl = open_symmetric(torch, dist, dev, slot_bytes)
    except Exception as e:  # noqa: BLE001
        ok, why = 0, f"{type(e).__name__}: {e}"
    okt = torch.tensor([ok], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if int(okt[0]) == 0:
        if rank == 0:
            with open(os.path.join(out, "skipped.txt"), "w") as f:
                f.write("no symmetric multicast memory on this box: " + why)
        dist.destroy_process_group()
        return
    torch.cuda.synchronize()
    dist.barrier()

    rng = np.random.default_rng(11)
    A = (rng.standard_normal((M, K)) / np.sqrt(K)).astype(np.float32)
    Bs = [(rng.standard_normal((K, N)) / np.sqrt(K) * (e + 1)).astype(np.float32) for e in range(EPOCHS)]
    if rank == 0:
        np.savez(os.path.join(out, "inputs.npz"), A=A, epochs=EPOCHS, **{f"B{e}": b for e, b in enumerate(Bs)})
    lo, hi = shard_rows(M, world, rank)
    # the owner's pushes run on a stream of their own, unordered against the products: only the
    # acknowledgements keep a slot from being overwritten while it is read
    side = torch.cuda.Stream(device=dev, priority=-1)
    rep = Replicator(g, world, rank, 0, int(hdl.buffer_ptrs_dev), int(hdl.multicast_ptr), slot_bytes, ctrl,
                     ctas=16, send_stream=side.cuda_stream)
    slots = [buf[i * slot_bytes:(i + 1) * slot_bytes].view(torch.float16).view(K, N) for i in range(2)]
    bit_exact = True
    with torch.cuda.stream(stream):
        A16 = torch.from_numpy(A[lo:hi]).to(dev).half()
        B16 = [torch.from_numpy(b).to(dev).half() for b in Bs]
        Cs = [torch.zeros((hi - lo, N), device=dev, dtype=torch.float32) for _ in range(EPOCHS)]
        got = [torch.zeros((K, N), device=dev, dtype=torch.float16) for _ in range(EPOCHS)]
        stream.synchronize()
        L.gonngpu_set_blocking(0)
        # all epochs are queued back to back without a host wait: the ordering is the kernels' own
        for e in range(EPOCHS):
            slot = rep.replicate(B16[e].data_ptr() if rank == 0 else None)
            g.gemm_f16_device(A16.data_ptr(), (hi - lo, K), K, False, slots[slot].data_ptr(), (K, N), N,
                              False, Cs[e].data_ptr(), N)
            got[e].copy_(slots[slot])
        stream.synchronize()
        side.synchronize()
        g.synchronize()          # raises if a bounded wait ran out
        L.gonngpu_set_blocking(1)
        for e in range(EPOCHS):
            bit_exact = bit_exact and torch.equal(got[e], B16[e])
            np.save(os.path.join(out, f"c_{e}_{rank}.npy"), Cs[e].cpu().numpy())
    okt = torch.tensor([1 if bit_exact else 0], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(os.path.join(out, "bit_exact.txt"), "w") as f:
            f.write(str(int(okt[0])))
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
