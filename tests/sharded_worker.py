"""One rank of the two-GPU test of the row-sharded product that replicates B itself
(started by torchrun from tests/test_sharded_product.py).  Every epoch has its own B and all
epochs are queued back to back without a host wait, so a slot that was read too early or
overwritten too early shows up as a wrong product or a failed bit comparison.  The pass over
plain peer stores always runs; the pass over the NVSwitch multicast address runs when the
group has one."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))

M, K, N, EPOCHS = 40960, 512, 1280, 6


def main():
    out = sys.argv[1]
    import torch
    import torch.distributed as dist
    import gonngpu as g
    from replicate import ShardedProduct, open_symmetric
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
    buf, hdl, ctrl = open_symmetric(torch, dist, dev, slot_bytes, require_multicast=False)
    torch.cuda.synchronize()
    dist.barrier()
    modes = ["peer"] + (["multicast"] if int(hdl.multicast_ptr) else [])

    rng = np.random.default_rng(12)
    A = (rng.standard_normal((M, K)) / np.sqrt(K)).astype(np.float32)
    Bs = [(rng.standard_normal((K, N)) / np.sqrt(K) * (e + 1)).astype(np.float32) for e in range(EPOCHS)]
    if rank == 0:
        np.savez(os.path.join(out, "inputs.npz"), A=A, epochs=EPOCHS, **{f"B{e}": b for e, b in enumerate(Bs)})
        with open(os.path.join(out, "modes.txt"), "w") as f:
            f.write(" ".join(modes))
    lo, hi = shard_rows(M, world, rank)
    slots = [buf[i * slot_bytes:(i + 1) * slot_bytes].view(torch.float16).view(K, N) for i in range(2)]
    with torch.cuda.stream(stream):
        A16 = torch.from_numpy(A[lo:hi]).to(dev).half()
        B16 = [torch.from_numpy(b).to(dev).half() for b in Bs]
        for mode in modes:
            buf.zero_()
            stream.synchronize()
            torch.cuda.synchronize()
            dist.barrier()
            prod = ShardedProduct(g, world, rank, 0, buf.data_ptr(), int(hdl.buffer_ptrs_dev),
                                  int(hdl.multicast_ptr) if mode == "multicast" else None, K, N)
            Cs = [torch.zeros((hi - lo, N), device=dev, dtype=torch.float32) for _ in range(EPOCHS)]
            L.gonngpu_set_blocking(0)
            for e in range(EPOCHS):
                prod.step(A16.data_ptr(), hi - lo, K, Cs[e].data_ptr(), N,
                          b_src_ptr=B16[e].data_ptr() if rank == 0 else None)
            stream.synchronize()
            g.synchronize()          # raises if a bounded wait ran out
            L.gonngpu_set_blocking(1)
            # a slot may be overwritten as soon as every rank's product of its epoch has finished,
            # so only the last two epochs can still be compared bit for bit afterwards
            bit_exact = all(torch.equal(slots[(e + 1) % 2], B16[e]) for e in (EPOCHS - 2, EPOCHS - 1))
            for e in range(EPOCHS):
                np.save(os.path.join(out, f"c_{mode}_{e}_{rank}.npy"), Cs[e].cpu().numpy())
            okt = torch.tensor([1 if bit_exact else 0], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            if rank == 0:
                with open(os.path.join(out, f"bit_exact_{mode}.txt"), "w") as f:
                    f.write(str(int(okt[0])))
            torch.cuda.synchronize()
            dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
