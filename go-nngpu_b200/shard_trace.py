"""Timeline of one step of the row-sharded product that replicates B itself
(`gonngpu_gemm_f16_sharded`), as the kernel records it with `gonngpu_set_sharded_trace`.

    python go-nngpu_b200/shard_trace.py [rows_per_rank] [first_group]                  (a group of one)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29517 go-nngpu_b200/shard_trace.py [rows_per_rank] [first_group]

K = N = 4096 (B = 32 MiB), fp16 operands.  After a few untimed steps every rank runs three
steps, each started behind a barrier, and prints the last one as a JSON line: the step's
duration (CUDA events), and in microseconds after the rank's own kernel start: when the
owner's watcher published each of the 16 column slabs (owner only), when a producer of the
rank first took each slab's flag (a slab that nobody had to wait for shows when it was first
needed), and when the last CTA left.  Times of different ranks come from different clocks.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

K = N = 4096


def main():
    import torch
    import gonngpu as g
    from replicate import ShardedProduct, open_symmetric
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    rows = int(sys.argv[1]) if len(sys.argv) > 1 else 16384
    first_group = int(sys.argv[2]) if len(sys.argv) > 2 else 0
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
    L = g.lib()
    assert L.gonngpu_set_device(local) == 0, "no usable B200 for this rank"
    stream = torch.cuda.ExternalStream(L.gonngpu_stream(), device=dev)
    slot_bytes = 2 * K * N
    with torch.cuda.stream(stream):
        A16 = (torch.randn((rows, K), device=dev) / 64).half()
        B16 = (torch.randn((K, N), device=dev) / 64).half()
        C = torch.empty((rows, N), device=dev)
        if world > 1:
            buf, hdl, _ = open_symmetric(torch, dist, dev, slot_bytes, require_multicast=False)
            base, bases, mc = buf.data_ptr(), int(hdl.buffer_ptrs_dev), int(hdl.multicast_ptr) or None
        else:  # a group of one: the owner writes its own slot with plain stores
            buf = torch.zeros(2 * slot_bytes + 4096, dtype=torch.uint8, device=dev)
            keep = torch.tensor([buf.data_ptr()], dtype=torch.int64, device=dev)
            base, bases, mc = buf.data_ptr(), keep.data_ptr(), None
        buf.zero_()
        stream.synchronize()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        prod = ShardedProduct(g, world, rank, 0, base, bases, mc, K, N, first_group)
        trace = torch.full((128,), -1, dtype=torch.int64, device=dev)
        L.gonngpu_set_blocking(0)

        def step():
            prod.step(A16.data_ptr(), rows, K, C.data_ptr(), N, b_src_ptr=B16.data_ptr() if rank == 0 else None)

        for _ in range(6):
            step()
        stream.synchronize()
        g.synchronize()
        L.gonngpu_set_sharded_trace(trace.data_ptr())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        line = None
        for _ in range(3):
            trace.fill_(-1)
            stream.synchronize()
            if dist:
                dist.barrier()
            e0.record(stream)
            step()
            e1.record(stream)
            stream.synchronize()
            g.synchronize()
            t = trace.cpu().numpy().astype(np.uint64)
            t0 = int(t[0])

            def rel(words):
                return [None if int(x) == 2 ** 64 - 1 else round((int(x) - t0) / 1e3, 1) for x in words]

            line = {"rank": rank, "world": world, "rows": rows, "ms": round(e0.elapsed_time(e1), 4),
                    "last_cta_left_us": rel(t[80:81])[0], "slab_published_us": rel(t[1:17]),
                    "slab_first_taken_us": rel(t[40:56])}
        L.gonngpu_set_sharded_trace(None)
        L.gonngpu_set_blocking(1)
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
