#!/usr/bin/env python
"""Benchmark of the dense-GEMM hot path.

    python bench.py --gpus N --steps K --warmup W            (our CUDA path)
    python bench.py --impl reference --gpus N --steps K ...  (CPU baseline arm)

Workload: the row-sharded tall GEMM of the benchmark configurations, fp16
inputs / fp32 accumulate / fp32 C, M=131072, K=4096, N=4096, A split by rows
across the N ranks (one process per GPU), B replicated from rank 0 over
NVLink inside every step when N > 1 (this library's multicast-store kernel
through NVSwitch, or NCCL's broadcast: --bcast).  Inputs are seeded synthetic
normal(0, 1/sqrt(K)) values.  One "step" is one full product.

`value` is device-timed with the operands already resident in HBM as fp16;
`e2e` is the same product through the handle-based C ABI from page-locked host
memory (float32 in, float32 out, copies and the fp32->fp16 pre-pass included).
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))
sys.path.insert(0, ROOT)

M_TOTAL, K_DIM, N_DIM = 131072, 4096, 4096
WORKLOAD = "row-sharded GEMM fp16-in/fp32-acc M=131072 K=4096 N=4096 (A rows split, B replicated)"
METRIC = "GEMM TFLOP/s"


from sharding import shard_rows  # go-nngpu_b200/sharding.py  # noqa: E402


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"burst": float(p["bf16_tflops"]), "sustained": float(p["bf16_tflops_sustained"]),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def result(self):
        self.stop_flag = True
        self.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_gemm_rate(rows, seconds_hint=None):
    """float64 product of a `rows`-row slice of the workload on the host cores
    (numpy / OpenBLAS): the stand-in for gonum's mat.Dense.Mul, which is not
    installable here.  Returns (TFLOP/s, seconds, threads)."""
    rng = np.random.default_rng(4)
    s = 1.0 / np.sqrt(K_DIM)
    A = (rng.standard_normal((rows, K_DIM)) * s).astype(np.float32).astype(np.float16).astype(np.float64)
    B = (rng.standard_normal((K_DIM, N_DIM)) * s).astype(np.float32).astype(np.float16).astype(np.float64)
    t0 = time.perf_counter()
    C = A @ B
    dt = time.perf_counter() - t0
    assert np.isfinite(C[0, 0])
    return 2.0 * rows * K_DIM * N_DIM / dt / 1e12, dt, blas_threads()


def blas_threads():
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 0) for p in threadpool_info() if p.get("user_api") == "blas"]
        return int(max(n)) if n else (os.cpu_count() or 1)
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, rank):
    """CPU arm: the float64 GEMM on the host cores over a bounded row sample."""
    if rank != 0:
        return
    # size the sample so that steps+warmup fit in ~2 minutes
    probe_rows = 256
    rate, dt, threads = cpu_gemm_rate(probe_rows)
    budget = 120.0 / max(args.steps + args.warmup, 1)
    rows = int(min(M_TOTAL, max(probe_rows, probe_rows * budget / max(dt, 1e-6))))
    rows = max(128, rows // 128 * 128)
    rng = np.random.default_rng(4)
    s = 1.0 / np.sqrt(K_DIM)
    A = (rng.standard_normal((rows, K_DIM)) * s).astype(np.float32).astype(np.float16).astype(np.float64)
    B = (rng.standard_normal((K_DIM, N_DIM)) * s).astype(np.float32).astype(np.float16).astype(np.float64)
    for _ in range(args.warmup):
        A @ B
    t0 = time.perf_counter()
    for _ in range(args.steps):
        A @ B
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    val = 2.0 * rows * K_DIM * N_DIM / dt / 1e12
    sample = f"{rows} of {M_TOTAL} rows per step (float64 numpy/OpenBLAS; stand-in for gonum mat.Dense.Mul, gonum/Go not installed)"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def setup_multimem(torch, dist, dev, rank, world, required, slabs, ctas=0, side_stream=True):
    """Symmetric buffer for B with an NVSwitch multicast address: one channel per column slab
    (two slots and 128 bytes of control words each).  torch's symmetric-memory allocator does
    the allocation, the exchange of handles between the processes and the multicast binding;
    the copies and the signalling are this library's kernels.  The owner's pushes go to a stream
    of their own, so that slab j+1 travels while slab j is multiplied.
    Returns None (on every rank alike) when the GPUs offer no multicast address, unless
    `required`."""
    from replicate import Replicator, open_symmetric  # go-nngpu_b200/replicate.py
    import gonngpu as g
    total = 2 * K_DIM * N_DIM
    slab_bytes, w = total // slabs, N_DIM // slabs
    res, why = None, ""
    try:
        buf, hdl, ctrl = open_symmetric(torch, dist, dev, total)
        # a stream of its own for the pushes (high priority: placed ahead of queued product grids)
        side = torch.cuda.Stream(device=dev, priority=-1) if side_stream else None
        chans = []
        for j in range(slabs):
            off = j * 2 * slab_bytes
            rep = Replicator(g, world, rank, 0, int(hdl.buffer_ptrs_dev), int(hdl.multicast_ptr), slab_bytes,
                             ctrl + 128 * j, ctas, data_offset=off,
                             send_stream=side.cuda_stream if side is not None else None)
            views = [buf[rep.slot_offset(i):rep.slot_offset(i) + slab_bytes].view(torch.float16).view(K_DIM, w)
                     for i in range(2)]
            chans.append((rep, views))
        res = {"buf": buf, "hdl": hdl, "chans": chans, "side": side}
    except Exception as e:  # noqa: BLE001 - any failure means "take the NCCL broadcast"
        why = f"{type(e).__name__}: {e}"
    ok = torch.tensor([1 if res is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    if int(ok[0]) == 0:
        if required:
            raise RuntimeError(f"--bcast multimem: symmetric multicast memory unavailable ({why})")
        if rank == 0 and why:
            print(f"[bench] multicast replication unavailable, using the NCCL broadcast: {why}",
                  file=sys.stderr, flush=True)
        return None
    return res


def run_ours(args, rank, world, local_rank):
    import torch
    import gonngpu as g
    import build as gonn_build
    if rank == 0:
        gonn_build.build()
    dist = None
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    L = g.lib()
    assert L.gonngpu_set_device(local_rank) == 0, "no usable B200 for this rank"
    stream = torch.cuda.ExternalStream(L.gonngpu_stream(), device=torch.device("cuda", local_rank))
    lo, hi = shard_rows(M_TOTAL, world, rank)
    rows = hi - lo
    dev = torch.device("cuda", local_rank)
    scale = 1.0 / np.sqrt(K_DIM)

    with torch.cuda.stream(stream):
        gen = torch.Generator(device=dev)
        gen.manual_seed(4 * 1000 + rank)
        A32 = torch.randn((rows, K_DIM), generator=gen, device=dev, dtype=torch.float32) * scale
        A16 = torch.empty((rows, K_DIM), device=dev, dtype=torch.float16)
        B16 = torch.zeros((K_DIM, N_DIM), device=dev, dtype=torch.float16)
        C = torch.empty((rows, N_DIM), device=dev, dtype=torch.float32)
        gen.manual_seed(4)
        B32 = torch.randn((K_DIM, N_DIM), generator=gen, device=dev, dtype=torch.float32) * scale
        L.gonngpu_set_blocking(0)
        g.convert_f16_device(A32.data_ptr(), rows, K_DIM, A16.data_ptr(), K_DIM)
        # every rank converts its own copy of B (same seed): rank 0's is the one that travels, the
        # others' only serve to check, bit for bit, what arrived
        g.convert_f16_device(B32.data_ptr(), K_DIM, N_DIM, B16.data_ptr(), N_DIM)
        stream.synchronize()

        # With several ranks B may travel as `slabs` column slabs: the product of slab j (its own
        # columns of C) starts as soon as slab j has arrived, so later slabs travel while earlier
        # ones are multiplied.  Measured on 8 GPUs it loses both ways: NCCL's broadcast kernels
        # take SMs from the GEMM, and the multicast push of slab j+1, sharing the owner's SMs with
        # the product of slab j, slows to less than its stand-alone rate (2 slabs 0.553 ms per
        # step against 0.506 ms with 1).  Default: 1 slab.
        use_mm = world > 1 and args.bcast in ("auto", "multimem")
        slabs = max(1, args.slabs) if world > 1 else 1
        if args.gemm_ctas:
            assert L.gonngpu_set_gemm_tuning(0, args.gemm_ctas) == 0
        assert N_DIM % (slabs * 256) == 0, "--slabs must leave whole 256-column tiles"
        w = N_DIM // slabs
        Bs = [torch.zeros((K_DIM, w), device=dev, dtype=torch.float16) for _ in range(slabs)]
        if rank == 0:
            for j in range(slabs):
                Bs[j].copy_(B16[:, j * w:(j + 1) * w])
        stream.synchronize()

        # B can also travel as scatter + all-gather: rank 0 sends each rank 1/world of B's rows,
        # then every rank gathers the pieces, instead of NCCL's broadcast.  Measured: slower
        # (8 GPUs 0.27 against 0.19 ms for the 32 MiB, 2 GPUs 0.19 against 0.07 ms): not the default.
        two_step = world > 1 and args.bcast == "scatter_allgather" and slabs == 1 and K_DIM % world == 0
        if two_step:
            piece = torch.zeros((K_DIM // world, N_DIM), device=dev, dtype=torch.float16)
            pieces = list(Bs[0].chunk(world, dim=0)) if rank == 0 else None

        # Default with several ranks: rank 0 pushes B once into NVSwitch with multimem stores
        # (gonngpu_replicate_send) and the switch delivers it to every GPU; two slots alternate so
        # that the next B can be written while products still read the previous one.
        mm = None
        transport = args.bcast if world > 1 else "none"
        if use_mm:
            mm = setup_multimem(torch, dist, dev, rank, world, args.bcast == "multimem", slabs,
                                args.bcast_ctas, args.push_stream == "side")
            transport = "multimem" if mm is not None else "broadcast"

        def step(events=None):
            if mm is not None:
                if rank == 0 and mm["side"] is not None:
                    # the pushes of this step start when the stream has reached this step (B of a
                    # step is not sent ahead of the step), then run beside the products
                    go = torch.cuda.Event()
                    go.record(stream)
                    mm["side"].wait_event(go)
                for j, (rep, _) in enumerate(mm["chans"]):
                    rep.send(Bs[j].data_ptr() if rank == 0 else None)
                for j, (rep, views) in enumerate(mm["chans"]):
                    slot = rep.wait()
                    if events is not None:
                        events[j][0].record(stream)
                    g.gemm_f16_device(A16.data_ptr(), (rows, K_DIM), K_DIM, False, views[slot].data_ptr(),
                                      (K_DIM, w), w, False, C.data_ptr() + 4 * j * w, N_DIM)
                    if events is not None:
                        events[j][1].record(stream)
                return
            if two_step:
                dist.scatter(piece, pieces, src=0)
                works = [dist.all_gather_into_tensor(Bs[0], piece, async_op=True)]
            else:
                works = [dist.broadcast(Bs[j], src=0, async_op=True) for j in range(slabs)] if world > 1 else []
            for j in range(slabs):
                if works:
                    works[j].wait()          # orders the stream, does not block the host
                if events is not None:
                    events[j][0].record(stream)
                g.gemm_f16_device(A16.data_ptr(), (rows, K_DIM), K_DIM, False, Bs[j].data_ptr(),
                                  (K_DIM, w), w, False, C.data_ptr() + 4 * j * w, N_DIM)
                if events is not None:
                    events[j][1].record(stream)

        def current_b():
            if mm is not None:
                return torch.cat([views[rep.slot] for rep, views in mm["chans"]], dim=1)
            return torch.cat(Bs, dim=1)

        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        g.synchronize()
        replica_ok = None
        if world > 1:
            okt = torch.tensor([1 if torch.equal(current_b(), B16) else 0], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            replica_ok = bool(int(okt[0]))
            dist.barrier()
        torch.cuda.synchronize()

        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = g.stats()["kernel_launches"]
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                for _ in range(slabs)] for _ in range(args.steps)]
        ev0.record(stream)
        for i in range(args.steps):
            step(kev[i])
        ev1.record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        clocks = sampler.result()
        g.synchronize()  # surfaces any kernel status
        launches = g.stats()["kernel_launches"] - launches0
        total_ms = ev0.elapsed_time(ev1)
        kernel_ms = float(np.mean([sum(a.elapsed_time(b) for a, b in per_step) for per_step in kev]))
        t = torch.tensor([total_ms, kernel_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, kernel_ms_max = float(t[0]), float(t[1])
        ms_per_step = total_ms / args.steps
        value = 2.0 * M_TOTAL * K_DIM * N_DIM / (ms_per_step * 1e-3) / 1e12

        # ---- spot check of the timed result against the CPU oracle (rank 0, a few rows)
        check = None
        if rank == 0:
            from oracle import oracle
            idx = torch.tensor([0, 1, rows // 2, rows - 1], device=dev)
            ref = oracle.gemm_f64(A16[idx].float().cpu().numpy(), current_b().float().cpu().numpy())
            check = oracle.rel_frobenius(C[idx].cpu().numpy(), ref)

        # ---- end to end through the handle-based C ABI from page-locked host memory
        L.gonngpu_set_blocking(1)
        e2e = None
        if not args.no_e2e:
            e2e = run_e2e(args, g, L, torch, dist, dev, rank, world, rows, A32, B32)
        del A32

    if rank == 0:
        report(args, g, world, rows, total_ms, kernel_ms_max, ms_per_step, value, clocks, launches, check, e2e,
               transport, replica_ok, slabs)
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, g, L, torch, dist, dev, rank, world, rows, A32, B32):
    if True:
        hA, pA = g.pinned_array((rows, K_DIM))
        hC, pC = g.pinned_array((rows, N_DIM))
        hB, pB = g.pinned_array((K_DIM, N_DIM))
        A32h = torch.from_numpy(hA)
        A32h.copy_(A32.cpu())
        torch.from_numpy(hB).copy_(B32.cpu())
        e2e_steps = max(1, min(args.steps, 4))

        def e2e_step():
            a = g.Buffer.from_host(hA)
            c = g.Buffer.from_host(hC)
            if world > 1:
                # rank 0 uploads B; every other rank receives it over NVLink
                Bdev = torch.empty((K_DIM, N_DIM), device=dev, dtype=torch.float32)
                b = g.Buffer.wrap(Bdev.data_ptr(), Bdev.numel() * 4, Bdev)
                if rank == 0:
                    b.upload(hB)
                dist.broadcast(Bdev, src=0)
                L.gonngpu_mark_modified(b.handle)
            else:
                b = g.Buffer.from_host(hB)
            g.matmul_ex(a, (rows, K_DIM), False, b, (K_DIM, N_DIM), False, c, (rows, N_DIM),
                        precision=g.FP16_RN)
            c.retrieve_into(hC)
            for x in (a, b, c):
                x.release()

        e2e_step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s0 = g.stats()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        s1 = g.stats()
        te = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_s = float(te[0])
        e2e_val = 2.0 * M_TOTAL * K_DIM * N_DIM / e2e_s / 1e12
        h2d = (s1["h2d_bytes"] - s0["h2d_bytes"]) // e2e_steps
        d2h = (s1["d2h_bytes"] - s0["d2h_bytes"]) // e2e_steps
        for p in (pA, pB, pC):
            L.gonngpu_host_free(p)
        return {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_s * 1e3, "steps": e2e_steps}


# DRAM bytes of one GEMM launch measured with ncu (dram__bytes_read.sum +
# dram__bytes_write.sum) on the M=8192 case of this kernel: see profiles/.
NCU_TRAFFIC_M8192 = {"read": 179.0e6, "write": 99.8e6, "rows": 8192}


def traffic_estimate(rows):
    """Scales the captured traffic to `rows`: A and C grow with the rows, B (33.6 MB) does not."""
    b_bytes = 2.0 * K_DIM * N_DIM
    per_row = (NCU_TRAFFIC_M8192["read"] + NCU_TRAFFIC_M8192["write"] - b_bytes) / NCU_TRAFFIC_M8192["rows"]
    return per_row * rows + b_bytes


def report(args, g, world, rows, total_ms, kernel_ms_max, ms_per_step, value, clocks, launches, check, e2e,
           transport="none", replica_ok=None, slabs=1):
    if True:
        peaks = load_peaks()
        timed_s = total_ms * 1e-3
        peak_kind = "sustained" if timed_s >= 1.0 else "burst"
        achieved = 2.0 * rows * K_DIM * N_DIM / (kernel_ms_max * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": rows, "parallelism": f"row-shard x{world}",
                       "l2": "operands and result (>=384 MiB per GPU) exceed the 126 MB L2",
                       "b_broadcast_in_step": world > 1, "b_slabs": slabs,
                       "b_transport": transport, "b_replica_bit_exact": replica_ok},
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks[peak_kind], "unit": "TFLOP/s",
                         "frac": achieved / peaks[peak_kind], "traffic": traffic_estimate(rows),
                         "peak_source": f"{peaks['source']} cuBLAS bf16 ({peak_kind})",
                         "kernel_ms": kernel_ms_max},
            "e2e": e2e,
            # the same job with B already resident on every GPU (slowest rank's kernel time only):
            # what the broadcast inside the step costs is the gap between this and `value`
            "value_b_resident": 2.0 * M_TOTAL * K_DIM * N_DIM / (kernel_ms_max * 1e-3) / 1e12,
            "gpu_launches": int(launches),  # GEMM kernels of this library inside the timed region
            "parity_spot_check_rel_frobenius": check,
        }
        if world == 1 and not args.no_cpu:
            rate, dt, threads = cpu_gemm_rate(512)
            # size the sample for roughly 15 s of CPU work (bounded by the whole workload)
            rows_cpu = int(min(M_TOTAL, max(512, 512 * 15.0 / max(dt, 1e-6)))) // 128 * 128
            rate, dt, threads = cpu_gemm_rate(max(rows_cpu, 128))
            line["cpu_baseline"] = {
                "value": rate, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"{max(rows_cpu, 128)} of {M_TOTAL} rows, float64 numpy/OpenBLAS "
                          f"(stand-in for gonum mat.Dense.Mul: Go and gonum are not installed), {dt:.1f} s"}
        print(json.dumps(line), flush=True)


def main():
    global M_TOTAL, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--slabs", type=int, default=1,
                    help="column slabs B travels in when there are several ranks (1, 2, 4 ...)")
    ap.add_argument("--bcast", default="auto",
                    choices=["auto", "multimem", "broadcast", "scatter_allgather"],
                    help="how B reaches the other ranks inside a step: multimem = this library's "
                         "multicast-store kernel over NVSwitch, broadcast = NCCL; auto takes multimem "
                         "when the GPUs offer a multicast address, else broadcast")
    ap.add_argument("--push-stream", default="main", choices=["side", "main"],
                    help="stream of the multicast pushes: the library's, or one of their own (they can "
                         "then run beside a product; costs an event wait per step, measured 8 us)")
    ap.add_argument("--bcast-ctas", type=int, default=32,
                    help="thread blocks of the multimem push (0 = one per SM; 16 already reach the "
                         "link rate, and the push shares the GPU with a product)")
    ap.add_argument("--gemm-ctas", type=int, default=0,
                    help="CTAs the GEMM may use (0 = one per SM); fewer leaves SMs to the broadcast kernels")
    ap.add_argument("--m-total", type=int, default=M_TOTAL,
                    help="rows of A (default: the benchmark's 131072; smaller only for profiler captures)")
    args = ap.parse_args()
    if args.m_total != M_TOTAL:
        M_TOTAL = args.m_total
        WORKLOAD = WORKLOAD.replace("M=131072", f"M={M_TOTAL} (reduced for profiling)")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
