#!/usr/bin/env python
"""Benchmark of the dense-GEMM hot path.

    python bench.py --gpus N --steps K --warmup W            (our CUDA path)
    python bench.py --impl reference --gpus N --steps K ...  (CPU baseline arm)

Workload: the row-sharded tall GEMM of the benchmark configurations, fp16
inputs / fp32 accumulate / fp32 C, M=131072, K=4096, N=4096, A split by rows
across the N ranks (one process per GPU), B held by rank 0 and replicated over
NVLink inside every step when N > 1: the product kernel itself pushes B through
NVSwitch (multimem stores) and multiplies the column slabs as they arrive
(gonngpu_gemm_f16_sharded).  One "step" is one full product.

Inputs are the seeded synthetic matrices of the benchmark definition:
numpy.random.default_rng(4), float64 normal draws scaled by 1/sqrt(K), A first,
then B, cast to float32; both arms multiply the same values.

`value` is device-timed with the operands already resident in HBM as fp16;
`e2e` is the same product through the handle-based C ABI from page-locked host
memory (float32 in, float32 out, copies and the fp32->fp16 pre-pass included).
At N=1 the line also carries the 8192^3 mixed-precision product (`c4`) and the
4096^2 transpose (`transpose_4096`).
"""
import argparse
import json
import os
import sys
import threading
import time

if "--impl" in sys.argv and "reference" in sys.argv:
    # The CPU arm uses every core it may run on, whatever the launcher exported
    # (torch.distributed.run sets OMP_NUM_THREADS=1); must happen before numpy loads its BLAS.
    _n = str(len(os.sched_getaffinity(0)))
    os.environ["OMP_NUM_THREADS"] = _n
    os.environ["OPENBLAS_NUM_THREADS"] = _n
    os.environ["MKL_NUM_THREADS"] = _n

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "go-nngpu_b200"))
sys.path.insert(0, ROOT)

M_TOTAL, K_DIM, N_DIM = 131072, 4096, 4096
SEED = 4
WORKLOAD = "row-sharded GEMM fp16-in/fp32-acc M=131072 K=4096 N=4096 (A rows split, B replicated)"
METRIC = "GEMM TFLOP/s"
GEN_CHUNK = 4096  # rows drawn at a time (the stream is the same as one draw of the whole matrix)


from sharding import shard_rows  # go-nngpu_b200/sharding.py  # noqa: E402


def draw_inputs(lo, hi, a_out=None, m_total=None):
    """The benchmark's A[lo:hi] and B as float32: default_rng(SEED), A drawn first (all of it, so
    that B is the same matrix on every rank and in both arms), then B.  `a_out`: float32 array
    of (hi - lo, K) to fill (page-locked memory of the end-to-end leg), else one is allocated."""
    m_total = M_TOTAL if m_total is None else m_total
    rng = np.random.default_rng(SEED)
    scale = 1.0 / np.sqrt(K_DIM)
    A = a_out if a_out is not None else np.empty((hi - lo, K_DIM), np.float32)
    for r0 in range(0, m_total, GEN_CHUNK):
        r1 = min(r0 + GEN_CHUNK, m_total)
        x = rng.standard_normal((r1 - r0, K_DIM))
        s0, s1 = max(r0, lo), min(r1, hi)
        if s0 < s1:
            np.multiply(x[s0 - r0:s1 - r0], scale, out=A[s0 - lo:s1 - lo], casting="same_kind")
    B = (rng.standard_normal((K_DIM, N_DIM)) * scale).astype(np.float32)
    return A, B


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
        self.power, self.power_limit = [], None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            try:
                self.power_limit = pynvml.nvmlDeviceGetEnforcedPowerLimit(self.h) / 1000.0
            except Exception:
                pass
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
            # not throttling, but reasons why a clock may sit below its maximum: somebody's
            # application-clock setting, a sync-boost group
            getattr(nv, "nvmlClocksEventReasonApplicationsClocksSetting", 0x2): "applications_clocks_setting",
            getattr(nv, "nvmlClocksEventReasonSyncBoost", 0x10): "sync_boost",
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
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            time.sleep(0.01)

    def result(self):
        self.stop_flag = True
        self.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples),
                "power_w": float(np.median(self.power)) if self.power else None,
                "power_limit_w": self.power_limit}


def use_all_cores():
    """Sets the BLAS pool to every core this process may run on and returns that count."""
    n = len(os.sched_getaffinity(0))
    try:
        from threadpoolctl import threadpool_limits, threadpool_info
        threadpool_limits(limits=n, user_api="blas")
        got = [p.get("num_threads", 0) for p in threadpool_info() if p.get("user_api") == "blas"]
        return int(max(got)) if got else n
    except Exception:
        return n


def f16_as_f64(x):
    return x.astype(np.float16).astype(np.float64)


def cpu_gemm_rate(A32, B32):
    """float64 product of the given rows of A by B (already rounded to fp16 values, as the GPU
    path multiplies them) on the host cores, numpy / OpenBLAS: the stand-in for gonum's
    mat.Dense.Mul, which is not installable here.  Returns (TFLOP/s, seconds)."""
    A, B = f16_as_f64(A32), f16_as_f64(B32)
    t0 = time.perf_counter()
    C = A @ B
    dt = time.perf_counter() - t0
    assert np.isfinite(C[0, 0])
    return 2.0 * A.shape[0] * K_DIM * N_DIM / dt / 1e12, dt


CPU_NOTE = ("float64 numpy/OpenBLAS; stand-in for gonum mat.Dense.Mul (Go and gonum are not installed); "
            "the first rows of the same seeded A, the same B")


def run_reference(args, rank):
    """CPU arm: the float64 GEMM on all host cores over a bounded row sample of the workload
    (the first rows of the same A, the same B)."""
    if rank != 0:
        return
    cores = use_all_cores()
    max_rows = min(32768, M_TOTAL)
    A32, B32 = draw_inputs(0, max_rows)
    rate, dt = cpu_gemm_rate(A32[:256], B32)
    # size the sample so that steps + warmup fit in about two minutes
    budget = 120.0 / max(args.steps + args.warmup, 1)
    rows = int(min(max_rows, max(256, 256 * budget / max(dt, 1e-6)))) // 128 * 128
    A, B = f16_as_f64(A32[:rows]), f16_as_f64(B32)
    for _ in range(args.warmup):
        A @ B
    t0 = time.perf_counter()
    for _ in range(args.steps):
        A @ B
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    val = 2.0 * rows * K_DIM * N_DIM / dt / 1e12
    sample = f"{rows} of {M_TOTAL} rows per step ({CPU_NOTE})"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def bind_near_gpu(local_rank):
    """Runs this process (and places the page-locked memory it allocates next) on the CPUs of the
    NUMA node the GPU hangs off, so that the ranks' host copies do not all cross one socket's
    memory.  Best effort: without the sysfs entries nothing changes."""
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(local_rank)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return node
    except Exception:
        pass
    return None


def open_exchange(args, torch, dist, g, dev, rank, world):
    """Sets up how B reaches the other ranks inside a step.  Returns a dict with `step_fn`
    pieces; the transport falls back to NCCL's broadcast when symmetric memory is unavailable."""
    from replicate import Replicator, ShardedProduct, open_symmetric
    slot_bytes = 2 * K_DIM * N_DIM
    want = args.transport
    res, why = None, ""
    if want in ("fused", "kernels"):
        try:
            buf, hdl, ctrl = open_symmetric(torch, dist, dev, slot_bytes, require_multicast=(want == "kernels"))
            mc = int(hdl.multicast_ptr) or None
            views = [buf[i * slot_bytes:(i + 1) * slot_bytes].view(torch.float16).view(K_DIM, N_DIM)
                     for i in range(2)]
            if want == "fused":
                obj = ShardedProduct(g, world, rank, 0, buf.data_ptr(), int(hdl.buffer_ptrs_dev), mc,
                                     K_DIM, N_DIM, args.first_group)
                label = "fused into the product kernel, " + ("multimem stores" if mc else "peer stores")
            else:
                obj = Replicator(g, world, rank, 0, int(hdl.buffer_ptrs_dev), mc, slot_bytes, ctrl, 32)
                label = "send and wait kernels (multimem stores), then the product"
            res = {"kind": want, "obj": obj, "views": views, "buf": buf, "hdl": hdl, "label": label}
        except Exception as e:  # noqa: BLE001 - any failure means "take the NCCL broadcast"
            why = f"{type(e).__name__}: {e}"
    ok = torch.tensor([1 if (res is not None or want == "nccl") else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    if int(ok[0]) == 0 or want == "nccl":
        if rank == 0 and why:
            print(f"[bench] symmetric memory unavailable, using the NCCL broadcast: {why}",
                  file=sys.stderr, flush=True)
        return {"kind": "nccl", "label": "NCCL broadcast, then the product"}
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
    numa = bind_near_gpu(local_rank) if world > 1 else None
    L = g.lib()
    assert L.gonngpu_set_device(local_rank) == 0, "no usable B200 for this rank"
    dev = torch.device("cuda", local_rank)
    stream = torch.cuda.ExternalStream(L.gonngpu_stream(), device=dev)
    lo, hi = shard_rows(M_TOTAL, world, rank)
    rows = hi - lo

    # ---- inputs: this rank's rows of A and all of B, in page-locked memory (the e2e leg reads them there)
    # (with several ranks, rank 0 keeps all of A: it also drives gonngpu_matmul_sharded over every GPU)
    whole = world > 1 and rank == 0 and not args.no_e2e
    hA_all, pA = g.pinned_array((M_TOTAL if whole else rows, K_DIM))
    hB, pB = g.pinned_array((K_DIM, N_DIM))
    hB[...] = draw_inputs(0 if whole else lo, M_TOTAL if whole else hi, a_out=hA_all)[1]
    hA = hA_all[lo:hi] if whole else hA_all

    with torch.cuda.stream(stream):
        L.gonngpu_set_blocking(0)
        A32 = torch.empty((rows, K_DIM), device=dev, dtype=torch.float32)
        A32.copy_(torch.from_numpy(hA), non_blocking=True)
        B32 = torch.empty((K_DIM, N_DIM), device=dev, dtype=torch.float32)
        B32.copy_(torch.from_numpy(hB), non_blocking=True)
        A16 = torch.empty((rows, K_DIM), device=dev, dtype=torch.float16)
        B16 = torch.empty((K_DIM, N_DIM), device=dev, dtype=torch.float16)
        C = torch.empty((rows, N_DIM), device=dev, dtype=torch.float32)
        g.convert_f16_device(A32.data_ptr(), rows, K_DIM, A16.data_ptr(), K_DIM)
        # every rank converts its own copy of B (same seed): rank 0's is the one that travels, the
        # others' only serve to check, bit for bit, what arrived
        g.convert_f16_device(B32.data_ptr(), K_DIM, N_DIM, B16.data_ptr(), N_DIM)
        stream.synchronize()
        del A32

        ex = open_exchange(args, torch, dist, g, dev, rank, world) if world > 1 else {"kind": "none", "label": "none"}
        Bdst = torch.zeros((K_DIM, N_DIM), device=dev, dtype=torch.float16) if ex["kind"] == "nccl" else None
        if Bdst is not None and rank == 0:
            Bdst.copy_(B16)

        def product(b_ptr):
            g.gemm_f16_device(A16.data_ptr(), (rows, K_DIM), K_DIM, False, b_ptr, (K_DIM, N_DIM), N_DIM,
                              False, C.data_ptr(), N_DIM)

        def step():
            kind = ex["kind"]
            if kind == "none":
                product(B16.data_ptr())
            elif kind == "fused":
                ex["obj"].step(A16.data_ptr(), rows, K_DIM, C.data_ptr(), N_DIM,
                               b_src_ptr=B16.data_ptr() if rank == 0 else None)
            elif kind == "kernels":
                slot = ex["obj"].replicate(B16.data_ptr() if rank == 0 else None)
                product(ex["views"][slot].data_ptr())
            else:
                dist.broadcast(Bdst, src=0, async_op=True).wait()   # orders the stream, does not block the host
                product(Bdst.data_ptr())

        def current_b():
            if ex["kind"] in ("fused", "kernels"):
                return ex["views"][ex["obj"].slot]
            return Bdst if Bdst is not None else B16

        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        g.synchronize()
        replica_ok = None
        if world > 1:
            okt = torch.tensor([1 if torch.equal(current_b(), B16) else 0], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            replica_ok = bool(int(okt[0]))
        # everything that takes a different time on every rank (NVML start-up, event creation)
        # comes before the barrier: a rank that starts late makes the others wait inside their
        # first step, and that wait would be counted as step time
        sampler = ClockSampler(local_rank)
        sampler.start()
        launches0 = g.stats()["kernel_launches"]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev[0].record(stream)
        for i in range(args.steps):
            step()
            ev[i + 1].record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        clocks = sampler.result()
        g.synchronize()  # surfaces any kernel status
        launches = g.stats()["kernel_launches"] - launches0
        total_ms = ev[0].elapsed_time(ev[-1])

        # the dominant kernel alone, B resident: its launch duration for the roofline (with one
        # rank the timed steps above are exactly that)
        resident_ms = total_ms / args.steps
        if world > 1:
            res_steps = max(3, min(args.steps, 20))
            product(current_b().data_ptr())
            kev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            kev[0].record(stream)
            for i in range(res_steps):
                product(current_b().data_ptr())
            kev[1].record(stream)
            stream.synchronize()
            g.synchronize()
            resident_ms = kev[0].elapsed_time(kev[1]) / res_steps
        # at N = 1 the step IS that kernel; with several ranks the step's kernel also moves B
        kernel_ms = total_ms / args.steps if world == 1 else resident_ms
        step()                      # C of a complete step for the parity check below
        stream.synchronize()
        g.synchronize()
        t = torch.tensor([total_ms, kernel_ms, resident_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, kernel_ms, resident_ms = float(t[0]), float(t[1]), float(t[2])
        ms_per_step = total_ms / args.steps
        value = 2.0 * M_TOTAL * K_DIM * N_DIM / (ms_per_step * 1e-3) / 1e12

        # ---- parity of the timed configuration against the CPU oracle: every rank checks sampled
        # rows of its own shard of C, its first and last row among them
        from oracle import oracle
        n_check = min(rows, max(256, -(-2048 // world)))
        rs = np.random.default_rng(1000 + rank)
        idx = np.unique(np.concatenate([[0, rows - 1], rs.choice(rows, size=n_check, replace=False)]))[:n_check + 2]
        Bh = current_b().float().cpu().numpy()
        ref = oracle.gemm_f64(hA[idx].astype(np.float16).astype(np.float32), Bh)
        got = C[torch.from_numpy(idx).to(dev)].cpu().numpy()
        check = float(oracle.rel_frobenius(got, ref))
        pt = torch.tensor([check, float(len(idx))], device=dev, dtype=torch.float64)
        if world > 1:
            mx = pt.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(pt, op=dist.ReduceOp.SUM)
            check, rows_checked = float(mx[0]), int(pt[1])
        else:
            rows_checked = len(idx)

        extras = {}
        if world == 1 and not args.no_extras:
            extras = run_extras(g, L, torch, dev, stream)

        # ---- end to end through the handle-based C ABI from page-locked host memory
        L.gonngpu_set_blocking(1)
        e2e = None
        if not args.no_e2e:
            del A16, C
            e2e = run_e2e(args, g, L, torch, dist, dev, rank, world, rows, hA, hB)
            if world > 1:
                one_call = run_e2e_one_call(args, g, L, torch, dist, dev, rank, world, hA_all, hB)
                if rank == 0:
                    e2e = merge_e2e(e2e, one_call)
            if numa is not None:
                e2e["host_numa_node_rank0"] = numa

    if rank == 0:
        report(args, g, world, rows, total_ms, kernel_ms, resident_ms, ms_per_step, value, clocks, launches,
               check, rows_checked, e2e, ex["label"], replica_ok, extras, hA, hB)
    for p in (pA, pB):
        L.gonngpu_host_free(p)
    if world > 1:
        dist.destroy_process_group()


def run_extras(g, L, torch, dev, stream):
    """Two more configurations of the benchmark set on one GPU, device-timed with CUDA events:
    the 8192^3 mixed-precision product through the handle API, once with the fp32 -> fp16
    conversion of both operands inside every call (fresh contents) and once with the converted
    operands cached; and the 4096^2 float32 transpose over a working set larger than L2."""
    peaks = load_peaks()
    out = {}
    n = 8192
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    s = 1.0 / np.sqrt(n)
    A = torch.randn((n, n), generator=gen, device=dev, dtype=torch.float32) * s
    B = torch.randn((n, n), generator=gen, device=dev, dtype=torch.float32) * s
    Cc = torch.empty((n, n), device=dev, dtype=torch.float32)
    a, b, c = (g.Buffer.wrap(t.data_ptr(), t.numel() * 4, t) for t in (A, B, Cc))
    reps = 50

    def timed(fresh):
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        for _ in range(5):
            g.matmul_ex(a, (n, n), False, b, (n, n), False, c, (n, n), precision=g.FP16_RN)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            if fresh:
                L.gonngpu_mark_modified(a.handle)
                L.gonngpu_mark_modified(b.handle)
            g.matmul_ex(a, (n, n), False, b, (n, n), False, c, (n, n), precision=g.FP16_RN)
        e1.record(stream)
        stream.synchronize()
        g.synchronize()
        return e0.elapsed_time(e1) / reps, sampler.result()

    ms_cached, clk = timed(False)
    ms_fresh, _ = timed(True)
    flops = 2.0 * n ** 3
    out["c4"] = {
        "workload": "8192^3 fp16-in/fp32-acc through gonngpu_matmul_ex(FP16_RN), float32 operands on the device",
        "launches": reps, "ms": ms_cached, "tflops": flops / ms_cached / 1e9,
        "frac": flops / ms_cached / 1e9 / peaks["burst"],
        "ms_with_conversion": ms_fresh, "tflops_with_conversion": flops / ms_fresh / 1e9,
        "frac_with_conversion": flops / ms_fresh / 1e9 / peaks["burst"],
        "peak": peaks["burst"], "peak_source": f"{peaks['source']} cuBLAS bf16 (burst)", "clocks": clk,
        "note": "ms: converted operands cached between calls; ms_with_conversion: both operands marked "
                "modified before every call, so each call converts 2 x 256 MiB to fp16 first",
    }
    for x in (a, b, c):
        x.release()
    del A, B, Cc
    # transpose: four input/output pairs in rotation = 512 MiB, four times the L2
    m = 4096
    ins = [torch.randn((m, m), generator=gen, device=dev, dtype=torch.float32) for _ in range(4)]
    outs = [torch.empty((m, m), device=dev, dtype=torch.float32) for _ in range(4)]
    hi_ = [g.Buffer.wrap(t.data_ptr(), t.numel() * 4, t) for t in ins]
    ho_ = [g.Buffer.wrap(t.data_ptr(), t.numel() * 4, t) for t in outs]
    for i in range(8):
        g.transpose(hi_[i % 4], (m, m), ho_[i % 4])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(100):
        g.transpose(hi_[i % 4], (m, m), ho_[i % 4])
    e1.record(stream)
    stream.synchronize()
    g.synchronize()
    ms = e0.elapsed_time(e1) / 100
    exact = bool(torch.equal(outs[3], ins[3].t()))
    gbs = 2.0 * m * m * 4 / (ms * 1e-3) / 1e9
    out["transpose_4096"] = {"ms": ms, "gbs": gbs, "frac": gbs / peaks["hbm_gbs"], "peak": peaks["hbm_gbs"],
                             "peak_source": f"{peaks['source']} copy bandwidth", "launches": 100,
                             "working_set": "4 input/output pairs in rotation, 512 MiB", "bit_exact": exact}
    for x in hi_ + ho_:
        x.release()
    return out


def run_e2e(args, g, L, torch, dist, dev, rank, world, rows, hA, hB):
    """The same product through create_gpu_buffer -> gonngpu_matmul_ex(FP16_RN) -> retrieve with
    host buffers in page-locked memory; with several ranks B crosses PCIe on rank 0 only and
    reaches the others over NVLink."""
    hC, pC = g.pinned_array((rows, N_DIM))
    e2e_steps = max(1, min(args.steps, 4))
    Bdev = bdev = None
    if world > 1:
        Bdev = torch.empty((K_DIM, N_DIM), device=dev, dtype=torch.float32)
        bdev = g.Buffer.wrap(Bdev.data_ptr(), Bdev.numel() * 4, Bdev)

    def e2e_step():
        a = g.Buffer.from_host(hA)
        c = g.Buffer.from_host(hC)
        if world > 1:
            if rank == 0:
                bdev.upload(hB)
            dist.broadcast(Bdev, src=0)
            L.gonngpu_mark_modified(bdev.handle)
            b = bdev
        else:
            b = g.Buffer.from_host(hB)
        g.matmul_ex(a, (rows, K_DIM), False, b, (K_DIM, N_DIM), False, c, (rows, N_DIM), precision=g.FP16_RN)
        c.retrieve_into(hC)
        for x in (a, c) + (() if world > 1 else (b,)):
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
    # the result that came back to the host, against the oracle (a few rows)
    from oracle import oracle
    idx = np.array([0, rows // 3, rows - 1])
    ref = oracle.gemm_f64(hA[idx].astype(np.float16).astype(np.float32),
                          hB.astype(np.float16).astype(np.float32))
    err = float(oracle.rel_frobenius(hC[idx], ref))
    if bdev is not None:
        bdev.release()
    L.gonngpu_host_free(pC)
    return {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
            "rank0_rows_rel_frobenius": err}


def run_e2e_one_call(args, g, L, torch, dist, dev, rank, world, hA_all, hB):
    """The same product as ONE library call of ONE process: rank 0 hands the whole host
    matrices to gonngpu_matmul_sharded, which splits the rows over all `world` GPUs, while the
    other ranks wait on the host (a gloo barrier: nothing of theirs runs on the GPUs meanwhile)."""
    cpu = dist.new_group(backend="gloo")
    torch.cuda.synchronize()
    dist.barrier(group=cpu)
    res = None
    if rank == 0:
        from oracle import oracle
        hC, pC = g.pinned_array((M_TOTAL, N_DIM))
        steps = max(1, min(args.steps, 4))
        g.matmul_sharded(hA_all, hB, hC, precision=g.FP16_RN, n_devices=world)   # warm-up: contexts, scratch
        s0 = g.stats()
        t0 = time.perf_counter()
        for _ in range(steps):
            g.matmul_sharded(hA_all, hB, hC, precision=g.FP16_RN, n_devices=world)
        dt = (time.perf_counter() - t0) / steps
        s1 = g.stats()
        idx = np.unique(np.concatenate([[r for d in range(world) for r in g.shard_plan(M_TOTAL, world, d)],
                                        np.random.default_rng(7).choice(M_TOTAL, 64, replace=False)]))
        idx = idx[idx < M_TOTAL]
        idx = np.unique(np.concatenate([idx, np.maximum(idx - 1, 0)]))     # first and last row of every shard
        ref = oracle.gemm_f64(hA_all[idx].astype(np.float16).astype(np.float32),
                              hB.astype(np.float16).astype(np.float32))
        res = {"value": 2.0 * M_TOTAL * K_DIM * N_DIM / dt / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int((s1["h2d_bytes"] - s0["h2d_bytes"]) // steps),
               "d2h_bytes_per_step": int((s1["d2h_bytes"] - s0["d2h_bytes"]) // steps),
               "ms_per_step": dt * 1e3, "steps": steps, "rows_checked": int(len(idx)),
               "rel_frobenius": float(oracle.rel_frobenius(hC[idx], ref)),
               "call": f"gonngpu_matmul_sharded(n_devices={world}) from one process"}
        L.gonngpu_host_free(pC)
        L.gonngpu_trim_cache()
        L.gonngpu_set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.barrier(group=cpu)
    return res


def merge_e2e(per_rank, one_call):
    """`e2e` is the faster of the two public ways to run the job on N GPUs; both are kept."""
    per_rank = dict(per_rank, call="create_gpu_buffer / gonngpu_matmul_ex / retrieve_gpu_buffer_data in every rank "
                                   "on its own rows (B over PCIe on rank 0, then NCCL broadcast)")
    best = one_call if one_call["value"] > per_rank["value"] else per_rank
    out = dict(best)
    out["one_process_call"] = one_call
    out["per_rank_calls"] = per_rank
    return out


# DRAM bytes of one GEMM launch measured with ncu (dram__bytes_read.sum +
# dram__bytes_write.sum) on the M=8192 case of this kernel: see profiles/.
NCU_TRAFFIC_M8192 = {"read": 178.2e6, "write": 99.7e6, "rows": 8192}


def traffic_estimate(rows):
    """Scales the captured traffic to `rows`: A and C grow with the rows, B (33.6 MB) does not."""
    b_bytes = 2.0 * K_DIM * N_DIM
    per_row = (NCU_TRAFFIC_M8192["read"] + NCU_TRAFFIC_M8192["write"] - b_bytes) / NCU_TRAFFIC_M8192["rows"]
    return per_row * rows + b_bytes


def report(args, g, world, rows, total_ms, kernel_ms, resident_ms, ms_per_step, value, clocks, launches, check,
           rows_checked, e2e, transport, replica_ok, extras, hA, hB):
    peaks = load_peaks()
    timed_s = total_ms * 1e-3
    peak_kind = "sustained" if timed_s >= 1.0 else "burst"
    achieved = 2.0 * rows * K_DIM * N_DIM / (kernel_ms * 1e-3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 in, f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": rows, "parallelism": f"row-shard x{world}",
                   "inputs": f"numpy default_rng({SEED}), normal(0, 1/sqrt(K)) drawn in float64, A then B",
                   "l2": "operands and result (>=384 MiB per GPU) exceed the 126 MB L2",
                   "b_replicated_in_step": world > 1, "b_transport": transport,
                   "b_replica_bit_exact": replica_ok},
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks[peak_kind], "unit": "TFLOP/s",
                     "frac": achieved / peaks[peak_kind], "traffic": traffic_estimate(rows),
                     "peak_source": f"{peaks['source']} cuBLAS bf16 ({peak_kind})",
                     # the same against the other figure of the pair (a 3.4 ms launch repeated for
                     # 0.2 s runs into the power cap like the sustained loop, not like a burst)
                     "frac_of_sustained_peak": achieved / peaks["sustained"],
                     "kernel_ms": kernel_ms,
                     "kernel": "gemm_f16_pair_kernel, one launch = one rank's shard"
                               + ("" if world == 1 else " (timed with B resident)")},
        "e2e": e2e,
        # the same job with B already resident on every GPU (slowest rank's kernel time only):
        # what the replication inside the step costs is the gap between this and `value`
        "value_b_resident": 2.0 * M_TOTAL * K_DIM * N_DIM / (resident_ms * 1e-3) / 1e12,
        "gpu_launches": int(launches),  # kernels of this library inside the timed region
        "parity_spot_check_rel_frobenius": check, "rows_checked": rows_checked,
        "parity_note": "sampled rows of every rank's C shard (first and last row included) against the "
                       "float64 oracle on the fp16-rounded inputs; tolerance 1e-2",
    }
    line.update(extras)
    if world == 1 and not args.no_cpu:
        cores = use_all_cores()
        _, dt = cpu_gemm_rate(hA[:512], hB)
        # size the sample for roughly 15 s of CPU work (bounded by the whole workload)
        rows_cpu = max(128, int(min(M_TOTAL, max(512, 512 * 15.0 / max(dt, 1e-6)))) // 128 * 128)
        rate, dt = cpu_gemm_rate(hA[:rows_cpu], hB)
        line["cpu_baseline"] = {
            "value": rate, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{rows_cpu} of {M_TOTAL} rows ({CPU_NOTE}), {dt:.1f} s"}
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
    ap.add_argument("--no-extras", action="store_true", help="skip the c4 / transpose sub-records")
    ap.add_argument("--transport", default="fused", choices=["fused", "kernels", "nccl"],
                    help="how B reaches the other ranks inside a step: fused = inside the product kernel "
                         "(default); kernels = this library's send and wait kernels ahead of the product; "
                         "nccl = NCCL's broadcast ahead of the product (the last two for comparison)")
    ap.add_argument("--first-group", type=int, default=0,
                    help="fused transport: 256-row tiles swept slab by slab while B arrives (0 = library's choice)")
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
