"""Per-configuration timings of the dense path on one GPU (device-resident inputs).

    python microbench.py [--config c1|c2|c2nn|transpose|c3|c4|gonum|elementwise|all] [--iters N] [--cpu] [--fresh]

Prints one JSON line per measured operation: time, TFLOP/s or GB/s, and the
fraction of the measured peaks when MEASURED_PEAKS.json lies beside the
repository root.  Inputs are the seeded synthetic matrices of the benchmark
configurations (numpy PCG64).  Timing: `iters` asynchronous calls on the
library's stream between two synchronisations; operands rotate over several
buffer sets where one set would fit in the 126 MB L2.  By default the converted
operand planes of a GEMM are cached between calls (weights of a layer); with
--fresh both operands are marked modified before every call, so every call pays
its fp32 -> fp16 / tf32 pre-pass as a product of new activations does.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "go-nngpu_b200"))
import gonngpu as g  # noqa: E402


CPU_LEG = False
FRESH = False


def peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tensor": p["bf16_tflops"], "hbm": p["hbm_gbs"], "source": "measured"}
    return {"tensor": 1590.0, "hbm": 6650.0, "source": "fallback"}


def timed(fn, iters, sets=1):
    L = g.lib()
    L.gonngpu_set_blocking(1)
    for s in range(sets):
        fn(s)
    L.gonngpu_set_blocking(0)
    g.synchronize()
    t0 = time.perf_counter()
    for i in range(iters):
        fn(i % sets)
    g.synchronize()
    dt = (time.perf_counter() - t0) / iters
    L.gonngpu_set_blocking(1)
    return dt


def emit(name, dt, flops=None, bytes_=None, extra=None):
    pk = peaks()
    line = {"op": name, "us": round(dt * 1e6, 2)}
    if flops:
        line["tflops"] = round(flops / dt / 1e12, 2)
        line["frac_of_cublas_bf16_peak"] = round(flops / dt / 1e12 / pk["tensor"], 4)
    if bytes_:
        line["gb_per_s"] = round(bytes_ / dt / 1e9, 1)
        line["frac_of_hbm_copy_peak"] = round(bytes_ / dt / 1e9 / pk["hbm"], 4)
    line["peaks"] = pk["source"]
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def gemm_case(name, A, B, ta, tb, precision, iters):
    M = A.shape[1] if ta else A.shape[0]
    K = A.shape[0] if ta else A.shape[1]
    N = B.shape[0] if tb else B.shape[1]
    a, b = g.Buffer.from_host(A), g.Buffer.from_host(B)
    c = g.Buffer.empty(M * N * 4)
    def call(_):
        if FRESH:
            g.lib().gonngpu_mark_modified(a.handle)
            g.lib().gonngpu_mark_modified(b.handle)
        g.matmul_ex(a, A.shape, ta, b, B.shape, tb, c, (M, N), precision=precision)

    dt = timed(call, iters)
    extra = {"operands": "fresh (pre-pass inside every call)" if FRESH else "converted planes cached"}
    if precision == g.FP32_3XTF32:
        # tensor-pipe work per useful product, in tf32 MMAs: the single-CTA kernel issues three;
        # the CTA-pair kernel (products of 32 or more 256 x 256 tiles) one tf32 and two bf16 MMAs,
        # which take the time of two.  1100 TFLOP/s is the nominal dense tf32 rate.
        pair = M >= 256 and N >= 128 and -(-M // 256) * -(-N // 256) >= 32
        per = 2 if pair else 3
        issued = per * 2.0 * M * N * K / dt / 1e12
        extra.update({"tf32_equivalents_per_product": per, "tf32_equivalent_tflops": round(issued, 1),
                      "frac_of_nominal_tf32": round(issued / 1100.0, 3)})
    if CPU_LEG:
        # float64 product on the host cores: the comparator the benchmark names is gonum's
        # mat.Dense.Mul, which is not installed here; numpy/OpenBLAS float64 stands in for it
        A64 = (A.T if ta else A).astype(np.float64)
        B64 = (B.T if tb else B).astype(np.float64)
        t0 = time.perf_counter()
        ref = A64 @ B64
        cpu = time.perf_counter() - t0
        got = c.retrieve((M, N))
        err = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
        extra.update({"cpu_f64_ms": round(cpu * 1e3, 2), "cpu_tflops": round(2.0 * M * N * K / cpu / 1e12, 3),
                      "cpu_cores": os.cpu_count(), "cpu_impl": "numpy/OpenBLAS float64 (stand-in for gonum)",
                      "rel_frobenius_vs_f64": err})
    emit(name, dt, flops=2.0 * M * N * K, extra=extra)
    for x in (a, b, c):
        x.release()


def config1(iters):
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    B = rng.uniform(-1, 1, (1024, 1024)).astype(np.float32)
    gemm_case("c1 fp32 1024^3 A.B", A, B, False, False, g.FP32_3XTF32, iters)


def config2(iters, transposes=True):
    rng = np.random.default_rng(1)
    A = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    B = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    gemm_case("c2 fp32 4096^3 A.B", A, B, False, False, g.FP32_3XTF32, iters)
    if transposes:
        gemm_case("c2 fp32 4096^3 At.B", A, B, True, False, g.FP32_3XTF32, iters)
        gemm_case("c2 fp32 4096^3 A.Bt", A, B, False, True, g.FP32_3XTF32, iters)


def transpose_case(iters, n=4096):
    rng = np.random.default_rng(1)
    X = (rng.standard_normal((n, n)) / 64).astype(np.float32)
    sets = 4  # 4 x (64 + 64) MiB: no set is still in L2 when its turn comes again
    ins = [g.Buffer.from_host(X) for _ in range(sets)]
    outs = [g.Buffer.empty(X.nbytes) for _ in range(sets)]
    dt = timed(lambda s: g.transpose(ins[s], X.shape, outs[s]), iters, sets)
    emit(f"transpose {n}x{n} fp32", dt, bytes_=2.0 * X.nbytes)
    for x in ins + outs:
        x.release()


def config3(iters):
    rng = np.random.default_rng(2)
    dims = (784, 1024, 1024, 10)
    batch = 512
    X = rng.uniform(0, 1, (batch, dims[0])).astype(np.float32)
    Ws = [(rng.standard_normal((dims[i], dims[i + 1])) * np.sqrt(2.0 / dims[i])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(dims[i + 1], np.float32) for i in range(3)]
    dY3 = (rng.standard_normal((batch, dims[3])) * 1e-2).astype(np.float32)
    w = [g.Buffer.from_host(W) for W in Ws]
    b = [g.Buffer.from_host(x) for x in bs]
    h = [g.Buffer.from_host(X)] + [g.Buffer.empty(batch * dims[i + 1] * 4) for i in range(3)]
    dh = [g.Buffer.empty(batch * dims[i] * 4) for i in range(3)] + [g.Buffer.from_host(dY3)]
    dw = [g.Buffer.empty(W.nbytes) for W in Ws]
    db = [g.Buffer.empty(dims[i + 1] * 4) for i in range(3)]

    def step(_):
        for i in range(3):
            g.fused_linear_activation(h[i], batch, dims[i], w[i], dims[i + 1], b[i], 0 if i < 2 else -1, 0.0, h[i + 1])
        for i in (2, 1, 0):
            g.linear_backward(h[i], w[i], dh[i + 1], h[i + 1] if i < 2 else None, batch, dims[i], dims[i + 1],
                              dx=dh[i], dw=dw[i], db=db[i])

    dt = timed(step, iters)
    flops = sum(3 * 2.0 * batch * dims[i] * dims[i + 1] for i in range(3))
    emit("c3 MLP step 512x(784-1024-1024-10) fwd+bwd, 6 fused calls", dt, flops=flops)
    for x in w + b + h + dh + dw + db:
        x.release()
    # the same step as a caller of the layer stack drives it (C++ mirror of Sequential)
    import subprocess
    import tempfile
    pkg = os.path.join(HERE, "go-nngpu_b200")
    exe = os.path.join(tempfile.mkdtemp(), "mlp_step")
    subprocess.run(["g++", "-std=c++17", "-O2", "-o", exe, os.path.join(pkg, "host", "mlp_step.cpp"),
                    "-L" + pkg, "-lgonngpu_cuda", "-Wl,-rpath," + pkg], check=True)
    for fuse in ("1", "0"):
        print(subprocess.run([exe, str(iters), fuse], capture_output=True, text=True).stdout.strip(), flush=True)


def config4(iters):
    rng = np.random.default_rng(3)
    s = 1.0 / np.sqrt(8192)
    A = (rng.standard_normal((8192, 8192)) * s).astype(np.float32)
    B = (rng.standard_normal((8192, 8192)) * s).astype(np.float32)
    gemm_case("c4 fp16-in/fp32-acc 8192^3 A.B", A, B, False, False, g.FP16_RN, iters)


def gonum_facade(iters, n=4096):
    """GPUDense.Mul as a gonum user calls it: float64 matrices on the host in,
    float64 product out, everything inside the timed region.  `host` narrows and
    widens on the CPU (what FromGonum / ToGonum do in the reference, here with
    numpy's vector loops instead of per-element At calls); `device` sends the
    float64 data as it is and converts on the GPU."""
    rng = np.random.default_rng(1)
    A = rng.standard_normal((n, n)) / 64
    B = rng.standard_normal((n, n)) / 64
    pa, pb, pc = (g.pinned_array((n, n), np.float64)[0] for _ in range(3))
    pa[:], pb[:] = A, B
    a, b, c = g.Buffer.empty(n * n * 4), g.Buffer.empty(n * n * 4), g.Buffer.empty(n * n * 4)
    fa, fb, fc = (g.pinned_array((n, n), np.float32)[0] for _ in range(3))
    iters = max(3, iters // 10)

    def host_path():
        np.copyto(fa, pa, casting="same_kind")
        np.copyto(fb, pb, casting="same_kind")
        a.upload(fa)
        b.upload(fb)
        g.matmul(a, (n, n), b, (n, n), c, (n, n))
        c.retrieve_into(fc)
        np.copyto(pc, fc)

    def device_path():
        a.upload_f64(pa)
        b.upload_f64(pb)
        g.matmul(a, (n, n), b, (n, n), c, (n, n))
        c.retrieve_f64((n, n), out=pc)

    for name, fn in (("host conversion", host_path), ("device conversion", device_path)):
        fn()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        dt = (time.perf_counter() - t0) / iters
        emit(f"gonum facade {n}^3 float64 in/out, {name}", dt, flops=2.0 * n ** 3,
             extra={"pcie_bytes": (3 * n * n * 8) if fn is device_path else (3 * n * n * 4)})
    for x in (a, b, c):
        x.release()


def elementwise_family(iters, n=8192):
    """HBM-bound members of the family on [n, n] float32 (256 MiB per operand)."""
    rng = np.random.default_rng(6)
    X = rng.standard_normal((n, n)).astype(np.float32)
    a, b, c = g.Buffer.from_host(X), g.Buffer.from_host(X + np.float32(3.0)), g.Buffer.empty(X.nbytes)
    nb = float(X.nbytes)
    emit(f"add {n}x{n}", timed(lambda s: g.elementwise("add", a, b, c, X.shape), iters), bytes_=3 * nb)
    emit(f"scalar_multiply {n}x{n}", timed(lambda s: g.scalar_op("scalar_multiply", a, X.shape, 1.5, c), iters), bytes_=2 * nb)
    emit(f"sigmoid {n}x{n}", timed(lambda s: g.activation_forward("sigmoid", a, X.size, c), iters), bytes_=2 * nb)
    emit(f"gelu {n}x{n}", timed(lambda s: g.activation_forward("gelu", a, X.size, c), iters), bytes_=2 * nb)
    emit(f"gelu backward {n}x{n}", timed(lambda s: g.activation_backward("gelu", a, c, X.size, b), iters), bytes_=3 * nb)
    emit(f"softmax rows {n}x{n}", timed(lambda s: g.softmax_2d(a, n, n, c), iters), bytes_=2 * nb)
    emit(f"softmax rows {n * n // 16}x16", timed(lambda s: g.softmax_2d(a, n * n // 16, 16, c), iters), bytes_=2 * nb)
    emit(f"softmax rows {n * n // 10}x10", timed(lambda s: g.softmax_2d(a, n * n // 10, 10, c), iters),
         bytes_=2.0 * (n * n // 10) * 40)
    for x in (a, b, c):
        x.release()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--cpu", action="store_true",
                    help="also time the float64 product on the host cores and report the error against it")
    ap.add_argument("--fresh", action="store_true",
                    help="mark both GEMM operands modified before every call (pre-pass inside the timing)")
    args = ap.parse_args()
    global CPU_LEG, FRESH
    CPU_LEG = args.cpu
    FRESH = args.fresh
    assert g.lib().gonngpu_set_device(0) == 0, "no usable B200"
    run = {"c1": lambda: config1(args.iters), "c2": lambda: config2(args.iters),
           "c2nn": lambda: config2(args.iters, transposes=False),
           "transpose": lambda: transpose_case(args.iters), "c3": lambda: config3(args.iters),
           "c4": lambda: config4(args.iters), "gonum": lambda: gonum_facade(args.iters),
           "elementwise": lambda: elementwise_family(args.iters)}
    names = ["c1", "c2", "transpose", "c3", "c4"] if args.config == "all" else [args.config]
    for n in names:
        run[n]()


if __name__ == "__main__":
    main()
