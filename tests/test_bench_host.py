"""Host side of bench.py: the seeded inputs and the CPU arm's thread count."""
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(m)
    finally:
        sys.argv = argv
    return m


def test_row_shards_of_the_seeded_inputs_equal_one_draw_of_the_whole_stream():
    b = _bench()
    b.M_TOTAL, b.K_DIM, b.N_DIM, b.GEN_CHUNK = 1000, 96, 40, 128
    rng = np.random.default_rng(b.SEED)
    s = 1.0 / np.sqrt(96)
    A = (rng.standard_normal((1000, 96)) * s).astype(np.float32)
    B = (rng.standard_normal((96, 40)) * s).astype(np.float32)
    for lo, hi in [(0, 1000), (0, 250), (250, 777), (900, 1000), (5, 5)]:
        a, bb = b.draw_inputs(lo, hi)
        assert np.array_equal(a, A[lo:hi]) and np.array_equal(bb, B)


def test_cpu_arm_uses_every_core_even_when_the_launcher_exports_one_thread():
    env = dict(os.environ, OMP_NUM_THREADS="1", OPENBLAS_NUM_THREADS="1")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--m-total", "1024"], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["value"] > 0
    assert line["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["higher_is_better"] is True
