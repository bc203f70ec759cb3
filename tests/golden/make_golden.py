"""Generates tests/golden/oracle_kats.npz from the CPU oracle.

The reference (Go + Metal) cannot run outside macOS, so these vectors come
from the oracle's restatement of it (oracle/oracle.c); the vectors that the
reference's own tests hold are kept separately in reference_kats.json.  The
cases here are chosen so that the expected output is EXACT in every precision
path (small integers, permutations, powers of two), which makes them
known-answer tests rather than tolerance tests, plus a few seeded float cases
stored with their float64 reference.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402


def main():
    rng = np.random.default_rng(20240607)
    out = {}

    # Integer-valued GEMMs: |entries| <= 4 and K <= 96, so every product and
    # partial sum is an integer below 2^11: exact in fp16-in/fp32-acc and in tf32.
    for name, (m, n, k) in {"int_a": (5, 7, 3), "int_b": (130, 70, 96), "int_c": (64, 10, 33)}.items():
        A = rng.integers(-4, 5, (m, k)).astype(np.float32)
        B = rng.integers(-4, 5, (k, n)).astype(np.float32)
        out[f"{name}_A"], out[f"{name}_B"] = A, B
        out[f"{name}_C"] = oracle.gemm_f64_naive(A, B).astype(np.float32)

    # Permutation matrix times a matrix of distinct values: reveals any index mix-up.
    perm = rng.permutation(96)
    P = np.zeros((96, 96), dtype=np.float32)
    P[np.arange(96), perm] = 1.0
    V = (np.arange(96 * 40, dtype=np.float32).reshape(96, 40) % 2048) - 1024
    out["perm_P"], out["perm_V"] = P, V
    out["perm_C"] = oracle.gemm_f64_naive(P, V).astype(np.float32)

    # Transpose of a ragged matrix with special values (moves must be bit-exact).
    T = rng.standard_normal((37, 101)).astype(np.float32)
    T[0, 0], T[1, 2], T[3, 4], T[5, 6] = np.float32("nan"), np.float32("-0.0"), np.float32("inf"), np.float32(1e-42)
    out["tr_in"] = T
    out["tr_out"] = oracle.transpose(T)

    # Truncating fp16 conversion over the interesting ranges.
    x = np.concatenate([
        (rng.standard_normal(2000) * 10.0 ** rng.integers(-9, 6, 2000)),
        [0.0, -0.0, 65504.0, 65520.0, 70000.0, -70000.0, 6.1e-5, 6.0e-5, 5.96e-8, 2.9e-8, 1e-45, np.inf, -np.inf],
    ]).astype(np.float32)
    out["f16_in"] = x
    out["f16_trunc_out"] = oracle.f16_trunc(x)

    # Fused linear + bias + activation, every code the reference decodes plus identity.
    X = rng.uniform(-1, 1, (9, 20)).astype(np.float32)
    W = rng.uniform(-1, 1, (20, 13)).astype(np.float32)
    b = rng.uniform(-1, 1, 13).astype(np.float32)
    out["fl_X"], out["fl_W"], out["fl_b"] = X, W, b
    for act in (0, 1, 2, 3, 4, 9):
        out[f"fl_act{act}_f32"] = oracle.fused_linear_activation(X, W, b, act, 0.25)
        out[f"fl_act{act}_f64"] = oracle.fused_linear_activation_f64(X, W, b, act, 0.25)

    # alpha/beta GEMM and the four broadcast patterns.
    A = rng.integers(-3, 4, (17, 12)).astype(np.float32)
    B = rng.integers(-3, 4, (12, 21)).astype(np.float32)
    C0 = rng.integers(-3, 4, (17, 21)).astype(np.float32)
    out["ab_A"], out["ab_B"], out["ab_C0"] = A, B, C0
    out["ab_out"] = oracle.gemm_alpha_beta(A, B, C0, 0.5, -2.0)
    M = rng.standard_normal((6, 11)).astype(np.float32)
    row = rng.standard_normal((1, 11)).astype(np.float32)
    col = rng.standard_normal((6, 1)).astype(np.float32)
    out["bc_M"], out["bc_row"], out["bc_col"] = M, row, col
    out["bc_m_row"] = oracle.add_broadcast(M, row, (6, 11))[1]
    out["bc_row_m"] = oracle.add_broadcast(row, M, (6, 11))[1]
    out["bc_m_col"] = oracle.add_broadcast(M, col, (6, 11))[1]
    out["bc_col_m"] = oracle.add_broadcast(col, M, (6, 11))[1]
    out["colsum_in"] = M
    out["colsum_out"] = oracle.column_sum(M)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_kats.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
