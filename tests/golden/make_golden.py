"""Regenerates tests/golden/ref_kernels.npz from the reference project's own x86 kernels.

Needs oracle/_ref/libcg_ref.so, i.e. the reference tree at build time (`make -C oracle`).
The fixtures hold inputs and the outputs the reference's JIT kernels produced for them:
  add / relu(a*b)      benchmarks/benchmark_multithread.py:54-124
  relu(a*b+c)*0.5      same loop shape, emitter ops of include/cg/backend/x86/x86_emitter.hpp:90-119
  matmul (fma chain)   benchmarks/benchmark.py:326-438
plus the emitter-level known answers the reference's tests pin
(tests/correctness/correctness_tests.cpp:30-89: vaddps {1,2,3,4}+{10,20,30,40}, vmulps,
vfmadd231ps 1+2*3).
Run from the repo root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402


def main():
    out = {}
    rng = np.random.default_rng(1)
    n = 4096
    a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
    # edge values the relu/max semantics depend on
    a[:8] = [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 3.0]
    b[:8] = [1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, -0.0]
    c[:8] = [-0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0]
    out["ew_a"], out["ew_b"], out["ew_c"] = a, b, c
    out["ew_add"] = O.ref_binary(0, a, b)
    out["ew_relu_mul"] = O.ref_binary(1, a, b)
    out["ew_chain"] = O.ref_fma_relu_scale(a, b, c, 0.5)

    rng = np.random.default_rng(0)
    for tag, (M, K, N) in {"mm_small": (24, 40, 56), "mm_sq": (64, 64, 64), "mm_odd": (37, 129, 17)}.items():
        A = (rng.random((M, K), dtype=np.float32) * 2 - 1).astype(np.float32)
        B = (rng.random((K, N), dtype=np.float32) * 2 - 1).astype(np.float32)
        out[tag + "_A"], out[tag + "_B"], out[tag + "_C"] = A, B, O.ref_matmul(A, B)

    # the reference's emitter-level known answers, run through the same kernels
    ka = np.array([1, 2, 3, 4], dtype=np.float32)
    kb = np.array([10, 20, 30, 40], dtype=np.float32)
    out["kat_add"] = O.ref_binary(0, ka, kb)
    assert out["kat_add"].tolist() == [11, 22, 33, 44]
    out["kat_fma"] = O.ref_matmul(np.array([[2.0]], dtype=np.float32), np.array([[3.0]], dtype=np.float32))
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_kernels.npz"), **out)
    print("wrote ref_kernels.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
