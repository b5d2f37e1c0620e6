"""CPU oracle of the pre-LN encoder block: composition of the oracle's ops, every op result rounded
to the storage type (each Tensor-IR op produces a tensor of that type).

TEST INFRASTRUCTURE ONLY. Dataflow: the reference's transformer benchmark graph
(benchmarks/benchmark_transformer.py:98-119); PARITY UNPINNED - the reference never executes it.
"""
import math

import numpy as np

from . import oracle as O


def encoder_block(x, w_qkv, w_o, w_1, b_1, w_2, b_2, n_heads, dtype, eps=1e-5):
    """x: [B, S, D] in storage representation (`dtype`); weights [in, out]. Returns y [B, S, D]."""
    B, S, D = x.shape
    H, dh, F = n_heads, D // n_heads, w_1.shape[1]
    rows = B * S
    x2 = np.ascontiguousarray(x.reshape(rows, D))
    ln1 = O.layernorm(x2, dtype, None, None, eps)
    qkv = O.gemm(O.make_gemm_desc(rows, 3 * D, D, dtype, dtype), ln1, w_qkv).reshape(rows, 3 * D)
    ctx = np.zeros((rows, D), dtype=x2.dtype)
    for b in range(B):
        blk = qkv[b * S:(b + 1) * S]
        for h in range(H):
            q = np.ascontiguousarray(blk[:, h * dh:(h + 1) * dh])
            k = np.ascontiguousarray(blk[:, D + h * dh:D + (h + 1) * dh])
            v = np.ascontiguousarray(blk[:, 2 * D + h * dh:2 * D + (h + 1) * dh])
            sc = O.gemm(O.make_gemm_desc(S, S, dh, dtype, dtype, epilogue="scale", alpha=1.0 / math.sqrt(dh),
                                         b_transposed=1), q, k).reshape(S, S)
            pr = O.softmax(sc, dtype)
            ctx[b * S:(b + 1) * S, h * dh:(h + 1) * dh] = O.gemm(O.make_gemm_desc(S, dh, S, dtype, dtype), pr, v).reshape(S, dh)
    hres = O.gemm(O.make_gemm_desc(rows, D, D, dtype, dtype, epilogue="residual"), ctx, w_o, residual=x2).reshape(rows, D)
    ln2 = O.layernorm(hres, dtype, None, None, eps)
    ff = O.gemm(O.make_gemm_desc(rows, F, D, dtype, dtype, epilogue="bias_gelu_tanh"), ln2, w_1, bias=b_1).reshape(rows, F)
    y = O.gemm(O.make_gemm_desc(rows, D, F, dtype, dtype, epilogue="bias_residual"), ff, w_2, bias=b_2, residual=hres)
    return y.reshape(B, S, D)
