"""The CPU oracle against the reference's own kernels: committed golden vectors, and the
reference emitter built into oracle/_ref when it is present. No GPU."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN)


def bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def chain(O, prog, n_in):
    return O.make_eltwise_desc(O.F32, prog, ["full"] * n_in)


PROG_CHAIN = [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu", ("imm", 0.5), "mul"]


def test_eltwise_matches_reference_kernels(oracle, gold):
    O = oracle
    a, b, c = gold["ew_a"], gold["ew_b"], gold["ew_c"]
    n = a.size
    add = O.eltwise(chain(O, [("input", 0), ("input", 1), "add"], 2), [a, b], n)
    assert np.array_equal(bits(add), bits(gold["ew_add"]))
    rm = O.eltwise(chain(O, [("input", 0), ("input", 1), "mul", "relu"], 2), [a, b], n)
    assert np.array_equal(bits(rm), bits(gold["ew_relu_mul"]))
    # relu written as max(x, 0): same operand order as the reference's vmaxps
    rm2 = O.eltwise(chain(O, [("input", 0), ("input", 1), "mul", ("imm", 0.0), "max"], 2), [a, b], n)
    assert np.array_equal(bits(rm2), bits(gold["ew_relu_mul"]))
    ch = O.eltwise(chain(O, PROG_CHAIN, 3), [a, b, c], n)
    assert np.array_equal(bits(ch), bits(gold["ew_chain"]))


def test_reference_known_answers(gold):
    # tests/correctness/correctness_tests.cpp:30-89 of the reference
    assert gold["kat_add"].tolist() == [11.0, 22.0, 33.0, 44.0]
    assert gold["kat_fma"].tolist() == [[6.0]]


@pytest.mark.parametrize("tag", ["mm_small", "mm_sq", "mm_odd"])
def test_gemm_matches_reference_fma_chain(oracle, gold, tag):
    O = oracle
    A, B, Cref = gold[tag + "_A"], gold[tag + "_B"], gold[tag + "_C"]
    M, K = A.shape
    N = B.shape[1]
    d = O.make_gemm_desc(M, N, K, O.F32, O.F32)
    C = O.gemm(d, A, B).reshape(M, N)
    assert np.array_equal(bits(C), bits(Cref))
    # transposed storage of B gives the same bits
    dt = O.make_gemm_desc(M, N, K, O.F32, O.F32, b_transposed=1)
    Ct = O.gemm(dt, A, np.ascontiguousarray(B.T)).reshape(M, N)
    assert np.array_equal(bits(Ct), bits(Cref))
    # and the double-accumulated variant stays within fp32 rounding of it
    C64 = O.gemm(d, A, B, acc64=True).reshape(M, N)
    assert np.abs(C64 - Cref).max() <= 1e-5 * max(1.0, np.abs(Cref).max())


def test_live_reference_if_built(oracle):
    O = oracle
    if not O.have_ref():
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(7)
    n = 1 << 16
    a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
    ref = O.ref_fma_relu_scale(a, b, c, 0.5, threads=3)
    mine = O.eltwise(chain(O, PROG_CHAIN, 3), [a, b, c], n)
    assert np.array_equal(bits(ref), bits(mine))
    A = (rng.random((33, 70), dtype=np.float32) * 2 - 1).astype(np.float32)
    B = (rng.random((70, 45), dtype=np.float32) * 2 - 1).astype(np.float32)
    d = O.make_gemm_desc(33, 45, 70, O.F32, O.F32)
    assert np.array_equal(bits(O.gemm(d, A, B).reshape(33, 45)), bits(O.ref_matmul(A, B)))


def test_eltwise_validation_and_broadcast(oracle):
    O = oracle
    assert O.lib().cgo_eltwise_validate(O.make_eltwise_desc(O.F32, ["add"], []), 0) != 0  # stack underflow
    assert O.lib().cgo_eltwise_validate(O.make_eltwise_desc(O.F32, [("input", 0), ("input", 0)], ["full"]), 1) != 0
    rows, inner = 5, 12
    x = np.arange(rows * inner, dtype=np.float32)
    r = np.arange(inner, dtype=np.float32) * 10
    col = np.arange(rows, dtype=np.float32) * 100
    s = np.array([0.25], dtype=np.float32)
    d = O.make_eltwise_desc(O.F32, [("input", 0), ("input", 1), "add", ("input", 2), "add", ("input", 3), "mul"],
                            ["full", "row", "col", "scalar"], inner=inner)
    y = O.eltwise(d, [x, r, col, s], x.size).reshape(rows, inner)
    expect = (x.reshape(rows, inner) + r[None, :] + col[:, None]) * 0.25
    assert np.array_equal(y, expect.astype(np.float32))
    assert O.eltwise(d, [x, r, col, s], 0).size == 0


def test_bf16_rounding_and_row_ops(oracle):
    O = oracle
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], dtype=np.float32)
    h = O.to_bf16(x)
    back = O.from_bf16(h)
    # 1 + 2^-8 is a tie and rounds to even (1.0); 1 + 3*2^-8 rounds up to 1 + 2^-6
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == 1.015625 and back[3] == -2.5
    rng = np.random.default_rng(3)
    xs = rng.standard_normal((7, 50), dtype=np.float32)
    sm = O.softmax(xs, O.F32)
    e = np.exp(xs.astype(np.float64) - xs.max(axis=1, keepdims=True))
    assert np.allclose(sm, e / e.sum(axis=1, keepdims=True), rtol=1e-6, atol=1e-9)
    g = rng.standard_normal(50, dtype=np.float32)
    b = rng.standard_normal(50, dtype=np.float32)
    ln = O.layernorm(xs, O.F32, g, b, eps=1e-5)
    x64 = xs.astype(np.float64)
    want = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    assert np.allclose(ln, want, rtol=1e-5, atol=1e-6)
    # fused form = the two ops with a storage-type tensor between them
    xb = O.to_bf16(xs)
    two = O.layernorm(O.softmax(xb, O.BF16), O.BF16)
    one = O.softmax_layernorm(xb, O.BF16)
    assert np.array_equal(two, one)
    # empty inputs are no-ops
    assert O.softmax(np.zeros((0, 8), dtype=np.float32), O.F32).shape == (0, 8)


def test_gemm_epilogues_and_batch(oracle):
    O = oracle
    rng = np.random.default_rng(5)
    Bt, M, N, K = 3, 9, 14, 11
    A = rng.standard_normal((Bt, M, K), dtype=np.float32)
    B = rng.standard_normal((K, N), dtype=np.float32)   # broadcast over batch
    bias = rng.standard_normal(N, dtype=np.float32)
    res = rng.standard_normal((Bt, M, N), dtype=np.float32)
    d = O.make_gemm_desc(M, N, K, O.F32, O.F32, epilogue="bias_residual", batch=Bt, bsb=0)
    C = O.gemm(d, A, B, bias=bias, residual=res, acc64=True).reshape(Bt, M, N)
    want = A.astype(np.float64) @ B + bias + res
    assert np.allclose(C, want, rtol=1e-5, atol=1e-5)
    d = O.make_gemm_desc(M, N, K, O.F32, O.F32, epilogue="bias_gelu_tanh", batch=Bt, bsb=0)
    C = O.gemm(d, A, B, bias=bias, acc64=True).reshape(Bt, M, N)
    z = A.astype(np.float64) @ B + bias
    gelu = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    assert np.allclose(C, gelu, rtol=1e-5, atol=1e-5)
    # row subset only touches those rows
    rows = np.array([1, 10, 26], dtype=np.int64)
    d = O.make_gemm_desc(M, N, K, O.F32, O.F32, batch=Bt, bsb=0)
    part = O.gemm(d, A, B, rows=rows).reshape(Bt * M, N)
    full = O.gemm(d, A, B).reshape(Bt * M, N)
    assert np.array_equal(part[rows], full[rows])
    mask = np.ones(Bt * M, dtype=bool)
    mask[rows] = False
    assert not part[mask].any()


def test_reduce_definitions_and_boxes(oracle):
    """reduce_sum / reduce_max / reduce_mean of the oracle against their definitions (src/ir/ops.cpp:74-102: axes,
    keep_dims, result dtype = operand dtype), and the [outer, reduce, inner] box the kernel is given."""
    from cantors_gift_b200 import ops
    O = oracle
    rng = np.random.default_rng(11)
    x = rng.standard_normal((3, 4, 5), dtype=np.float32)
    xs = O.to_storage(x, O.BF16)
    xf = O.to_f32(xs, O.BF16).astype(np.float64)
    for axes in ([0], [1], [2], [-1], [0, 1], [1, 2], [0, 1, 2]):
        for keep in (False, True):
            ax = tuple(axes)
            got = O.to_f32(O.reduce(xs, O.BF16, "sum", axes, keep), O.BF16)
            want = O.to_f32(O.to_storage(np.asarray(xf.sum(axis=ax, keepdims=keep), dtype=np.float32), O.BF16), O.BF16)
            assert np.array_equal(got.reshape(want.shape), want)
            got = O.to_f32(O.reduce(xs, O.BF16, "max", axes, keep), O.BF16)
            assert np.array_equal(got.reshape(xf.max(axis=ax, keepdims=keep).shape), xf.max(axis=ax, keepdims=keep).astype(np.float32))
    # max ignores NaN, sum does not
    y = np.array([[1.0, np.nan, 3.0]], dtype=np.float32)
    assert O.reduce(y, O.F32, "max", [1])[0] == 3.0 and np.isnan(O.reduce(y, O.F32, "sum", [1])[0])
    assert ops.reduce_box((3, 4, 5), [1]) == (3, 4, 5)
    assert ops.reduce_box((3, 4, 5), [-1]) == (12, 5, 1)
    assert ops.reduce_box((3, 4, 5), [0, 1]) == (1, 12, 5)
    assert ops.reduce_box((3, 4, 5), [2, 1, 0]) == (1, 60, 1)
    assert ops.reduce_box((3, 4, 5), [0, 2]) is None and ops.reduce_box((3, 4, 5), [3]) is None
