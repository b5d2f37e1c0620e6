"""Parity of reduce_sum / reduce_max / reduce_mean over adjacent axes against the CPU oracle, through the C ABI.
Bounds of the path: 1e-4 for fp32, 1e-2 for 16-bit storage (both metrics of conftest.assert_close); max is
exact in every type (it selects an input)."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu

TOL = {"F32": 1e-4, "BF16": 1e-2, "F16": 1e-2}


def _to_dev(ops, store, dtype):
    import torch
    raw = torch.from_numpy(store.view(np.int16) if store.dtype != np.float32 else store).cuda()
    return raw.view(ops.TORCH_DTYPE[dtype]) if store.dtype != np.float32 else raw


def _to_host_f32(O, t, dtype):
    import torch
    c = t.cpu()
    if dtype == O.F32:
        return c.numpy()
    return O.to_f32(c.view(torch.int16).numpy().view(np.uint16 if dtype == O.BF16 else np.float16), dtype)


CASES = [
    ((7, 13), [1]), ((7, 13), [0]), ((1, 1), [-1]), ((3, 1000), [-1]), ((5, 4096), [1]), ((2, 20000), [1]),
    ((33, 17, 9), [1]), ((33, 17, 9), [0]), ((33, 17, 9), [1, 2]), ((33, 17, 9), [0, 1]), ((33, 17, 9), [0, 1, 2]),
    ((4, 6, 100, 3), [2]), ((1000, 3), [0]), ((2, 300, 64), [-2]), ((64, 2049), [1]),
]


@pytest.mark.parametrize("dtype_name", ["F32", "BF16", "F16"])
@pytest.mark.parametrize("op", ["sum", "max", "mean"])
@pytest.mark.parametrize("shape,axes", CASES)
def test_reduce_matches_oracle(ops, cgb, oracle, dtype_name, op, shape, axes):
    import torch
    O = oracle
    dtype = getattr(cgb.capi, dtype_name)
    rng = np.random.default_rng(abs(hash((shape, tuple(axes)))) % (1 << 31))
    # a non-zero mean, so that sums do not sit at a cancellation point where only absolute error means anything
    xs = O.to_storage(rng.standard_normal(shape, dtype=np.float32) + 0.5, dtype)
    xd = _to_dev(ops, xs, dtype)
    for keep in (False, True):
        want = O.to_f32(O.reduce(xs, dtype, op, axes, keep), dtype)
        got_t = ops.reduce(xd, op, axes, keep_dims=keep)
        torch.cuda.synchronize()
        ax = {a % len(shape) for a in axes}
        assert tuple(got_t.shape) == tuple(1 if i in ax else d for i, d in enumerate(shape) if keep or i not in ax)
        want = want.reshape(tuple(got_t.shape))   # (the oracle's storage conversion turns a 0-d result into one element)
        got = _to_host_f32(O, got_t, dtype).reshape(tuple(got_t.shape))
        if op == "max":
            assert np.array_equal(got, want), f"reduce_max {shape} {axes}"
        else:
            assert_close(got, want, TOL[dtype_name], f"reduce_{op} {dtype_name} {shape} axes {axes}")


def test_reduce_full_size_rows(ops, cgb, oracle):
    """[32768, 4096] bf16 (the row-reduction configuration's shape), last axis: sampled rows against the oracle, and
    sum == mean * cols up to the rounding of each."""
    import torch
    O = oracle
    rows, cols = 32768, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(rows, cols, device="cuda", generator=g) + 0.25).to(torch.bfloat16)
    s, m, mx = (ops.reduce(x, op, [1]) for op in ("sum", "mean", "max"))
    torch.cuda.synchronize()
    assert ops.last_device_error() == 0
    pick = [0, 1, 4097, 20000, rows - 1]
    xs = x[pick].cpu().view(torch.int16).numpy().view(np.uint16)
    for t, op in ((s, "sum"), (m, "mean"), (mx, "max")):
        got = O.to_f32(t[pick].cpu().view(torch.int16).numpy().view(np.uint16), O.BF16)
        want = O.to_f32(O.reduce(xs, O.BF16, op, [1]), O.BF16)
        if op == "max":
            assert np.array_equal(got, want)
        else:
            assert_close(got, want, 1e-2, f"full-size reduce_{op}")
    assert torch.equal(mx, x.max(dim=1).values)
    assert torch.allclose(s.float(), m.float() * cols, rtol=2e-2, atol=1.0)


def test_reduce_edge_cases(ops, cgb):
    import torch
    capi = cgb.capi
    L = cgb.lib()
    x = torch.ones(4, 8, device="cuda")
    out = torch.full((4,), 7.0, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    assert L.cg_b200_reduce(capi.F32, 0, p(x), p(out), 0, 8, 1, None) == capi.OK          # no rows: nothing written
    assert L.cg_b200_reduce(capi.F32, 0, p(x), p(out), 4, 8, 0, None) == capi.OK
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full((4,), 7.0, device="cuda"))
    assert L.cg_b200_reduce(capi.F32, 0, p(x), p(out), 4, 0, 1, None) == capi.ERR_INVALID_ARG
    assert L.cg_b200_reduce(capi.F32, 3, p(x), p(out), 4, 8, 1, None) == capi.ERR_INVALID_ARG
    assert L.cg_b200_reduce(capi.F32, 0, None, p(out), 4, 8, 1, None) == capi.ERR_NULL_POINTER
    # max ignores NaN operands; a sum does not
    y = torch.tensor([[1.0, float("nan"), 3.0], [float("-inf"), -2.0, float("nan")]], device="cuda")
    assert torch.equal(ops.reduce(y, "max", [1]), torch.tensor([3.0, -2.0], device="cuda"))
    assert torch.isnan(ops.reduce(y, "sum", [1])).all()
    # an unaligned row start (offset view): the 16-byte path must not be taken blindly
    z = torch.arange(0, 4 * 37 + 1, device="cuda", dtype=torch.float32)[1:].view(4, 37)
    assert torch.equal(ops.reduce(z.contiguous(), "sum", [1]), z.sum(dim=1))
    zz = torch.arange(0, 4 * 37 + 1, device="cuda", dtype=torch.float32)
    out2 = torch.empty(4, device="cuda")
    assert L.cg_b200_reduce(capi.F32, 0, C.c_void_p(zz.data_ptr() + 4), p(out2), 4, 37, 1, None) == capi.OK
    torch.cuda.synchronize()
    assert torch.equal(out2, z.sum(dim=1))
    with pytest.raises(ValueError):
        ops.reduce(torch.ones(2, 3, 4, device="cuda"), "sum", [0, 2])
