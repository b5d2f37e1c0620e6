"""Parity of the fused elementwise CUDA path against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PROG_CHAIN = [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu", ("imm", 0.5), "mul"]


def _run(ops, cgb, O, dtype, prog, arrays_f32, bcast, n, inner=1, round_each_op=0, offset=0):
    """arrays_f32: fp32 numpy inputs; returns (gpu result, oracle result) in storage representation."""
    import torch
    capi = cgb.capi
    store = [O.to_storage(a, dtype) for a in arrays_f32]
    want = O.eltwise(O.make_eltwise_desc(dtype, prog, bcast, inner, round_each_op), store, n)
    tdt = ops.TORCH_DTYPE[dtype]
    dev = []
    for s in store:
        raw = torch.from_numpy(s.view(np.int16) if s.dtype != np.float32 else s).cuda()
        t = raw.view(tdt) if s.dtype != np.float32 else raw
        if offset:  # misalign by `offset` elements
            buf = torch.empty(t.numel() + offset, dtype=tdt, device="cuda")
            buf[offset:].copy_(t)
            t = buf[offset:]
        dev.append(t)
    out_buf = torch.empty(n + offset, dtype=tdt, device="cuda")
    out = out_buf[offset:]
    ops.eltwise(capi.make_eltwise_desc(dtype, prog, bcast, inner, round_each_op), dev, out, n=n)
    torch.cuda.synchronize()
    got = out.cpu()
    got = got.view(torch.int16).numpy().view(want.dtype) if dtype != capi.F32 else got.numpy()
    return got, want


def _bits(a):
    """Bit patterns with every NaN mapped to one canonical pattern: IEEE 754 leaves the payload
    and sign of a generated NaN to the implementation (x86 keeps the input's, the GPU emits its
    own canonical one); everything else must match bit for bit."""
    if a.dtype == np.float32:
        b = a.view(np.uint32).copy()
        b[np.isnan(a)] = 0x7FC00000
        return b
    b = a.view(np.uint16).copy()
    f = a if a.dtype == np.float16 else (a.astype(np.uint32) << 16).view(np.float32)
    b[np.isnan(f)] = 0x7FC0
    return b


@pytest.mark.parametrize("n", [1, 3, 4, 5, 1023, 4096, (1 << 20) + 7])
def test_chain_fp32_bit_exact(ops, cgb, oracle, n):
    rng = np.random.default_rng(1)
    a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
    got, want = _run(ops, cgb, oracle, cgb.capi.F32, PROG_CHAIN, [a, b, c], ["full"] * 3, n)
    assert np.array_equal(_bits(got), _bits(want))


def test_chain_matches_reference_golden(ops, cgb, oracle):
    import os
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels.npz"))
    a, b, c = gold["ew_a"], gold["ew_b"], gold["ew_c"]
    F32 = cgb.capi.F32
    for prog, ins, key in [(PROG_CHAIN, [a, b, c], "ew_chain"),
                           ([("input", 0), ("input", 1), "add"], [a, b], "ew_add"),
                           ([("input", 0), ("input", 1), "mul", "relu"], [a, b], "ew_relu_mul"),
                           ([("input", 0), ("input", 1), "mul", ("imm", 0.0), "max"], [a, b], "ew_relu_mul")]:
        got, _ = _run(ops, cgb, oracle, F32, prog, ins, ["full"] * len(ins), a.size)
        assert np.array_equal(_bits(got), _bits(gold[key])), key


@pytest.mark.parametrize("offset", [1, 3])
def test_unaligned_pointers_take_scalar_path(ops, cgb, oracle, offset):
    rng = np.random.default_rng(2)
    n = 10007
    a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
    got, want = _run(ops, cgb, oracle, cgb.capi.F32, PROG_CHAIN, [a, b, c], ["full"] * 3, n, offset=offset)
    assert np.array_equal(_bits(got), _bits(want))


def test_interpreter_integer_exact_ops(ops, cgb, oracle):
    """A chain no compile-time program matches: add/sub/mul/max/min/neg/abs are exact."""
    rng = np.random.default_rng(3)
    n = 70001
    a, b, c, d = (rng.standard_normal(n, dtype=np.float32) for _ in range(4))
    prog = [("input", 0), ("input", 1), "sub", "abs", ("input", 2), "min", ("input", 3), "neg", "max",
            ("imm", 3.0), "mul", ("input", 0), "add"]
    got, want = _run(ops, cgb, oracle, cgb.capi.F32, prog, [a, b, c, d], ["full"] * 4, n)
    assert np.array_equal(_bits(got), _bits(want))


def test_broadcast_kinds(ops, cgb, oracle):
    rng = np.random.default_rng(4)
    for rows, inner in [(37, 24), (64, 1000), (5, 7)]:
        n = rows * inner
        x = rng.standard_normal(n, dtype=np.float32)
        r = rng.standard_normal(inner, dtype=np.float32)
        col = rng.standard_normal(rows, dtype=np.float32)
        s = np.array([1.5], dtype=np.float32)
        prog = [("input", 0), ("input", 1), "add", ("input", 2), "mul", ("input", 3), "sub"]
        got, want = _run(ops, cgb, oracle, cgb.capi.F32, prog, [x, r, col, s], ["full", "row", "col", "scalar"],
                         n, inner=inner)
        assert np.array_equal(_bits(got), _bits(want)), (rows, inner)


@pytest.mark.parametrize("dtype_name", ["BF16", "F16"])
@pytest.mark.parametrize("round_each_op", [0, 1])
def test_16bit_storage_exact_ops(ops, cgb, oracle, dtype_name, round_each_op):
    dtype = getattr(cgb.capi, dtype_name)
    rng = np.random.default_rng(5)
    n = 33333
    a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
    got, want = _run(ops, cgb, oracle, dtype, PROG_CHAIN, [a, b, c], ["full"] * 3, n, round_each_op=round_each_op)
    assert np.array_equal(_bits(got), _bits(want))


def test_transcendental_ops_within_fp32_tolerance(ops, cgb, oracle):
    from conftest import assert_close
    rng = np.random.default_rng(6)
    n = 50000
    x = rng.standard_normal(n, dtype=np.float32) * 3
    pos = np.abs(x) + 0.1
    for prog, ins in [([("input", 0), "gelu_tanh"], [x]), ([("input", 0), "tanh"], [x]),
                      ([("input", 0), "sigmoid"], [x]), ([("input", 0), "exp"], [x]),
                      ([("input", 0), "log"], [pos]), ([("input", 0), "sqrt"], [pos]),
                      ([("input", 0), "rsqrt"], [pos]), ([("input", 0), ("input", 0), "div"], [pos])]:
        got, want = _run(ops, cgb, oracle, cgb.capi.F32, prog, ins, ["full"], n)
        assert_close(got, want, 1e-4, what=str(prog))   # fp32 bound of the path: rel-err <= 1e-4


def test_full_size_config_properties(ops, cgb, oracle):
    """y = relu(a*b+c)*0.5 over 2^26 fp32: checked on a strided sample against the oracle and by
    properties that hold at any size (non-negativity, zero where a*b+c <= 0, scaling linearity)."""
    import torch
    capi = cgb.capi
    n = 1 << 26
    g = torch.Generator(device="cuda").manual_seed(1)
    a, b, c = (torch.randn(n, device="cuda", generator=g) for _ in range(3))
    y = torch.empty_like(a)
    ops.eltwise(capi.make_eltwise_desc(capi.F32, PROG_CHAIN, ["full"] * 3), [a, b, c], y)
    y2 = torch.empty_like(a)
    prog2 = PROG_CHAIN[:-2] + [("imm", 1.0), "mul"]
    ops.eltwise(capi.make_eltwise_desc(capi.F32, prog2, ["full"] * 3), [a, b, c], y2)
    torch.cuda.synchronize()
    assert bool((y >= 0).all())
    assert bool((y2 * 0.5 == y).all())                      # scaling by 0.5 is exact in fp32
    idx = torch.arange(0, n, 4099, device="cuda")
    sa, sb, sc = (t[idx].cpu().numpy() for t in (a, b, c))
    want = oracle.eltwise(oracle.make_eltwise_desc(oracle.F32, PROG_CHAIN, ["full"] * 3), [sa, sb, sc], sa.size)
    assert np.array_equal(_bits(y[idx].cpu().numpy()), _bits(want))


def test_host_buffers_through_the_slab_pipeline(ops, cgb, oracle):
    """Host arrays in, host array out, in eight slabs on three streams chained by events
    (HostRunner.run_slabs, cg_b200_stream_wait_event): every slab's kernel must see its own copy-in
    and every copy-out its own kernel, so the result is the oracle's, bit for bit."""
    import ctypes as C
    import torch
    capi, O = cgb.capi, oracle
    L = capi.lib()
    n, slabs = (1 << 20), 8
    per = n // slabs
    rng = np.random.default_rng(5)
    prog = [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu", ("imm", 0.5), "mul"]
    host_in = [torch.from_numpy(rng.standard_normal(n, dtype=np.float32)).pin_memory() for _ in range(3)]
    host_out = torch.zeros(n, dtype=torch.float32).pin_memory()
    want = O.eltwise(O.make_eltwise_desc(O.F32, prog, ["full"] * 3), [t.numpy() for t in host_in], n)
    desc = capi.make_eltwise_desc(capi.F32, prog, ["full"] * 3)
    r = ops.HostRunner()
    try:
        for rep in range(3):   # the buffers are reused: a slab of one pass must not meet the next pass's copies
            host_out.zero_()
            d = [r.dev(f"in{k}", 4 * n) for k in range(3)]
            o = r.dev("out", 4 * n)
            nb = 4 * per

            def copy_in(i, s):
                for k in range(3):
                    capi.check(L.cg_b200_memcpy_h2d(C.c_void_p(d[k].value + i * nb), C.c_void_p(host_in[k].data_ptr() + i * nb), nb, s))

            def compute(i, s):
                arr = (C.c_void_p * 3)(*[p.value + i * nb for p in d])
                capi.check(L.cg_b200_eltwise(C.byref(desc), arr, 3, C.c_void_p(o.value + i * nb), per, s))

            def copy_out(i, s):
                capi.check(L.cg_b200_memcpy_d2h(C.c_void_p(host_out.data_ptr() + i * nb), C.c_void_p(o.value + i * nb), nb, s))

            r.run_slabs(slabs, copy_in, compute, copy_out)
            assert np.array_equal(host_out.numpy().view(np.uint32), want.view(np.uint32)), f"pass {rep}"
    finally:
        r.close()
