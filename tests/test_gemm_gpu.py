"""Parity of the tcgen05 GEMM (+ fused epilogue) against the CPU oracle, through the C ABI.

Tolerances are the path's stated bounds: rel-err <= 1e-4 for fp32 (3xTF32 split), <= 1e-2 for
bf16/f16, on both metrics of conftest.assert_close."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _dev(ops, store, dtype):
    import torch
    if store is None:
        return None
    raw = torch.from_numpy(store.view(np.int16) if store.dtype != np.float32 else store).cuda()
    return raw.view(ops.TORCH_DTYPE[dtype]) if store.dtype != np.float32 else raw


def _host_f32(O, t, dtype):
    import torch
    c = t.cpu()
    if dtype == O.F32:
        return c.numpy()
    return O.to_f32(c.view(torch.int16).numpy().view(np.uint16 if dtype == O.BF16 else np.float16), dtype)


def run_case(ops, cgb, O, M, N, K, in_dt, out_dt, epilogue="none", batch=1, b_transposed=0, bsb=None,
             compute="default", scale=0.05, seed=0, alpha=1.0, rows=None, pad=0, return_operands=False):
    """Returns (gpu fp32 [batch*M, N], oracle fp32 [batch*M, N] (only `rows` valid when given))."""
    import torch
    capi = cgb.capi
    rng = np.random.default_rng(seed)
    lda, ldc = K + pad, N + pad
    ldb = (K if b_transposed else N) + pad
    b_batches = 1 if bsb == 0 else batch
    A = np.zeros((batch, M, lda), dtype=np.float32)
    A[:, :, :K] = rng.standard_normal((batch, M, K), dtype=np.float32) * scale
    Bshape = (b_batches, N, ldb) if b_transposed else (b_batches, K, ldb)
    B = np.zeros(Bshape, dtype=np.float32)
    if b_transposed:
        B[:, :, :K] = rng.standard_normal((b_batches, N, K), dtype=np.float32) * scale
    else:
        B[:, :, :N] = rng.standard_normal((b_batches, K, N), dtype=np.float32) * scale
    bias = rng.standard_normal(N, dtype=np.float32)
    res = np.zeros((batch, M, ldc), dtype=np.float32)
    res[:, :, :N] = rng.standard_normal((batch, M, N), dtype=np.float32)
    As, Bs = O.to_storage(A, in_dt), O.to_storage(B, in_dt)
    bs_, rs_ = O.to_storage(bias, out_dt), O.to_storage(res, out_dt)
    kw = dict(epilogue=epilogue, batch=batch, b_transposed=b_transposed, lda=lda, ldb=ldb, ldc=ldc, bsb=bsb, alpha=alpha)
    od = O.make_gemm_desc(M, N, K, in_dt, out_dt, **kw)
    want = O.gemm(od, As, Bs, bias=bs_, residual=rs_, rows=rows, out=np.zeros(batch * M * ldc, dtype=O.NP_OF[out_dt]))
    want = O.to_f32(want, out_dt).reshape(batch * M, ldc)[:, :N]
    gd = capi.make_gemm_desc(M, N, K, in_dt, out_dt, compute=compute, **kw)
    Ad, Bd = _dev(ops, As, in_dt), _dev(ops, Bs, in_dt)
    Cd = torch.zeros(batch * M * ldc, dtype=ops.TORCH_DTYPE[out_dt], device="cuda")
    ops.gemm(gd, Ad, Bd, Cd, bias=_dev(ops, bs_, out_dt), residual=_dev(ops, rs_, out_dt))
    assert ops.last_device_error() == 0, "a bounded device-side wait ran out"
    got = _host_f32(O, Cd, out_dt).reshape(batch * M, ldc)[:, :N]
    if return_operands:
        return got, want, A[:, :, :K], (B[:, :, :K].transpose(0, 2, 1) if b_transposed else B[:, :, :N])
    return got, want


def assert_dot_close(got, want, A, B, tol, what):
    """Error bound for raw dot products: max|y-ref| / max|ref| <= tol and, componentwise,
    |y-ref|_ij <= tol * (|A| |B|)_ij. The second is the scale on which any floating-point
    summation of sum_k a_ik b_kj can be compared (results near zero by cancellation have no
    meaningful relative error of their own: the reference's own fp32 FMA chain is 1e-6 * (|A||B|)
    away from the exact sum)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    scale = np.abs(A[0].astype(np.float64)) @ np.abs(B[0].astype(np.float64))
    norm = np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)
    comp = (np.abs(got - want) / np.maximum(scale, 1e-30)).max()
    assert norm <= tol and comp <= tol, f"{what}: max-normalised {norm:.3e}, componentwise {comp:.3e}, tol {tol}"


SHAPES = [(128, 256, 64), (128, 256, 256), (256, 512, 192), (128, 64, 64), (128, 128, 128),
          (100, 200, 72), (1, 8, 8), (130, 264, 328), (384, 768, 1024)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("b_transposed", [0, 1])
def test_bf16_gemm_plain(ops, cgb, oracle, M, N, K, b_transposed):
    capi = cgb.capi
    got, want = run_case(ops, cgb, oracle, M, N, K, capi.BF16, capi.BF16, b_transposed=b_transposed, seed=M + N + K)
    assert_close(got, want, 1e-2, f"bf16 {M}x{N}x{K} bT={b_transposed}")


@pytest.mark.parametrize("b_transposed", [0, 1])
def test_bf16_gemm_tail_half_tiles(ops, cgb, oracle, b_transposed):
    """80 tiles of 256x256 on 74 CTA pairs: the last 6 tiles run as 12 half-width units; the N tail
    (2000 columns) also puts a half unit partly and one wholly out of range."""
    capi = cgb.capi
    got, want = run_case(ops, cgb, oracle, 2560, 2000, 192, capi.BF16, capi.BF16, b_transposed=b_transposed,
                         epilogue="bias_relu", seed=77)
    assert_close(got, want, 1e-2, f"tail halves bT={b_transposed}")


@pytest.mark.parametrize("epilogue", ["bias", "bias_relu", "bias_gelu_tanh", "bias_residual", "residual", "scale", "relu", "gelu_tanh"])
@pytest.mark.parametrize("out_name", ["BF16", "F32"])
def test_bf16_gemm_epilogues(ops, cgb, oracle, epilogue, out_name):
    capi = cgb.capi
    out_dt = getattr(capi, out_name)
    got, want = run_case(ops, cgb, oracle, 200, 328, 136, capi.BF16, out_dt, epilogue=epilogue, scale=0.2, alpha=0.125)
    assert_close(got, want, 1e-2 if out_name == "BF16" else 2e-3, f"{epilogue} -> {out_name}")


def test_f16_gemm(ops, cgb, oracle):
    capi = cgb.capi
    got, want = run_case(ops, cgb, oracle, 256, 256, 256, capi.F16, capi.F16, epilogue="bias_gelu_tanh", scale=0.1)
    assert_close(got, want, 1e-2, "f16 gelu")


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (128, 128, 256), (200, 136, 100), (256, 384, 512), (5, 3, 7)])
@pytest.mark.parametrize("b_transposed", [0, 1])
def test_fp32_gemm_3xtf32(ops, cgb, oracle, M, N, K, b_transposed):
    """fp32 in/out: hi/lo TF32 split. Inputs ~U[-1,1) as in the 1024^3 configuration."""
    capi = cgb.capi
    pad = (-N) % 4  # C rows must be 16-byte multiples
    got, want, A, B = run_case(ops, cgb, oracle, M, N, K, capi.F32, capi.F32, b_transposed=b_transposed, scale=0.5,
                               seed=K, pad=pad, return_operands=True)
    assert_dot_close(got, want, A, B, 1e-4, f"fp32 {M}x{N}x{K} bT={b_transposed}")


def test_fp32_gemm_matches_reference_golden(ops, cgb, oracle):
    """The reference's own JIT matmul outputs (tests/golden) within the fp32 bound."""
    import torch
    capi = cgb.capi
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_kernels.npz"))
    A, B, Cref = gold["mm_sq_A"], gold["mm_sq_B"], gold["mm_sq_C"]
    M, K = A.shape
    N = B.shape[1]
    gd = capi.make_gemm_desc(M, N, K, capi.F32, capi.F32)
    Cd = torch.zeros(M, N, device="cuda")
    ops.gemm(gd, torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), Cd)
    assert ops.last_device_error() == 0
    assert_dot_close(Cd.cpu().numpy(), Cref, A[None], B[None], 1e-4, "golden mm_sq")


def test_fp32_matmul_1024_cubed_matches_the_reference_jit_kernel(ops, cgb, oracle):
    """The fp32 configuration at its full size: M = N = K = 1024, A then B ~ U[-1, 1) from one
    default_rng(0) stream. The GPU result (3xTF32 split) against the reference's own scalar-FMA JIT
    matmul (benchmarks/benchmark.py:326-438, run from its compiled emitter when that checker library
    is present) within 1e-4; the oracle's restatement must equal the reference's kernel bit for bit,
    so where the reference library is absent the restatement stands in for it."""
    import torch
    capi, O = cgb.capi, oracle
    n = 1024
    rng = np.random.default_rng(0)
    A = (rng.random((n, n), dtype=np.float32) * 2 - 1).astype(np.float32)
    B = (rng.random((n, n), dtype=np.float32) * 2 - 1).astype(np.float32)
    port = O.gemm(O.make_gemm_desc(n, n, n, O.F32, O.F32), A, B).reshape(n, n)
    if O.have_ref():
        want = O.ref_matmul(A, B)
        assert np.array_equal(want.view(np.uint32), port.view(np.uint32)), "oracle port differs from the reference's JIT matmul"
    else:
        want = port
    Cd = torch.zeros(n, n, device="cuda")
    ops.gemm(capi.make_gemm_desc(n, n, n, capi.F32, capi.F32), torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), Cd)
    assert ops.last_device_error() == 0
    got = Cd.cpu().numpy()
    assert_dot_close(got, want, A[None], B[None], 1e-4, "fp32 1024^3 vs reference JIT")
    exact = A.astype(np.float64) @ B.astype(np.float64)
    from conftest import report_metrics
    report_metrics("fp32 1024^3 vs fp64", gpu_max_normalised=np.abs(got - exact).max() / np.abs(exact).max(),
                   reference_max_normalised=np.abs(want - exact).max() / np.abs(exact).max())


@pytest.mark.parametrize("M,N,K", [(5, 3, 7), (200, 136, 100), (256, 384, 512), (300, 520, 256)])
@pytest.mark.parametrize("b_transposed", [0, 1])
def test_fp32_gemm_single_pass_tf32(ops, cgb, oracle, M, N, K, b_transposed):
    """compute = tf32: one kind::tf32 pass on operands truncated to tf32 (10 mantissa bits), the
    one-copy workspace layout and the wider tiles that pass uses. Bound: 2e-3 of max|C| and,
    componentwise, of (|A||B|)_ij - two truncations of 2^-10 relative each."""
    capi = cgb.capi
    pad = (-N) % 4
    got, want, A, B = run_case(ops, cgb, oracle, M, N, K, capi.F32, capi.F32, b_transposed=b_transposed, scale=0.5,
                               seed=K + 1, pad=pad, compute="tf32", return_operands=True)
    assert_dot_close(got, want, A, B, 2e-3, f"tf32 {M}x{N}x{K} bT={b_transposed}")


def test_batched_and_broadcast(ops, cgb, oracle):
    capi = cgb.capi
    got, want = run_case(ops, cgb, oracle, 136, 72, 64, capi.BF16, capi.BF16, batch=5, epilogue="scale", alpha=0.5)
    assert_close(got, want, 1e-2, "batched")
    got, want = run_case(ops, cgb, oracle, 136, 264, 64, capi.BF16, capi.BF16, batch=3, bsb=0, b_transposed=1)
    assert_close(got, want, 1e-2, "B broadcast over batch")


def test_two_level_batch_strided_operands(ops, cgb, oracle):
    """Heads inside sequences: A and B are column blocks of one [rows, 3D] buffer (row stride 3D), the
    inner batch level steps by the head width, the outer by a whole sequence; C is written into
    column blocks of a [rows, D] buffer. The layout of the attention GEMMs."""
    import torch
    capi, O = cgb.capi, oracle
    Bo, H, S, dh = 3, 4, 136, 64
    D = H * dh
    rng = np.random.default_rng(9)
    qkv = O.to_bf16(rng.standard_normal((Bo * S, 3 * D), dtype=np.float32) * 0.3)
    kw = dict(batch=Bo * H, batch_inner=H, lda=3 * D, ldb=3 * D, b_transposed=1, bsa=S * 3 * D, bsb=S * 3 * D, isa=dh, isb=dh)
    # scores = Q K^T * 0.125 -> [Bo, H, S, S]
    od = O.make_gemm_desc(S, S, dh, O.BF16, O.BF16, epilogue="scale", alpha=0.125, ldc=S, bsc=H * S * S, isc=S * S, **kw)
    k_view = qkv.reshape(-1)[D:]
    want = O.from_bf16(O.gemm(od, qkv, k_view, out=np.zeros(Bo * H * S * S, dtype=np.uint16)))
    gd = capi.make_gemm_desc(S, S, dh, capi.BF16, capi.BF16, epilogue="scale", alpha=0.125, ldc=S, bsc=H * S * S, isc=S * S, **kw)
    qd = torch.from_numpy(qkv.view(np.int16)).cuda().view(torch.bfloat16)
    sc = torch.zeros(Bo * H * S * S, dtype=torch.bfloat16, device="cuda")
    ops.gemm(gd, qd, qd.view(-1)[D:], sc)
    assert ops.last_device_error() == 0
    assert_close(_host_f32(O, sc, capi.BF16), want, 1e-2, "QK^T two-level batch")
    # ctx[:, h*dh:(h+1)*dh] = P_bh V_bh with V = third column block, N contiguous
    P = O.to_bf16(rng.random((Bo * H * S, S), dtype=np.float32) / S)
    kw2 = dict(batch=Bo * H, batch_inner=H, lda=S, ldb=3 * D, ldc=D, bsa=H * S * S, bsb=S * 3 * D, bsc=S * D, isa=S * S, isb=dh, isc=dh)
    od2 = O.make_gemm_desc(S, dh, S, O.BF16, O.BF16, **kw2)
    want2 = O.from_bf16(O.gemm(od2, P, qkv.reshape(-1)[2 * D:], out=np.zeros(Bo * S * D, dtype=np.uint16)))
    gd2 = capi.make_gemm_desc(S, dh, S, capi.BF16, capi.BF16, **kw2)
    ctx = torch.zeros(Bo * S * D, dtype=torch.bfloat16, device="cuda")
    ops.gemm(gd2, torch.from_numpy(P.view(np.int16)).cuda().view(torch.bfloat16), qd.view(-1)[2 * D:], ctx)
    assert ops.last_device_error() == 0
    assert_close(_host_f32(O, ctx, capi.BF16), want2, 1e-2, "PV two-level batch")


def test_fused_allgather_writes_every_destination(ops, cgb, oracle):
    """cg_b200_gemm_allgather on one GPU, the two 'peers' being other local buffers: rank 1 of 3 must
    put its rows into rows [M, 2M) of all three full-size buffers and touch nothing else."""
    import ctypes as C
    import torch
    capi, O = cgb.capi, oracle
    M, N, K, world, rank = 200, 328, 136, 3, 1   # ragged in M (tile tail) and N (partial 32-column chunk)
    ldc = 336
    rng = np.random.default_rng(12)
    A = O.to_bf16(rng.standard_normal((M, K), dtype=np.float32) * 0.1)
    B = O.to_bf16(rng.standard_normal((K, N), dtype=np.float32) * 0.1)
    bias = O.to_bf16(rng.standard_normal(N, dtype=np.float32))
    od = O.make_gemm_desc(M, N, K, O.BF16, O.BF16, epilogue="bias_gelu_tanh", ldc=ldc)
    want = O.from_bf16(O.gemm(od, A, B, bias=bias, out=np.zeros(M * ldc, dtype=np.uint16))).reshape(M, ldc)[:, :N]
    dev = lambda h: torch.from_numpy(h.view(np.int16)).cuda().view(torch.bfloat16)  # noqa: E731
    bufs = [torch.zeros(world * M, ldc, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    peers = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    gd = capi.make_gemm_desc(M, N, K, capi.BF16, capi.BF16, epilogue="bias_gelu_tanh", ldc=ldc)
    Ad, Bd, bd = dev(A), dev(B), dev(bias)
    st = cgb.lib().cg_b200_gemm_allgather(C.byref(gd), C.c_void_p(Ad.data_ptr()), C.c_void_p(Bd.data_ptr()),
                                          C.c_void_p(bd.data_ptr()), None, C.c_void_p(bufs[rank].data_ptr()), peers,
                                          world, rank, None, 0, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    capi.check(st, "gemm_allgather")
    assert ops.last_device_error() == 0
    for b in bufs:
        full = _host_f32(O, b.view(-1), capi.BF16).reshape(world * M, ldc)
        assert_close(full[rank * M:(rank + 1) * M, :N], want, 1e-2, "fused all-gather rows")
        assert not full[:rank * M].any() and not full[(rank + 1) * M:].any() and not full[:, N:].any()
    assert torch.equal(bufs[0], bufs[1]) and torch.equal(bufs[1], bufs[2])


@pytest.mark.parametrize("tile_n,pair", [(0, 0), (128, 2), (128, 1), (64, 1)])
def test_fused_allgather_with_the_barrier_in_its_tail(ops, cgb, oracle, tile_n, pair):
    """cg_b200_gemm_allgather_sync on one GPU: the "peers" are local buffers, and their side of the flag
    barrier is played by the host, which writes the epochs this rank will wait for into its flag buffer
    before the launch. Checked: every destination holds the rows, the peers' flag buffers hold this
    rank's epoch, a second call (epoch 2) works - so the kernel's CTA counter returned to zero - and
    every tile choice gives the same bits."""
    import torch
    capi, O = cgb.capi, oracle
    L = cgb.lib()
    world, rank, M, N, K = 3, 1, 520, 392, 136
    rng = np.random.default_rng(5)
    A = O.to_bf16(rng.standard_normal((M, K), dtype=np.float32) * 0.05)
    B = O.to_bf16(rng.standard_normal((K, N), dtype=np.float32) * 0.05)
    bias = O.to_bf16(rng.standard_normal(N, dtype=np.float32))
    od = O.make_gemm_desc(M, N, K, O.BF16, O.BF16, epilogue="bias_gelu_tanh")
    want = O.from_bf16(O.gemm(od, A, B, bias=bias, out=np.zeros(M * N, dtype=np.uint16))).reshape(M, N)
    dev = lambda h: torch.from_numpy(h.view(np.int16)).cuda().view(torch.bfloat16)  # noqa: E731
    bufs = [torch.zeros(world * M, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    flags[rank][:] = 2   # the peers' epochs 1 and 2 "have arrived"
    peers = (C.c_void_p * world)(*[b.data_ptr() for b in bufs])
    ftab = (C.c_void_p * world)(*[f.data_ptr() for f in flags])
    bar = C.c_void_p()
    capi.check(L.cg_b200_peer_barrier_create(C.byref(bar), ftab, world, rank), "peer_barrier_create")
    capi.check(L.cg_b200_peer_barrier_set_timeout(bar, 50_000_000), "set_timeout")
    gd = capi.make_gemm_desc(M, N, K, capi.BF16, capi.BF16, epilogue="bias_gelu_tanh")
    tuning = capi.GemmTuning(tile_n=tile_n, cta_pair=pair, tail_split=0, reserved=0)
    Ad, Bd, bd = dev(A), dev(B), dev(bias)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    try:
        for epoch in (1, 2):
            for b in bufs:
                b.zero_()
            capi.check(L.cg_b200_gemm_allgather_sync(C.byref(gd), C.byref(tuning), C.c_void_p(Ad.data_ptr()),
                                                     C.c_void_p(Bd.data_ptr()), C.c_void_p(bd.data_ptr()), None,
                                                     C.c_void_p(bufs[rank].data_ptr()), peers, world, rank, bar, None, 0, stream),
                       "gemm_allgather_sync")
            assert ops.last_device_error() == 0, "the flag wait ran out"
            for r in range(world):
                if r != rank:
                    assert int(flags[r][rank].item()) == epoch
            full = _host_f32(O, bufs[0].view(-1), capi.BF16).reshape(world * M, N)
            assert_close(full[rank * M:(rank + 1) * M], want, 1e-2, f"sync all-gather rows tile_n={tile_n} pair={pair}")
            assert not full[:rank * M].any() and not full[(rank + 1) * M:].any()
            assert torch.equal(bufs[0], bufs[1]) and torch.equal(bufs[1], bufs[2])
        plain = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        ops.gemm(gd, Ad, Bd, plain, bias=bd)
        assert torch.equal(plain, bufs[0][rank * M:(rank + 1) * M])   # the sharded kernel's bits are the one-GPU kernel's
    finally:
        capi.check(L.cg_b200_peer_barrier_destroy(bar), "peer_barrier_destroy")


def test_peer_push_copies_to_every_destination_and_ends_in_the_barrier(ops, cgb):
    """cg_b200_peer_push with local stand-ins for the peers: odd sizes, the grid's tail loop, and the
    barrier in the kernel's tail (peers' epochs pre-written by the host)."""
    import torch
    capi = cgb.capi
    L = cgb.lib()
    world, rank = 4, 2
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    flags = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    flags[rank][:] = 1
    ftab = (C.c_void_p * world)(*[f.data_ptr() for f in flags])
    bar = C.c_void_p()
    capi.check(L.cg_b200_peer_barrier_create(C.byref(bar), ftab, world, rank), "peer_barrier_create")
    capi.check(L.cg_b200_peer_barrier_set_timeout(bar, 50_000_000), "set_timeout")
    try:
        for n_bytes, with_barrier in ((16, False), (16 * 2049, False), (16 * (1 << 18) + 48, True)):
            src = torch.randint(-128, 127, (n_bytes,), dtype=torch.int8, device="cuda")
            dst = [torch.zeros(n_bytes + 32, dtype=torch.int8, device="cuda") for _ in range(world)]
            tab = (C.c_void_p * world)(*[d.data_ptr() + 16 for d in dst])
            capi.check(L.cg_b200_peer_push(C.c_void_p(src.data_ptr()), tab, world, rank, n_bytes, bar if with_barrier else None,
                                           stream), "peer_push")
            assert ops.last_device_error() == 0
            for r in range(world):
                if r == rank:
                    assert not dst[r].any()                     # the rank's own entry is never written
                else:
                    assert torch.equal(dst[r][16:16 + n_bytes], src) and not dst[r][:16].any() and not dst[r][16 + n_bytes:].any()
            if with_barrier:
                assert all(int(flags[r][rank].item()) == 1 for r in range(world) if r != rank)
        assert L.cg_b200_peer_push(None, None, world, rank, 24, None, stream) == capi.ERR_INVALID_ARG   # not a multiple of 16
    finally:
        capi.check(L.cg_b200_peer_barrier_destroy(bar), "peer_barrier_destroy")


def test_k_zero_gives_epilogue_of_zero(ops, cgb, oracle):
    capi = cgb.capi
    got, want = run_case(ops, cgb, oracle, 130, 72, 0, capi.BF16, capi.BF16, epilogue="bias")
    assert_close(got, want, 1e-2, "K=0")


def test_full_size_bf16_gemm_bias_gelu(ops, cgb, oracle):
    """M=N=K=4096, bias + GELU(tanh): 48 sampled rows against the oracle (all columns), plus
    linearity in A on the raw product, which holds at any size."""
    import torch
    capi = cgb.capi
    O = oracle
    M = N = K = 4096
    rng = np.random.default_rng(2)
    A = O.to_bf16(rng.standard_normal((M, K), dtype=np.float32) * 0.02)
    B = O.to_bf16(rng.standard_normal((K, N), dtype=np.float32) * 0.02)
    bias = O.to_bf16(rng.standard_normal(N, dtype=np.float32))
    rows = np.sort(rng.choice(M, size=48, replace=False)).astype(np.int64)
    od = O.make_gemm_desc(M, N, K, O.BF16, O.BF16, epilogue="bias_gelu_tanh")
    want = O.from_bf16(O.gemm(od, A, B, bias=bias, rows=rows)).reshape(M, N)[rows]
    gd = capi.make_gemm_desc(M, N, K, capi.BF16, capi.BF16, epilogue="bias_gelu_tanh")
    Ad, Bd, bd = _dev(ops, A, capi.BF16), _dev(ops, B, capi.BF16), _dev(ops, bias, capi.BF16)
    Cd = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm(gd, Ad, Bd, Cd, bias=bd)
    assert ops.last_device_error() == 0
    got = _host_f32(O, Cd, capi.BF16).reshape(M, N)[rows]
    assert_close(got, want, 1e-2, "4096^3 bias+gelu sample")
    # linearity: (2A) B == 2 (A B) exactly in bf16/fp32 arithmetic (power-of-two scaling)
    gd0 = capi.make_gemm_desc(M, N, K, capi.BF16, capi.F32)
    C1 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    C2 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    ops.gemm(gd0, Ad, Bd, C1)
    ops.gemm(gd0, Ad * 2, Bd, C2)
    torch.cuda.synchronize()
    assert torch.equal(C1 * 2, C2)


def test_tuned_variants_agree_bit_for_bit(ops, cgb, oracle):
    """cg_b200_gemm_tuned: every tile choice an autotuner may ask for gives the heuristic's result
    bit for bit (same K order of accumulation), and combinations no kernel has are refused."""
    import torch
    capi, O = cgb.capi, oracle
    M, N, K = 600, 840, 320   # several tile rows and columns with ragged edges for every tile shape
    rng = np.random.default_rng(77)
    A = O.to_storage(rng.standard_normal((M, K), dtype=np.float32) * 0.05, capi.BF16)
    B = O.to_storage(rng.standard_normal((K, N), dtype=np.float32) * 0.05, capi.BF16)
    bias = O.to_storage(rng.standard_normal(N, dtype=np.float32), capi.BF16)
    desc = capi.make_gemm_desc(M, N, K, capi.BF16, capi.BF16, epilogue="bias_gelu_tanh")
    Ad, Bd, bd = (_dev(ops, t, capi.BF16) for t in (A, B, bias))

    def run(tuning):
        Cd = torch.zeros(M * N, dtype=torch.bfloat16, device="cuda")
        ops.gemm(desc, Ad, Bd, Cd, bias=bd, tuning=tuning)
        assert ops.last_device_error() == 0
        return Cd.view(torch.int16).cpu().numpy()

    base = run(None)
    want = O.gemm(O.make_gemm_desc(M, N, K, capi.BF16, capi.BF16, epilogue="bias_gelu_tanh"), A, B, bias=bias,
                  out=np.zeros(M * N, dtype=O.NP_OF[capi.BF16]))
    assert_close(O.to_f32(base.view(np.uint16), capi.BF16), O.to_f32(want, capi.BF16), 1e-2, "tuned gemm baseline")
    ran = 0
    for tile_n in (0, 64, 128, 256):
        for pair in (0, 1, 2):
            for tail in (0, 1, 2):
                t = capi.GemmTuning(tile_n=tile_n, cta_pair=pair, tail_split=tail, reserved=0)
                if pair == 2 and tile_n == 64:
                    with pytest.raises(capi.CgB200Error) as e:
                        run(t)
                    assert e.value.status == capi.ERR_UNSUPPORTED
                    continue
                got = run(t)
                assert np.array_equal(got, base), f"tile_n={tile_n} pair={pair} tail={tail} differs from the default"
                ran += 1
    assert ran == 33
    bad = capi.GemmTuning(tile_n=96, cta_pair=0, tail_split=0, reserved=0)
    assert cgb.lib().cg_b200_gemm_tuned(C.byref(desc), C.byref(bad), None, None, None, None, None, None, 0, None) == capi.ERR_INVALID_ARG
    f32 = capi.make_gemm_desc(128, 128, 64, capi.F32, capi.F32)
    pair = capi.GemmTuning(tile_n=0, cta_pair=2, tail_split=0, reserved=0)
    x = torch.zeros(128 * 128, dtype=torch.float32, device="cuda")
    with pytest.raises(capi.CgB200Error) as e:
        ops.gemm(f32, x, x, x.clone(), tuning=pair)
    assert e.value.status == capi.ERR_UNSUPPORTED
