"""The pybind11 module over the C++ host layer: graph -> lowering -> NvidiaBackend -> Runtime.bind ->
launch, from Python, with the reference module's class names."""
import os
import tempfile

import numpy as np
import pytest


@pytest.fixture(scope="module")
def h(cgb):
    from cantors_gift_b200 import hostapi
    return hostapi.host()


def _chain(h, n):
    m = h.Module()
    f = m.create_function("chain")
    b = h.Builder(f)
    a, bb, c = (b.input_tensor([n], h.DType.F32) for _ in range(3))
    b.output_tensor(b.mul(b.relu(b.add(b.mul(a, bb), c)), b.constant_scalar(0.5, h.DType.F32)))
    return m


def test_compile_without_a_device(h):
    m = _chain(h, 1000)
    low = h.TensorToCodegenLowering()
    cg = low.lower(m)
    assert low.status() == 0 and cg.num_functions() == 1
    backend = h.NvidiaBackend()
    exe = backend.compile(cg)
    assert backend.name() == "nvidia" and exe.name == "chain" and exe.entrypoints == [("chain", 0)]
    assert len(exe.machine_code) > 0 and "eltwise" in exe.ptx_text
    with tempfile.TemporaryDirectory() as d:
        rt = h.Runtime(os.path.join(d, "cache"))
        key = h.KernelCache.compute_key("chain", "1000", "f32", "b200")
        first = rt.compile_and_cache(key, cg, backend)
        second = rt.compile_and_cache(key, cg, backend)
        assert not first.cache_hit and second.cache_hit and rt.kernel_cache().size() == 1
        assert rt.bind(first.executable, h.DeviceId.cuda(0)) is None   # no device was added: None, as the reference's bind
    # schedules: the reference's grid and what the lowering makes of a tile
    space = h.ScheduleSpace.grid_matmul([128, 256], [64, 128, 256], [64], [8])
    assert space.size() == 6 and h.gemm_tuning_from_schedule(space.schedules()[5]) == (256, 2, 0)
    assert h.gemm_tuning_from_schedule(space.schedules()[3]) is None
    bad = h.Schedule()
    bad.add(h.Transform(h.TransformKind.Tile, "n", 96))
    low.lower(m, bad)
    assert low.status() != 0


@pytest.mark.gpu
def test_graph_runs_on_torch_tensors(h, oracle):
    import torch
    from cantors_gift_b200 import hostapi
    O = oracle
    n = (1 << 18) + 5
    rng = np.random.default_rng(11)
    a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
    prog = [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu", ("imm", 0.5), "mul"]
    want = O.eltwise(O.make_eltwise_desc(O.F32, prog, ["full"] * 3), [a, b, c], n)
    with tempfile.TemporaryDirectory() as d:
        rt = h.Runtime(os.path.join(d, "cache"))
        assert rt.add_cuda_device(0) and rt.num_devices() == 1
        low, backend = h.TensorToCodegenLowering(), h.NvidiaBackend()
        exe = backend.compile(low.lower(_chain(h, n)))
        bound = rt.bind(exe, h.DeviceId.cuda(0))
        assert bound is not None
        stream = rt.create_stream(h.DeviceId.cuda(0))
        ins = [torch.from_numpy(t).cuda() for t in (a, b, c)]
        y = torch.empty(n, device="cuda")
        torch.cuda.synchronize()   # the inputs were written on torch's stream
        bound.launch([hostapi.tensor_of(t) for t in ins], [hostapi.tensor_of(y)], stream)
        stream.sync()
        assert bound.status() == 0
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))   # bit-exact, as the C ABI path

        # a matmul with a fused epilogue and a tile taken from a schedule
        M, N, K = 384, 512, 256
        m = h.Module()
        f = m.create_function("mm")
        bl = h.Builder(f)
        xa = bl.input_tensor([M, K], h.DType.BF16)
        xb = bl.input_tensor([K, N], h.DType.BF16)
        bl.output_tensor(bl.relu(bl.matmul(xa, xb)))
        s = h.Schedule()
        s.add(h.Transform(h.TransformKind.Tile, "m", 128, 128))
        s.add(h.Transform(h.TransformKind.Tile, "n", 128))
        cg = low.lower(m, s)
        assert low.status() == 0
        bound2 = rt.bind(backend.compile(cg), h.DeviceId.cuda(0))
        A = O.to_bf16(rng.standard_normal((M, K), dtype=np.float32) * 0.05)
        B = O.to_bf16(rng.standard_normal((K, N), dtype=np.float32) * 0.05)
        dev = lambda x: torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16)  # noqa: E731
        Ad, Bd = dev(A), dev(B)
        Cd = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        bound2.launch([hostapi.tensor_of(Ad), hostapi.tensor_of(Bd)], [hostapi.tensor_of(Cd)], stream)
        stream.sync()
        assert bound2.status() == 0
        ref = np.maximum(np.asarray(O.gemm(O.make_gemm_desc(M, N, K, O.BF16, O.F32), A, B), dtype=np.float32), 0.0).reshape(M, N)
        got = O.from_bf16(Cd.cpu().view(torch.int16).numpy().view(np.uint16))
        assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()
