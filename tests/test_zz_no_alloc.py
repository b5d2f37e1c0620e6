"""cg_b200_gemm_f32_static: the fp32 GEMM for callers that cannot allocate device memory.

Such a caller has nowhere to get the workspace cg_b200_gemm asks for on fp32 inputs - for example
a launch routine that receives only tensors and a stream, or a process whose device memory is
already committed to its own pools. The entry point keeps the scratch in a fixed 16 MiB array
inside the library. Here it is called through the C ABI twice in a row, with different shapes so
the second call meets the first call's leftovers in the shared array, and each result is
compared with what cg_b200_gemm computes for the same operands with an ordinary workspace.

This file sorts last so a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest


def test_oversize_and_wrong_dtype_are_rejected_on_the_host(cgb):
    capi = cgb.capi
    L = cgb.lib()
    p = C.c_void_p(4096)
    big = capi.make_gemm_desc(2048, 2048, 2048, capi.F32, capi.F32)       # needs 64 MiB of scratch
    need = C.c_size_t(0)
    assert L.cg_b200_gemm_workspace_bytes(C.byref(big), C.byref(need)) == capi.OK
    assert need.value > capi.GEMM_F32_STATIC_SCRATCH_BYTES
    assert L.cg_b200_gemm_f32_static(C.byref(big), p, p, None, None, p, None, None) == capi.ERR_WORKSPACE
    bf = capi.make_gemm_desc(128, 128, 64, capi.BF16, capi.BF16)            # no scratch needed: other entry point
    assert L.cg_b200_gemm_f32_static(C.byref(bf), p, p, None, None, p, None, None) == capi.ERR_UNSUPPORTED
    assert L.cg_b200_gemm_f32_static(None, p, p, None, None, p, None, None) == capi.ERR_NULL_POINTER


@pytest.mark.gpu
def test_two_calls_in_a_row_match_the_workspace_entry_point(ops, cgb, oracle):
    import torch
    capi, O = cgb.capi, oracle
    L = cgb.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(11)
    # the second shape is smaller and has a K that is not a multiple of 4: its pad columns land on
    # bytes the first call wrote; then K = 0 (no scratch read at all), a batch of three, the largest
    # problem the array holds
    cases = [(384, 520, 300, 1, "bias_relu"), (130, 264, 77, 1, "none"), (96, 72, 0, 1, "bias"), (200, 136, 100, 3, "none"),
             (1024, 1024, 1024, 1, "none")]
    for call, (M, N, K, batch, epi) in enumerate(cases):
        A = torch.rand(batch, M, K, device="cuda", generator=g) * 2 - 1
        B = torch.rand(batch, K, N, device="cuda", generator=g) * 2 - 1
        bias = torch.randn(N, device="cuda", generator=g)
        d = capi.make_gemm_desc(M, N, K, capi.F32, capi.F32, epilogue=epi, batch=batch)
        want = torch.empty(batch * M, N, device="cuda")
        ops.gemm(d, A, B, want, bias=bias if epi != "none" else None)
        got = torch.full((batch * M, N), float("nan"), device="cuda")
        torch.cuda.synchronize()
        # what the entry point exists for: the call itself takes no device memory. The first call on a
        # device only looks up the address of the array that the library's image already holds.
        free_before, _ = torch.cuda.mem_get_info()
        st = L.cg_b200_gemm_f32_static(C.byref(d), C.c_void_p(A.data_ptr()), C.c_void_p(B.data_ptr()),
                                       C.c_void_p(bias.data_ptr()) if epi != "none" else None, None,
                                       C.c_void_p(got.data_ptr()), C.c_void_p(status.data_ptr()), stream)
        capi.check(st, "gemm_f32_static")
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, f"call {call}: {free_before - free_after} bytes of device memory were taken"
        assert int(status.item()) == 0, "a bounded device-side wait ran out"
        assert ops.last_device_error() == 0
        # same kernels, same operands, same order of accumulation: the two entry points agree bit for bit
        assert torch.equal(got, want), f"{M}x{N}x{K} batch {batch}: differs from cg_b200_gemm"
        if call < 4:
            # and against the CPU oracle, within the fp32 bound of the GEMM tests (1e-4 of max|C|)
            od = O.make_gemm_desc(M, N, K, O.F32, O.F32, epilogue=epi, batch=batch)
            ref = O.gemm(od, A.cpu().numpy(), B.cpu().numpy(), bias=bias.cpu().numpy()).reshape(batch * M, N)
            err = np.abs(got.cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert err <= 1e-4, f"{M}x{N}x{K} batch {batch} vs oracle: {err:.3e}"
