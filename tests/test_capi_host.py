"""The C-ABI library without a GPU: it loads, exports every declared symbol, and its host-side
argument checks answer before any device is touched. No compute call needs a device here."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cg_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cg_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(cgb):
    names = declared_symbols()
    assert len(names) >= 30
    L = C.CDLL(cgb.library_path())
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing
    # the ctypes table binds exactly the header's declarations
    assert sorted(cgb.capi.SIGNATURES) == names


def test_version_and_status_strings(cgb):
    L = cgb.lib()
    assert L.cg_b200_version() == (0 << 16) | 1
    seen = set()
    for code in range(0, 12):
        s = L.cg_b200_status_string(code).decode()
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 12
    assert L.cg_b200_status_string(999).decode() == "unknown status"


def test_eltwise_validate_is_host_only(cgb):
    capi = cgb.capi
    L = cgb.lib()
    good = capi.make_eltwise_desc(capi.F32, [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu",
                                             ("imm", 0.5), "mul"], ["full"] * 3)
    assert L.cg_b200_eltwise_validate(C.byref(good), 3) == capi.OK
    assert L.cg_b200_eltwise_validate(C.byref(good), 2) == capi.ERR_INVALID_ARG      # input index out of range
    under = capi.make_eltwise_desc(capi.F32, [("input", 0), "add"], ["full"])
    assert L.cg_b200_eltwise_validate(C.byref(under), 1) == capi.ERR_INVALID_ARG     # stack underflow
    left = capi.make_eltwise_desc(capi.F32, [("input", 0), ("input", 0)], ["full"])
    assert L.cg_b200_eltwise_validate(C.byref(left), 1) == capi.ERR_INVALID_ARG      # two values left
    deep = capi.make_eltwise_desc(capi.F32, [("input", 0)] * 5 + ["add"] * 4, ["full"])
    assert L.cg_b200_eltwise_validate(C.byref(deep), 1) == capi.ERR_INVALID_ARG      # deeper than 4
    bad_dtype = capi.make_eltwise_desc(7, [("input", 0)], ["full"])
    assert L.cg_b200_eltwise_validate(C.byref(bad_dtype), 1) == capi.ERR_INVALID_ARG
    assert L.cg_b200_eltwise_validate(None, 1) == capi.ERR_NULL_POINTER


def test_argument_errors_come_before_device_access(cgb):
    capi = cgb.capi
    L = cgb.lib()
    d = capi.make_eltwise_desc(capi.F32, [("input", 0), "relu"], ["full"])
    ins = (C.c_void_p * 1)(None)
    assert L.cg_b200_eltwise(C.byref(d), ins, 1, C.c_void_p(256), 16, None) == capi.ERR_NULL_POINTER
    assert L.cg_b200_eltwise(C.byref(d), ins, 1, None, 0, None) == capi.OK            # n == 0: no-op
    ins = (C.c_void_p * 1)(258)
    assert L.cg_b200_eltwise(C.byref(d), ins, 1, C.c_void_p(256), 16, None) == capi.ERR_MISALIGNED
    assert L.cg_b200_softmax(capi.BF16, None, None, 4, 4, None) == capi.ERR_NULL_POINTER
    assert L.cg_b200_softmax(capi.BF16, None, None, 0, 4, None) == capi.OK
    assert L.cg_b200_softmax(9, C.c_void_p(256), C.c_void_p(512), 4, 4, None) == capi.ERR_INVALID_ARG
    assert L.cg_b200_layernorm(capi.F32, C.c_void_p(256), None, None, -1.0, C.c_void_p(512), 4, 4, None) \
        == capi.ERR_INVALID_ARG
    g = capi.make_gemm_desc(128, 128, 64, capi.BF16, capi.BF16)
    assert L.cg_b200_gemm(C.byref(g), None, None, None, None, None, None, 0, None) == capi.ERR_NULL_POINTER
    g = capi.make_gemm_desc(128, 128, 64, capi.BF16, capi.BF16, epilogue="bias")
    p = C.c_void_p(1024)
    assert L.cg_b200_gemm(C.byref(g), p, p, None, None, p, None, 0, None) == capi.ERR_NULL_POINTER  # bias missing
    g = capi.make_gemm_desc(128, 128, 60, capi.BF16, capi.BF16)   # lda*2 not a multiple of 16
    assert L.cg_b200_gemm(C.byref(g), p, p, None, None, p, None, 0, None) == capi.ERR_MISALIGNED
    # 3xTF32 splits its operands inside the kernel when TMA can read them in place (16-byte aligned bases and
    # strides); operands that are only 4-byte aligned are rewritten into a workspace first, which must be there
    g = capi.make_gemm_desc(128, 128, 64, capi.F32, capi.F32)
    need = C.c_size_t(0)
    assert L.cg_b200_gemm_workspace_bytes(C.byref(g), C.byref(need)) == capi.OK
    assert need.value == 2 * (128 * 64 + 64 * 128) * 4
    p4 = C.c_void_p(1028)
    assert L.cg_b200_gemm(C.byref(g), p4, p, None, None, p, None, 0, None) == capi.ERR_WORKSPACE
    g = capi.make_gemm_desc(128, 128, 62, capi.F32, capi.F32)     # row stride 248 bytes
    assert L.cg_b200_gemm(C.byref(g), p, p, None, None, p, None, 0, None) == capi.ERR_WORKSPACE
    # column blocks of C side by side (heads of an attention output) do not overlap; anything tighter does
    g = capi.make_gemm_desc(16, 64, 64, capi.BF16, capi.BF16, batch=4, ldc=256, bsc=64)
    assert L.cg_b200_gemm_workspace_bytes(C.byref(g), C.byref(need)) == capi.OK
    g = capi.make_gemm_desc(16, 64, 64, capi.BF16, capi.BF16, batch=4, ldc=256, bsc=32)
    assert L.cg_b200_gemm_workspace_bytes(C.byref(g), C.byref(need)) == capi.ERR_INVALID_ARG
    g = capi.make_gemm_desc(128, 128, 64, capi.BF16, capi.BF16, compute="tf32x3")
    assert L.cg_b200_gemm(C.byref(g), p, p, None, None, p, None, 0, None) == capi.ERR_INVALID_ARG
    g = capi.make_gemm_desc(0, 128, 64, capi.BF16, capi.BF16)
    assert L.cg_b200_gemm(C.byref(g), None, None, None, None, None, None, 0, None) == capi.OK       # empty problem


def test_no_device_is_an_error_not_a_fallback(cgb):
    """Without a GPU a well-formed compute call must fail with NO_DEVICE (there is no CPU path)."""
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present")
    capi = cgb.capi
    L = cgb.lib()
    n = C.c_int(-1)
    assert L.cg_b200_device_count(C.byref(n)) == capi.ERR_NO_DEVICE and n.value == 0
    d = capi.make_eltwise_desc(capi.F32, [("input", 0), "relu"], ["full"])
    ins = (C.c_void_p * 1)(256)
    assert L.cg_b200_eltwise(C.byref(d), ins, 1, C.c_void_p(512), 16, None) == capi.ERR_NO_DEVICE
    assert L.cg_b200_softmax(capi.BF16, C.c_void_p(256), C.c_void_p(512), 4, 8, None) == capi.ERR_NO_DEVICE
    p = C.c_void_p()
    assert L.cg_b200_malloc(C.byref(p), 1024) == capi.ERR_NO_DEVICE
