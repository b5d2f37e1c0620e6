"""ctypes bindings of include/cg_b200.h.

Loading fails loudly when lib/libcg_b200.so is absent: build it with
`python cantors-gift_b200/build.py`. Nothing here computes on the CPU.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))

OK = 0
ERR_INVALID_ARG, ERR_NULL_POINTER, ERR_MISALIGNED, ERR_UNSUPPORTED, ERR_CUDA = 1, 2, 3, 4, 5
ERR_NO_DEVICE, ERR_WORKSPACE, ERR_DEVICE_TIMEOUT, ERR_COMM, ERR_FUSED_IR, ERR_NOT_SM100 = 6, 7, 8, 9, 10, 11

F16, BF16, F32 = 0, 1, 2
DTYPE_BYTES = {F16: 2, BF16: 2, F32: 4}

EW_MAX_INSTR, EW_MAX_INPUTS, EW_MAX_STACK = 16, 8, 4
EW_OPS = {name: i for i, name in enumerate(
    ["input", "imm", "add", "sub", "mul", "div", "max", "min", "neg", "abs", "relu", "gelu_tanh",
     "tanh", "sigmoid", "exp", "log", "sqrt", "rsqrt"])}
BCAST = {"full": 0, "scalar": 1, "row": 2, "col": 3}
EPILOGUE = {"none": 0, "bias": 1, "bias_relu": 2, "bias_gelu_tanh": 3, "bias_residual": 4,
            "residual": 5, "scale": 6, "relu": 7, "gelu_tanh": 8}
COMPUTE = {"default": 0, "tf32x3": 1, "tf32": 2}
REDUCE = {"sum": 0, "max": 1, "mean": 2}
COMM_ID_BYTES = 128
IPC_HANDLE_BYTES = 64
GEMM_F32_STATIC_SCRATCH_BYTES = 16 << 20


class CgB200Error(RuntimeError):
    def __init__(self, status, what=""):
        self.status = status
        text = lib().cg_b200_status_string(status).decode()
        detail = lib().cg_b200_last_cuda_error().decode() if status in (ERR_CUDA, ERR_NO_DEVICE) else ""
        super().__init__(f"cg_b200 {what}: status {status} ({text}){' - ' + detail if detail else ''}")


class Props(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("cc_major", C.c_int32), ("cc_minor", C.c_int32),
                ("sm_count", C.c_int32), ("max_smem_per_block", C.c_int32), ("l2_bytes", C.c_int32),
                ("sm_clock_khz", C.c_int32), ("mem_clock_khz", C.c_int32), ("mem_bus_bits", C.c_int32),
                ("hbm_bytes", C.c_uint64), ("tmem_bytes_per_sm", C.c_uint64)]


class EltwiseInstr(C.Structure):
    _fields_ = [("op", C.c_int32), ("arg", C.c_int32), ("imm", C.c_float)]


class EltwiseDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("n_instr", C.c_int32),
                ("prog", EltwiseInstr * EW_MAX_INSTR),
                ("bcast", C.c_int32 * EW_MAX_INPUTS),
                ("inner", C.c_int64), ("round_each_op", C.c_int32), ("reserved", C.c_int32)]


class GemmDesc(C.Structure):
    _fields_ = [("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("batch", C.c_int64),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("batch_stride_a", C.c_int64), ("batch_stride_b", C.c_int64),
                ("batch_stride_c", C.c_int64),
                ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("compute", C.c_int32),
                ("epilogue", C.c_int32), ("b_transposed", C.c_int32), ("alpha", C.c_float),
                ("batch_inner", C.c_int64), ("inner_stride_a", C.c_int64), ("inner_stride_b", C.c_int64),
                ("inner_stride_c", C.c_int64)]


class GemmTuning(C.Structure):
    _fields_ = [("tile_n", C.c_int32), ("cta_pair", C.c_int32), ("tail_split", C.c_int32), ("reserved", C.c_int32)]


class AttentionDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("head_dim", C.c_int32), ("batch", C.c_int64), ("heads", C.c_int64),
                ("seq_q", C.c_int64), ("seq_kv", C.c_int64),
                ("ldq", C.c_int64), ("ldk", C.c_int64), ("ldv", C.c_int64), ("ldo", C.c_int64),
                ("head_stride_q", C.c_int64), ("head_stride_k", C.c_int64), ("head_stride_v", C.c_int64),
                ("head_stride_o", C.c_int64), ("batch_stride_q", C.c_int64), ("batch_stride_k", C.c_int64),
                ("batch_stride_v", C.c_int64), ("batch_stride_o", C.c_int64), ("scale", C.c_float),
                ("reserved", C.c_int32)]


_vp, _vpp, _sz, _i, _i64 = C.c_void_p, C.POINTER(C.c_void_p), C.c_size_t, C.c_int, C.c_int64

# name -> (restype, argtypes); exactly the declarations of include/cg_b200.h
SIGNATURES = {
    "cg_b200_version": (_i, []),
    "cg_b200_status_string": (C.c_char_p, [_i]),
    "cg_b200_last_cuda_error": (C.c_char_p, []),
    "cg_b200_device_count": (_i, [C.POINTER(_i)]),
    "cg_b200_device_props": (_i, [_i, C.POINTER(Props)]),
    "cg_b200_set_device": (_i, [_i]),
    "cg_b200_malloc": (_i, [_vpp, _sz]),
    "cg_b200_free": (_i, [_vp]),
    "cg_b200_malloc_host": (_i, [_vpp, _sz]),
    "cg_b200_free_host": (_i, [_vp]),
    "cg_b200_memcpy_h2d": (_i, [_vp, _vp, _sz, _vp]),
    "cg_b200_memcpy_d2h": (_i, [_vp, _vp, _sz, _vp]),
    "cg_b200_memset": (_i, [_vp, _i, _sz, _vp]),
    "cg_b200_stream_create": (_i, [_vpp]),
    "cg_b200_stream_destroy": (_i, [_vp]),
    "cg_b200_stream_sync": (_i, [_vp]),
    "cg_b200_event_create": (_i, [_vpp]),
    "cg_b200_event_destroy": (_i, [_vp]),
    "cg_b200_event_record": (_i, [_vp, _vp]),
    "cg_b200_event_sync": (_i, [_vp]),
    "cg_b200_stream_wait_event": (_i, [_vp, _vp]),
    "cg_b200_event_elapsed_sec": (_i, [_vp, _vp, C.POINTER(C.c_double)]),
    "cg_b200_eltwise_validate": (_i, [C.POINTER(EltwiseDesc), _i]),
    "cg_b200_eltwise": (_i, [C.POINTER(EltwiseDesc), _vpp, _i, _vp, _sz, _vp]),
    "cg_b200_softmax": (_i, [_i, _vp, _vp, _i64, _i64, _vp]),
    "cg_b200_layernorm": (_i, [_i, _vp, _vp, _vp, C.c_float, _vp, _i64, _i64, _vp]),
    "cg_b200_softmax_layernorm": (_i, [_i, _vp, _vp, _vp, C.c_float, _vp, _i64, _i64, _vp]),
    "cg_b200_reduce": (_i, [_i, _i, _vp, _vp, _i64, _i64, _i64, _vp]),
    "cg_b200_attention": (_i, [C.POINTER(AttentionDesc), _vp, _vp, _vp, _vp, _vp]),
    "cg_b200_gemm_workspace_bytes": (_i, [C.POINTER(GemmDesc), C.POINTER(_sz)]),
    "cg_b200_gemm": (_i, [C.POINTER(GemmDesc), _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "cg_b200_gemm_tuned": (_i, [C.POINTER(GemmDesc), C.POINTER(GemmTuning), _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "cg_b200_last_device_error": (_i, [_vp, C.POINTER(C.c_uint32)]),
    "cg_b200_gemm_f32_static": (_i, [C.POINTER(GemmDesc), _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "cg_b200_comm_unique_id": (_i, [_vp]),
    "cg_b200_comm_init_rank": (_i, [_vpp, _i, _i, _vp]),
    "cg_b200_allgather_inplace": (_i, [_vp, _vp, _sz, _vp]),
    "cg_b200_comm_barrier": (_i, [_vp, _vp]),
    "cg_b200_comm_destroy": (_i, [_vp]),
    "cg_b200_peer_barrier_create": (_i, [_vpp, _vpp, _i, _i]),
    "cg_b200_peer_barrier": (_i, [_vp, _vp]),
    "cg_b200_peer_barrier_set_timeout": (_i, [_vp, C.c_uint64]),
    "cg_b200_peer_barrier_destroy": (_i, [_vp]),
    "cg_b200_ipc_export": (_i, [_vp, _vp]),
    "cg_b200_ipc_open": (_i, [_vp, _vpp]),
    "cg_b200_ipc_close": (_i, [_vp]),
    "cg_b200_gemm_allgather": (_i, [C.POINTER(GemmDesc), _vp, _vp, _vp, _vp, _vp, _vpp, _i, _i, _vp, _sz, _vp]),
    "cg_b200_gemm_allgather_sync": (_i, [C.POINTER(GemmDesc), C.POINTER(GemmTuning), _vp, _vp, _vp, _vp, _vp, _vpp, _i, _i, _vp,
                                         _vp, _sz, _vp]),
    "cg_b200_peer_push": (_i, [_vp, _vpp, _i, _i, _sz, _vp, _vp]),
}

_lib = None


def library_path():
    return os.path.join(_HERE, "lib", "libcg_b200.so")


def lib():
    """The loaded C-ABI library. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing. Build it with `python cantors-gift_b200/build.py`; "
                "cg_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status, what=""):
    if status != OK:
        raise CgB200Error(status, what)


def make_eltwise_desc(dtype, prog, bcast=(), inner=1, round_each_op=0):
    """prog: sequence of ("input", i) | ("imm", value) | "opname" in postfix order."""
    d = EltwiseDesc()
    d.dtype = dtype
    d.n_instr = len(prog)
    for i, ins in enumerate(prog[:EW_MAX_INSTR]):
        if isinstance(ins, str):
            d.prog[i].op = EW_OPS[ins]
        elif ins[0] == "input":
            d.prog[i].op, d.prog[i].arg = EW_OPS["input"], int(ins[1])
        elif ins[0] == "imm":
            d.prog[i].op, d.prog[i].imm = EW_OPS["imm"], float(ins[1])
        else:
            raise ValueError(f"bad eltwise instruction {ins!r}")
    for i, b in enumerate(bcast):
        d.bcast[i] = BCAST[b] if isinstance(b, str) else int(b)
    d.inner = inner
    d.round_each_op = round_each_op
    return d


def make_gemm_desc(M, N, K, in_dtype, out_dtype, epilogue="none", batch=1, b_transposed=0,
                   lda=None, ldb=None, ldc=None, bsa=None, bsb=None, bsc=None, compute="default",
                   alpha=1.0, batch_inner=0, isa=0, isb=0, isc=0):
    d = GemmDesc()
    d.M, d.N, d.K, d.batch = M, N, K, batch
    d.lda = K if lda is None else lda
    d.ldb = (K if b_transposed else N) if ldb is None else ldb
    d.ldc = N if ldc is None else ldc
    d.batch_stride_a = M * d.lda if bsa is None else bsa
    d.batch_stride_b = (N if b_transposed else K) * d.ldb if bsb is None else bsb
    d.batch_stride_c = M * d.ldc if bsc is None else bsc
    d.in_dtype, d.out_dtype = in_dtype, out_dtype
    d.compute = COMPUTE[compute] if isinstance(compute, str) else compute
    d.epilogue = EPILOGUE[epilogue] if isinstance(epilogue, str) else epilogue
    d.b_transposed = b_transposed
    d.alpha = alpha
    d.batch_inner, d.inner_stride_a, d.inner_stride_b, d.inner_stride_c = batch_inner, isa, isb, isc
    return d
