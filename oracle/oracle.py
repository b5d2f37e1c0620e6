"""ctypes front end of the CPU oracle.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
leg of bench.py. The product package never imports this module.

Two shared objects are loaded from this directory:
  libcg_oracle.so     - the C restatement (cg_oracle.c)
  _ref/libcg_ref.so   - the reference project's own X86Emitter + JITMemory plus the driver
                        that assembles its benchmark kernels (ref_kernels.cpp); optional
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

F16, BF16, F32 = 0, 1, 2
NP_OF = {F16: np.float16, BF16: np.uint16, F32: np.float32}

EW_MAX_INSTR, EW_MAX_INPUTS = 16, 8


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


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "libcg_oracle.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} missing: run `make -C oracle` (or __graft_entry__.build())")
        L = C.CDLL(path)
        L.cgo_eltwise.argtypes = [C.POINTER(EltwiseDesc), C.POINTER(C.c_void_p), C.c_int,
                                  C.c_void_p, C.c_size_t]
        L.cgo_eltwise_validate.argtypes = [C.POINTER(EltwiseDesc), C.c_int]
        L.cgo_gemm.argtypes = [C.POINTER(GemmDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                               C.c_void_p, C.c_void_p, C.c_int64, C.c_int]
        for name in ("cgo_softmax",):
            getattr(L, name).argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
        for name in ("cgo_layernorm", "cgo_softmax_layernorm"):
            getattr(L, name).argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                         C.c_void_p, C.c_int64, C.c_int64]
        for name in ("cgo_f32_to_bf16", "cgo_bf16_to_f32", "cgo_f32_to_f16", "cgo_f16_to_f32"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
            getattr(L, name).restype = None
        L.cgo_set_num_threads.argtypes = [C.c_int]
        L.cgo_set_num_threads.restype = None
        _lib = L
    return _lib


def have_ref():
    return os.path.exists(os.path.join(_HERE, "_ref", "libcg_ref.so"))


def ref():
    """The reference project's own JIT kernels (None-safe: raises if not built)."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libcg_ref.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} missing: needs the reference tree at build time")
        L = C.CDLL(path)
        L.cgref_binary.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint]
        L.cgref_fma_relu_scale.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p,
                                           C.c_uint64, C.c_uint]
        L.cgref_matmul.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
        _ref = L
    return _ref


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _check(st, what):
    if st != 0:
        raise RuntimeError(f"oracle {what} failed with status {st}")


def num_threads():
    return lib().cgo_num_threads()


def set_num_threads(n):
    lib().cgo_set_num_threads(int(n))


# ---- dtype helpers (bf16 travels as uint16 bit patterns) -----------------------------------
def to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().cgo_f32_to_bf16(_p(x), _p(out), x.size)
    return out


def from_bf16(h):
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().cgo_bf16_to_f32(_p(h), _p(out), h.size)
    return out


def to_storage(x, dtype):
    """fp32 array -> array in the storage representation of `dtype`."""
    if dtype == F32:
        return np.ascontiguousarray(x, dtype=np.float32)
    if dtype == BF16:
        return to_bf16(x)
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16)


def to_f32(a, dtype):
    if dtype == F32:
        return np.asarray(a, dtype=np.float32)
    if dtype == BF16:
        return from_bf16(a)
    return np.asarray(a).astype(np.float32)


# ---- eltwise ---------------------------------------------------------------------------------
OPS = {name: i for i, name in enumerate(
    ["input", "imm", "add", "sub", "mul", "div", "max", "min", "neg", "abs", "relu", "gelu_tanh",
     "tanh", "sigmoid", "exp", "log", "sqrt", "rsqrt"])}
BCAST = {"full": 0, "scalar": 1, "row": 2, "col": 3}


def make_eltwise_desc(dtype, prog, bcast=(), inner=1, round_each_op=0, cls=EltwiseDesc):
    """prog: sequence of ("input", i) | ("imm", v) | "opname"."""
    d = cls()
    d.dtype = dtype
    d.n_instr = len(prog)
    for i, ins in enumerate(prog[:EW_MAX_INSTR]):
        if isinstance(ins, str):
            d.prog[i].op = OPS[ins]
        elif ins[0] == "input":
            d.prog[i].op, d.prog[i].arg = OPS["input"], int(ins[1])
        elif ins[0] == "imm":
            d.prog[i].op, d.prog[i].imm = OPS["imm"], float(ins[1])
        else:
            raise ValueError(ins)
    for i, b in enumerate(bcast):
        d.bcast[i] = BCAST[b] if isinstance(b, str) else int(b)
    d.inner = inner
    d.round_each_op = round_each_op
    return d


def eltwise(desc, inputs, n):
    out = np.empty(n, dtype=NP_OF[desc.dtype])
    arr = (C.c_void_p * max(1, len(inputs)))(*[a.ctypes.data for a in inputs])
    _check(lib().cgo_eltwise(C.byref(desc), arr, len(inputs), _p(out), n), "eltwise")
    return out


# ---- gemm ------------------------------------------------------------------------------------
EPI = {"none": 0, "bias": 1, "bias_relu": 2, "bias_gelu_tanh": 3, "bias_residual": 4,
       "residual": 5, "scale": 6, "relu": 7, "gelu_tanh": 8}


def make_gemm_desc(M, N, K, in_dtype, out_dtype, epilogue="none", batch=1, b_transposed=0,
                   lda=None, ldb=None, ldc=None, bsa=None, bsb=None, bsc=None, compute=0, alpha=1.0,
                   cls=GemmDesc, batch_inner=0, isa=0, isb=0, isc=0):
    d = cls()
    d.M, d.N, d.K, d.batch = M, N, K, batch
    d.lda = K if lda is None else lda
    d.ldb = (K if b_transposed else N) if ldb is None else ldb
    d.ldc = N if ldc is None else ldc
    d.batch_stride_a = M * d.lda if bsa is None else bsa
    d.batch_stride_b = (N if b_transposed else K) * d.ldb if bsb is None else bsb
    d.batch_stride_c = M * d.ldc if bsc is None else bsc
    d.in_dtype, d.out_dtype = in_dtype, out_dtype
    d.compute = compute
    d.epilogue = EPI[epilogue] if isinstance(epilogue, str) else epilogue
    d.b_transposed = b_transposed
    d.alpha = alpha
    d.batch_inner, d.inner_stride_a, d.inner_stride_b, d.inner_stride_c = batch_inner, isa, isb, isc
    return d


def gemm(desc, A, B, bias=None, residual=None, rows=None, acc64=False, out=None):
    """Returns C [batch*M, ldc-strided] storage array; with `rows` only those rows are valid."""
    n_c = (desc.batch - 1) * desc.batch_stride_c + (desc.M - 1) * desc.ldc + desc.N
    if out is None:
        out = np.zeros(max(n_c, 0), dtype=NP_OF[desc.out_dtype])
    r = None if rows is None else np.ascontiguousarray(rows, dtype=np.int64)
    _check(lib().cgo_gemm(C.byref(desc), _p(A), _p(B), _p(bias), _p(residual), _p(out), _p(r),
                          0 if r is None else r.size, int(acc64)), "gemm")
    return out


# ---- row reductions ------------------------------------------------------------------------------
def softmax(x, dtype):
    out = np.empty_like(x)
    _check(lib().cgo_softmax(dtype, _p(x), _p(out), x.shape[0], x.shape[1]), "softmax")
    return out


def layernorm(x, dtype, gamma=None, beta=None, eps=1e-5):
    out = np.empty_like(x)
    _check(lib().cgo_layernorm(dtype, _p(x), _p(gamma), _p(beta), eps, _p(out), x.shape[0],
                               x.shape[1]), "layernorm")
    return out


def softmax_layernorm(x, dtype, gamma=None, beta=None, eps=1e-5):
    out = np.empty_like(x)
    _check(lib().cgo_softmax_layernorm(dtype, _p(x), _p(gamma), _p(beta), eps, _p(out), x.shape[0],
                                       x.shape[1]), "softmax_layernorm")
    return out


# ---- the reference's own kernels --------------------------------------------------------------
def ref_binary(mode, a, b, threads=1):
    """mode 0: a + b; mode 1: relu(a * b) - the reference's count-parameterised JIT kernels."""
    out = np.empty_like(a)
    _check(ref().cgref_binary(mode, _p(a), _p(b), _p(out), a.size, threads), "ref_binary")
    return out


def ref_fma_relu_scale(a, b, c, scale, threads=1, out=None):
    if out is None:
        out = np.empty_like(a)
    _check(ref().cgref_fma_relu_scale(_p(a), _p(b), _p(c), scale, _p(out), a.size, threads),
           "ref_fma_relu_scale")
    return out


def ref_matmul(A, B):
    M, K = A.shape
    N = B.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    _check(ref().cgref_matmul(_p(A), _p(B), _p(out), M, K, N), "ref_matmul")
    return out


# ---- attention (restatement: matmul, softmax, matmul with fp32 intermediates) --------------------
def reduce(x, dtype, op, axes, keep_dims=False):
    """reduce_sum / reduce_max / reduce_mean (op: "sum" | "max" | "mean") over `axes` of x in storage representation
    (src/ir/ops.cpp:74-102, 417-436: `axes`, `keep_dims`, result dtype = operand dtype). Sums in double, one
    rounding to `dtype`; max ignores NaN operands. PARITY UNPINNED: the reference lowers these ops to a Reduce
    instruction its emitters print as a comment (src/backend/ptx/ptx_emitter.cpp:136-142)."""
    f = to_f32(x, dtype).astype(np.float64)
    ax = tuple(axes)
    if op == "sum":
        r = f.sum(axis=ax, keepdims=keep_dims)
    elif op == "mean":
        r = f.mean(axis=ax, keepdims=keep_dims)
    else:
        r = np.fmax.reduce(f, axis=ax, keepdims=keep_dims)
    return to_storage(np.asarray(r, dtype=np.float32), dtype)


def attention(q, k, v, dtype, scale):
    """q: [B, H, Sq, d], k/v: [B, H, Skv, d] in storage representation. Scores and probabilities stay
    fp32 (no rounding between the three ops); the result is rounded to `dtype`. PARITY UNPINNED:
    the reference defines the ops (src/ir/ops.cpp) and annotates the pattern
    (src/optimization/graph/graph_pattern.cpp:61-85) but executes neither."""
    B, H, Sq, d = q.shape
    Skv = k.shape[2]
    out = np.empty((B, H, Sq, d), dtype=NP_OF[dtype])
    for b in range(B):
        for h in range(H):
            qf = np.ascontiguousarray(q[b, h])
            kf = np.ascontiguousarray(k[b, h])
            s = gemm(make_gemm_desc(Sq, Skv, d, dtype, F32, epilogue="scale", alpha=scale, b_transposed=1), qf, kf)
            p = softmax(s.reshape(Sq, Skv), F32)
            vf = to_f32(np.ascontiguousarray(v[b, h]), dtype)
            o = gemm(make_gemm_desc(Sq, d, Skv, F32, F32), p, vf).reshape(Sq, d)
            out[b, h] = to_storage(o, dtype)
    return out
