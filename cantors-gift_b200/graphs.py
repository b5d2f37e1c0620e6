"""Tensor-IR graphs of the configured workloads, built with the reference's own Python module, and the
loader of that module as built against the B200 layer.

`cantors_gift` here is the reference's python/bindings.cpp compiled unmodified against the library in
which this repository's backend / lowering / runtime / vendor layer stands in; `cg_b200_ext` adds
what that file does not bind (CUDA devices, tensors over foreign memory, bind, launch). Both are
build products of host/Makefile. Import torch BEFORE calling host_modules() in a process that uses
both: the other order crashes inside pybind11's shared state.
"""
import math
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
MODULE_DIR = os.path.join(_HERE, "host", "_overlay", "python", "cantors_gift")


def host_modules():
    """(cantors_gift, cg_b200_ext). Raises ImportError with the build hint when they are not built."""
    if MODULE_DIR not in sys.path:
        sys.path.insert(0, MODULE_DIR)
    try:
        import cantors_gift as cg
        import cg_b200_ext as ext
    except ImportError as e:
        raise ImportError(f"{e}; build the host layer with `python __graft_entry__.py` where the reference "
                          "source tree is present") from e
    return cg, ext


def scalar_bytes(value, np_dtype_bits):
    """Little-endian bytes of `value` as fp32 (32) or bf16 (16, round to nearest even)."""
    import struct
    w = struct.unpack("<I", struct.pack("<f", value))[0]
    if np_dtype_bits == 32:
        return struct.pack("<I", w)
    w += 0x7FFF + ((w >> 16) & 1)
    return struct.pack("<H", (w >> 16) & 0xFFFF)


def chain_graph(cg, n):
    """cfg2: y = relu(a*b + c) * 0.5 over n fp32 elements."""
    m = cg.Module()
    ty = cg.tensor_type([n], cg.DType.F32)
    f = m.create_function("chain", [ty, ty, ty], [ty])
    b = cg.Builder(f)
    a = f.args()
    half = b.constant_tensor([], cg.DType.F32, scalar_bytes(0.5, 32))
    b.output_tensor(b.mul(b.relu(b.add(b.mul(a[0], a[1]), a[2])), half))
    return m


def encoder_block_graph(cg, B, S, D, H, F, dtype, weights_out_in=False):
    """cfg5: pre-LN encoder block  h = x + W_o attn(LN(x));  y = h + W_2 gelu(W_1 LN(h) + b_1) + b_2
    with a packed QKV projection and H heads (the dataflow of the reference's
    benchmarks/benchmark_transformer.py:122-170, with heads, biases and the 1/sqrt(d_head) scale the
    configuration asks for). Function arguments: x [B,S,D], W_qkv, W_o, W_1, b_1, W_2, b_2.
    weights_out_in: the weight matrices are stored [out, in] and enter each matmul through a transpose
    (x @ W^T), the layout the tensor cores read without a transposing descriptor."""
    dh = D // H
    m = cg.Module()
    t = lambda *s: cg.tensor_type(list(s), dtype)  # noqa: E731
    w = (lambda i, o: t(o, i)) if weights_out_in else (lambda i, o: t(i, o))
    f = m.create_function("encoder_block", [t(B, S, D), w(D, 3 * D), w(D, D), w(D, F), t(F), w(F, D), t(D)], [t(B, S, D)])
    b = cg.Builder(f)
    a = f.args()
    W = (lambda v: b.transpose(v, [1, 0])) if weights_out_in else (lambda v: v)
    x = a[0]
    qkv = b.matmul(b.layernorm(x), W(a[1]))                       # [B, S, 3D]

    def heads(i):
        part = b.slice(qkv, [0, 0, i * D], [B, S, (i + 1) * D])
        return b.transpose(b.reshape(part, [B, S, H, dh]), [0, 2, 1, 3])   # [B, H, S, dh]

    q, k, v = heads(0), heads(1), heads(2)
    bits = 32 if dtype == cg.DType.F32 else 16
    if dtype == cg.DType.F16:
        raise ValueError("scalar constants are built for fp32 and bf16 graphs here")
    scale = b.constant_tensor([], dtype, scalar_bytes(1.0 / math.sqrt(dh), bits))
    ctx = b.matmul(b.softmax(b.mul(b.matmul(q, b.transpose(k, [0, 1, 3, 2])), scale)), v)   # [B, H, S, dh]
    merged = b.reshape(b.transpose(ctx, [0, 2, 1, 3]), [B, S, D])
    h = b.add(b.matmul(merged, W(a[2])), x)
    ff = b.gelu(b.add(b.matmul(b.layernorm(h), W(a[3])), a[4]))
    b.output_tensor(b.add(b.add(b.matmul(ff, W(a[5])), a[6]), h))
    return m


def compile_for_b200(cg, ext, module):
    """Lowers and compiles `module` for sm_100a; raises with the lowering's message when it has no plan."""
    cgm = cg.TensorToCodegenLowering().lower(module)
    if ext.last_lowering_status() != 0:
        raise RuntimeError("lowering: " + ext.last_lowering_message())
    return cg.NvidiaBackend("sm_100a").compile(cgm)
