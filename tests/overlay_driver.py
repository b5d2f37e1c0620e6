"""Runs graphs through the reference's own Python module (cantors_gift, built unmodified against the B200
layer) plus cg_b200_ext on cuda:0 and checks them against the CPU oracle. Started as a child process by
test_reference_overlay.py: the two pybind11 modules live apart from any other extension the test process
may have loaded.

    python overlay_driver.py chain | block | block_full
"""
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "cantors-gift_b200", "host", "_overlay", "python", "cantors_gift"))

import cantors_gift as cg  # noqa: E402
import cg_b200_ext as ext  # noqa: E402
from oracle import oracle as O  # noqa: E402
from oracle import transformer as T  # noqa: E402


def compile_and_bind(m, rt):
    cgm = cg.TensorToCodegenLowering().lower(m)
    assert ext.last_lowering_status() == 0, ext.last_lowering_message()
    exe = cg.NvidiaBackend("sm_100a").compile(cgm)
    bound = ext.bind(rt, exe, 0)
    assert bound is not None, "Runtime.bind returned None"
    return exe, bound


def upload(rt, stream, host, dtype):
    t = ext.alloc(rt, list(host.shape), dtype)
    assert ext.copy_to_device(t, np.ascontiguousarray(host), stream) == 0
    return t


def chain(rt, stream):
    """y = relu(a*b + c) * 0.5 over 2^20 + 5 fp32 elements: bit-exact against the oracle."""
    n = (1 << 20) + 5
    m = cg.Module()
    ty = cg.tensor_type([n], cg.DType.F32)
    f = m.create_function("chain", [ty, ty, ty], [ty])
    b = cg.Builder(f)
    a = f.args()
    half = b.constant_tensor([], cg.DType.F32, np.float32(0.5).tobytes())
    b.output_tensor(b.mul(b.relu(b.add(b.mul(a[0], a[1]), a[2])), half))
    exe, bound = compile_and_bind(m, rt)
    assert ext.plan_summary(exe) == ["eltwise"]
    assert "ld.global" in exe.ptx_text or ".entry" in exe.ptx_text      # the old emitter's text is still there
    rng = np.random.default_rng(1)
    host = [rng.standard_normal(n, dtype=np.float32) for _ in range(3)]
    dev = [upload(rt, stream, h, cg.DType.F32) for h in host]
    out = ext.alloc(rt, [n], cg.DType.F32)
    assert bound.launch(dev, [out], stream) == 0
    got = np.empty(n, dtype=np.float32)
    assert ext.copy_to_host(got, out, stream) == 0
    prog = [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu", ("imm", 0.5), "mul"]
    want = O.eltwise(O.make_eltwise_desc(O.F32, prog, ["full"] * 3), host, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), "chain differs from the oracle"
    print("chain ok")


def encoder_block_graph(B, S, D, H, F, dt):
    dh = D // H
    m = cg.Module()
    t = lambda *s: cg.tensor_type(list(s), dt)  # noqa: E731
    f = m.create_function("encoder_block", [t(B, S, D), t(D, 3 * D), t(D, D), t(D, F), t(F), t(F, D), t(D)], [t(B, S, D)])
    b = cg.Builder(f)
    a = f.args()
    x = a[0]
    qkv = b.matmul(b.layernorm(x), a[1])

    def heads(i):
        part = b.slice(qkv, [0, 0, i * D], [B, S, (i + 1) * D])
        return b.transpose(b.reshape(part, [B, S, H, dh]), [0, 2, 1, 3])

    q, k, v = heads(0), heads(1), heads(2)
    scale = O.to_bf16(np.array([1.0 / math.sqrt(dh)], dtype=np.float32))
    sc = b.constant_tensor([], dt, scale.tobytes())
    ctx = b.matmul(b.softmax(b.mul(b.matmul(q, b.transpose(k, [0, 1, 3, 2])), sc)), v)
    merged = b.reshape(b.transpose(ctx, [0, 2, 1, 3]), [B, S, D])
    h = b.add(b.matmul(merged, a[2]), x)
    ff = b.gelu(b.add(b.matmul(b.layernorm(h), a[3]), a[4]))
    b.output_tensor(b.add(b.add(b.matmul(ff, a[5]), a[6]), h))
    return m


def block(rt, stream, B, S, D, H, F, check_sequences):
    """The pre-LN encoder block as a Tensor-IR graph: seven kernels, checked against oracle/transformer.py."""
    m = encoder_block_graph(B, S, D, H, F, cg.DType.BF16)
    exe, bound = compile_and_bind(m, rt)
    assert ext.plan_summary(exe) == ["layernorm", "gemm", "attention", "gemm", "layernorm", "gemm", "gemm"], ext.plan_summary(exe)
    rng = np.random.default_rng(B * 1000 + S)
    bf = lambda *s, scale=1.0: O.to_bf16(rng.standard_normal(s, dtype=np.float32) * scale)  # noqa: E731
    x = bf(B, S, D)
    w = dict(w_qkv=bf(D, 3 * D, scale=0.02), w_o=bf(D, D, scale=0.02), w_1=bf(D, F, scale=0.02), b_1=bf(F, scale=0.02),
             w_2=bf(F, D, scale=0.02), b_2=bf(D, scale=0.02))
    order = ["w_qkv", "w_o", "w_1", "b_1", "w_2", "b_2"]
    dev = [upload(rt, stream, x, cg.DType.BF16)] + [upload(rt, stream, w[k], cg.DType.BF16) for k in order]
    out = ext.alloc(rt, [B, S, D], cg.DType.BF16)
    assert bound.launch(dev, [out], stream) == 0, ext.status_string(ext.last_launch_status())
    got = np.empty((B, S, D), dtype=np.uint16)
    assert ext.copy_to_host(got, out, stream) == 0
    for s in check_sequences:
        want = O.from_bf16(T.encoder_block(x[s:s + 1], n_heads=H, dtype=O.BF16, **w))
        g = O.from_bf16(got[s:s + 1])
        err = np.abs(g - want)
        norm = err.max() / np.abs(want).max()
        rms = math.sqrt((err ** 2).mean()) / math.sqrt((want ** 2).mean())
        assert norm <= 1e-2 and rms <= 1e-2, f"sequence {s}: max-normalised {norm:.3e}, rms ratio {rms:.3e}"
    print(f"block B{B} S{S} D{D} H{H} F{F} ok")


def main():
    what = sys.argv[1]
    rt = cg.Runtime()
    assert ext.add_cuda_device(rt, 0), "no usable sm_100 device"
    stream = ext.create_stream(rt, 0)
    if what == "chain":
        chain(rt, stream)
    elif what == "block":
        block(rt, stream, 2, 128, 128, 2, 512, [0, 1])
        block(rt, stream, 3, 200, 256, 4, 384, [0, 2])
    elif what == "block_full":
        block(rt, stream, 32, 2048, 1024, 16, 4096, [5])
    else:
        raise SystemExit(f"unknown case {what}")


if __name__ == "__main__":
    main()
