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

import cantors_gift_b200  # noqa: E402,F401
from cantors_gift_b200 import graphs  # noqa: E402
from oracle import oracle as O  # noqa: E402
from oracle import transformer as T  # noqa: E402

cg, ext = graphs.host_modules()


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
    exe, bound = compile_and_bind(graphs.chain_graph(cg, n), rt)
    assert ext.plan_summary(exe) == ["eltwise"]
    assert ".entry" in exe.ptx_text and "ld.global" in exe.ptx_text      # the old emitter's text is still there
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


def block(rt, stream, B, S, D, H, F, check_sequences, weights_out_in=False):
    """The pre-LN encoder block as a Tensor-IR graph: seven kernels, checked against oracle/transformer.py."""
    m = graphs.encoder_block_graph(cg, B, S, D, H, F, cg.DType.BF16, weights_out_in=weights_out_in)
    exe, bound = compile_and_bind(m, rt)
    assert ext.plan_summary(exe) == ["layernorm", "gemm", "attention", "gemm", "layernorm", "gemm", "gemm"], ext.plan_summary(exe)
    rng = np.random.default_rng(B * 1000 + S)
    bf = lambda *s, scale=1.0: O.to_bf16(rng.standard_normal(s, dtype=np.float32) * scale)  # noqa: E731
    x = bf(B, S, D)
    w = dict(w_qkv=bf(D, 3 * D, scale=0.02), w_o=bf(D, D, scale=0.02), w_1=bf(D, F, scale=0.02), b_1=bf(F, scale=0.02),
             w_2=bf(F, D, scale=0.02), b_2=bf(D, scale=0.02))
    order = ["w_qkv", "w_o", "w_1", "b_1", "w_2", "b_2"]
    stored = lambda k: w[k].T if (weights_out_in and w[k].ndim == 2) else w[k]  # noqa: E731
    dev = [upload(rt, stream, x, cg.DType.BF16)] + [upload(rt, stream, stored(k), cg.DType.BF16) for k in order]
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
        block(rt, stream, 2, 136, 128, 2, 256, [1], weights_out_in=True)
    elif what == "block_full":
        block(rt, stream, 32, 2048, 1024, 16, 4096, [5])
    else:
        raise SystemExit(f"unknown case {what}")


if __name__ == "__main__":
    main()
