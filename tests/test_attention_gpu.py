"""Fused attention (tcgen05) against the CPU oracle, through the C ABI. Tolerance: the path's 16-bit
bound, 1e-2, on the max-normalised error and the RMS ratio (conftest.assert_close_rms)."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_close_rms as assert_close

pytestmark = pytest.mark.gpu


def _dev(ops, a, dtype):
    import torch
    return torch.from_numpy(a.view(np.int16)).cuda().view(ops.TORCH_DTYPE[dtype])


def _host(O, t, dtype):
    import torch
    return O.to_f32(t.cpu().view(torch.int16).numpy().view(np.uint16 if dtype == O.BF16 else np.float16), dtype)


def _run_contiguous(ops, cgb, oracle, dtype_name, B, H, Sq, Skv, scale=0.125, spread=1.0):
    import torch
    capi, O = cgb.capi, oracle
    dtype = getattr(capi, dtype_name)
    d = 64
    rng = np.random.default_rng(B * 100 + Sq + Skv)
    q, k, v = (O.to_storage(rng.standard_normal(s, dtype=np.float32) * f, dtype)
               for s, f in (((B, H, Sq, d), spread), ((B, H, Skv, d), spread), ((B, H, Skv, d), 1.0)))
    want = O.to_f32(O.attention(q, k, v, dtype, scale), dtype)
    desc = capi.AttentionDesc(dtype=dtype, head_dim=d, batch=B, heads=H, seq_q=Sq, seq_kv=Skv, ldq=d, ldk=d, ldv=d, ldo=d,
                              head_stride_q=Sq * d, head_stride_k=Skv * d, head_stride_v=Skv * d, head_stride_o=Sq * d,
                              batch_stride_q=H * Sq * d, batch_stride_k=H * Skv * d, batch_stride_v=H * Skv * d,
                              batch_stride_o=H * Sq * d, scale=scale)
    qd, kd, vd = (_dev(ops, np.ascontiguousarray(t), dtype) for t in (q, k, v))
    od = torch.zeros(B, H, Sq, d, dtype=ops.TORCH_DTYPE[dtype], device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    capi.check(cgb.lib().cg_b200_attention(C.byref(desc), p(qd), p(kd), p(vd), p(od),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream)), "attention")
    assert ops.last_device_error() == 0
    assert_close(_host(O, od, dtype), want, 1e-2, f"attention {dtype_name} B{B} H{H} Sq{Sq} Skv{Skv}")


@pytest.mark.parametrize("dtype_name", ["BF16", "F16"])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 1, 128, 128), (2, 3, 256, 384), (1, 2, 100, 200), (2, 2, 130, 77), (1, 1, 1, 1)])
def test_attention_contiguous_heads(ops, cgb, oracle, dtype_name, B, H, Sq, Skv):
    _run_contiguous(ops, cgb, oracle, dtype_name, B, H, Sq, Skv)


# The kernel's CTAs are persistent (one per SM) over units of 256 query rows, with rings of 5 K/V
# stages and 3 score buffers: more units than SMs, key-tile counts that wrap the rings, a second
# query tile that lies wholly past the end, and both ragged edges at once.
@pytest.mark.parametrize("B,H,Sq,Skv", [(40, 4, 256, 256), (1, 2, 300, 1000), (3, 50, 64, 640), (1, 1, 257, 129),
                                         (4, 40, 100, 100), (2, 80, 130, 300)])
def test_attention_persistent_units_and_ring_wraps(ops, cgb, oracle, B, H, Sq, Skv):
    _run_contiguous(ops, cgb, oracle, "BF16", B, H, Sq, Skv)


def test_attention_wide_score_range(ops, cgb, oracle):
    """Scores with a standard deviation of 32: the running row maximum moves by tens from tile to
    tile, so the rescale of the running sum and output by 2^(m_old - m_new) does real work."""
    _run_contiguous(ops, cgb, oracle, "BF16", 1, 2, 256, 768, scale=0.5, spread=2.0)


def test_attention_on_packed_qkv_rows(ops, cgb, oracle):
    """Q, K, V are column blocks of one [B*S, 3*D] buffer and O is written into [B*S, D]: the layout the
    encoder block uses."""
    import torch
    capi, O = cgb.capi, oracle
    B, H, S, d = 2, 4, 320, 64
    D = H * d
    rng = np.random.default_rng(3)
    qkv = O.to_bf16(rng.standard_normal((B * S, 3 * D), dtype=np.float32))
    f = O.from_bf16(qkv).reshape(B, S, 3, H, d)
    pick = lambda i: O.to_bf16(np.ascontiguousarray(f[:, :, i].transpose(0, 2, 1, 3)))  # noqa: E731  -> [B, H, S, d]
    want = O.from_bf16(O.attention(pick(0), pick(1), pick(2), O.BF16, 0.125)).transpose(0, 2, 1, 3).reshape(B * S, D)
    desc = capi.AttentionDesc(dtype=capi.BF16, head_dim=d, batch=B, heads=H, seq_q=S, seq_kv=S, ldq=3 * D, ldk=3 * D, ldv=3 * D,
                              ldo=D, head_stride_q=d, head_stride_k=d, head_stride_v=d, head_stride_o=d,
                              batch_stride_q=S * 3 * D, batch_stride_k=S * 3 * D, batch_stride_v=S * 3 * D,
                              batch_stride_o=S * D, scale=0.125)
    qd = _dev(ops, qkv, capi.BF16)
    od = torch.zeros(B * S, D, dtype=torch.bfloat16, device="cuda")
    base, es = qd.data_ptr(), 2
    capi.check(cgb.lib().cg_b200_attention(C.byref(desc), C.c_void_p(base), C.c_void_p(base + D * es), C.c_void_p(base + 2 * D * es),
                                           C.c_void_p(od.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)),
               "attention")
    assert ops.last_device_error() == 0
    assert_close(_host(O, od, capi.BF16), want, 1e-2, "attention on packed qkv")
