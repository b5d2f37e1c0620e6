"""Pre-LN transformer encoder block out of the path's kernels (C-ABI calls only).

    h = x + W_o . attn(LN(x))            attn: softmax(Q K^T / sqrt(d_h)) V per head
    y = h + W_2 . gelu(W_1 . LN(h) + b_1) + b_2

The dataflow is the reference's transformer benchmark graph (benchmarks/benchmark_transformer.py:98-119:
layernorm eps 1e-5, GELU, no mask, no dropout); the reference only ever compiles that graph, it
never executes it (benchmarks/REPORT_TRANSFORMER.md:53-57). Seven launches per block:
  layernorm | QKV GEMM | fused attention (reads Q, K, V in place from the QKV rows, writes
  [B*S, d_model]) | out-proj GEMM + residual | layernorm | FFN1 GEMM + bias + gelu |
  FFN2 GEMM + bias + residual
Without the fused kernel (head_dim != 64, fp32) attention is three launches: Q K^T GEMM (heads as the
inner batch level, scale in the epilogue), row softmax, P V GEMM. fp32 GEMMs take one batch level, so an
fp32 block (the dtype of the reference's own graph; a functional path, not a tuned one) runs the two
attention GEMMs once per sequence with the heads as that level: 5 + 2 * B + 1 launches.
Weights are [in, out] row-major (x @ W), all tensors bf16/f16/f32 of one dtype.
"""
import ctypes as C
import math

import torch

from . import capi, ops
from .capi import check, lib
from .ops import DTYPE_OF_TORCH


class EncoderBlock:
    def __init__(self, d_model, n_heads, d_ff, w_qkv, w_o, w_1, b_1, w_2, b_2, eps=1e-5, fused_attention=True):
        assert d_model % n_heads == 0
        self.D, self.H, self.F, self.dh, self.eps = d_model, n_heads, d_ff, d_model // n_heads, eps
        self.w_qkv, self.w_o, self.w_1, self.b_1, self.w_2, self.b_2 = w_qkv, w_o, w_1, b_1, w_2, b_2
        assert tuple(w_qkv.shape) == (d_model, 3 * d_model) and tuple(w_o.shape) == (d_model, d_model)
        assert tuple(w_1.shape) == (d_model, d_ff) and tuple(w_2.shape) == (d_ff, d_model)
        # The weights are constants of the block: they are kept [N, K] (K contiguous), the operand layout the
        # tensor cores read without a transposing descriptor - 3-7 % faster than [K, N] at K = 1024.
        self._wt = {name: w.t().contiguous() for name, w in (("qkv", w_qkv), ("o", w_o), ("1", w_1), ("2", w_2))}
        self.dtype = w_qkv.dtype
        self.dt = DTYPE_OF_TORCH[self.dtype]
        self._bufs = {}
        # the fused kernel covers head_dim 64 and 16-bit types; otherwise three launches
        self.fused_attention = fused_attention and self.dh == 64 and self.dtype in (torch.bfloat16, torch.float16)

    def _buf(self, name, shape, device):
        t = self._bufs.get(name)
        if t is None or tuple(t.shape) != tuple(shape):
            t = torch.empty(shape, dtype=self.dtype, device=device)
            self._bufs[name] = t
        return t

    @staticmethod
    def flops(B, S, D, H, F):
        """Matmul FLOPs of one block, 2*batch*M*K*N per matmul as the reference counts them
        (src/analysis/arithmetic_intensity.cpp:73-89)."""
        return 2.0 * B * S * (3 * D * D + D * D + 2 * D * F) + 2.0 * 2 * B * H * S * S * (D // H)

    def forward(self, x, out=None, stream=None, gather=None):
        """x: [B, S, D] contiguous CUDA tensor. Returns y of the same shape.

        gather: for a batch-sharded block, (y_full_ptr, peer_table, world, rank): the last GEMM then
        writes this rank's rows of y into the full-size y of every rank (its own at y_full_ptr, the
        peers' through the `world` pointers of peer_table, mapped with cg_b200_ipc_open) as its tiles
        are produced, instead of an all-gather after the block. `out` is ignored; the caller runs one
        cg_b200_peer_barrier before y is read."""
        B, S, D = x.shape
        H, dh, F, dt = self.H, self.dh, self.F, self.dt
        dev = x.device
        L = lib()
        st = C.c_void_p((torch.cuda.current_stream() if stream is None else stream).cuda_stream)
        p = lambda t: None if t is None else C.c_void_p(t.data_ptr())  # noqa: E731
        rows = B * S
        x2 = x.view(rows, D)
        ln1 = self._buf("ln1", (rows, D), dev)
        qkv = self._buf("qkv", (rows, 3 * D), dev)
        scores = None if self.fused_attention else self._buf("scores", (B * H, S, S), dev)
        ctx = self._buf("ctx", (rows, D), dev)
        h = self._buf("h", (rows, D), dev)
        ln2 = self._buf("ln2", (rows, D), dev)
        ff = self._buf("ff", (rows, F), dev)
        y = None if gather is not None else (torch.empty_like(x) if out is None else out)

        def gemm(desc, a, b, c, bias=None, res=None, a_off=0, b_off=0):
            es = a.element_size()
            # fp32 operands TMA cannot read in place (unaligned base or stride) are rewritten into a workspace
            ws, ws_bytes = ops.gemm_workspace(desc, dev) if self.dtype == torch.float32 else (None, 0)
            check(L.cg_b200_gemm(C.byref(desc), C.c_void_p(a.data_ptr() + a_off * es), C.c_void_p(b.data_ptr() + b_off * es),
                                 p(bias), p(res), p(c), p(ws), ws_bytes, st), "gemm")

        check(L.cg_b200_layernorm(dt, p(x2), None, None, self.eps, p(ln1), rows, D, st), "layernorm")
        gemm(capi.make_gemm_desc(rows, 3 * D, D, dt, dt, b_transposed=1), ln1, self._wt["qkv"], qkv)
        if self.fused_attention:
            es = qkv.element_size()
            ad = capi.AttentionDesc(dtype=dt, head_dim=dh, batch=B, heads=H, seq_q=S, seq_kv=S, ldq=3 * D, ldk=3 * D,
                                    ldv=3 * D, ldo=D, head_stride_q=dh, head_stride_k=dh, head_stride_v=dh, head_stride_o=dh,
                                    batch_stride_q=S * 3 * D, batch_stride_k=S * 3 * D, batch_stride_v=S * 3 * D,
                                    batch_stride_o=S * D, scale=1.0 / math.sqrt(dh))
            base = qkv.data_ptr()
            check(L.cg_b200_attention(C.byref(ad), C.c_void_p(base), C.c_void_p(base + D * es),
                                      C.c_void_p(base + 2 * D * es), p(ctx), st), "attention")
        else:
            self._unfused_attention(qkv, scores, ctx, B, S, gemm, p, st)
        gemm(capi.make_gemm_desc(rows, D, D, dt, dt, epilogue="residual", b_transposed=1), ctx, self._wt["o"], h, res=x2)
        check(L.cg_b200_layernorm(dt, p(h), None, None, self.eps, p(ln2), rows, D, st), "layernorm")
        gemm(capi.make_gemm_desc(rows, F, D, dt, dt, epilogue="bias_gelu_tanh", b_transposed=1), ln2, self._wt["1"], ff,
             bias=self.b_1)
        d_out = capi.make_gemm_desc(rows, D, F, dt, dt, epilogue="bias_residual", b_transposed=1)
        if gather is None:
            gemm(d_out, ff, self._wt["2"], y.view(rows, D), bias=self.b_2, res=h)
            return y
        y_full, table, world, rank = gather
        check(L.cg_b200_gemm_allgather(C.byref(d_out), p(ff), p(self._wt["2"]), p(self.b_2), p(h), y_full, table, world, rank,
                                       None, 0, st), "gemm_allgather")
        return None

    def _unfused_attention(self, qkv, scores, ctx, B, S, gemm, p, st):
        D, H, dh, dt = self.D, self.H, self.dh, self.dt
        L = lib()
        scale = 1.0 / math.sqrt(dh)
        if self.dtype == torch.float32:
            # one batch level per launch: the heads of one sequence (stride dh in the qkv rows)
            d_qk = capi.make_gemm_desc(S, S, dh, dt, dt, epilogue="scale", alpha=scale, batch=H, b_transposed=1,
                                       lda=3 * D, ldb=3 * D, ldc=S, bsa=dh, bsb=dh, bsc=S * S)
            d_pv = capi.make_gemm_desc(S, dh, S, dt, dt, batch=H, lda=S, ldb=3 * D, ldc=D, bsa=S * S, bsb=dh, bsc=dh)
            for b in range(B):
                gemm(d_qk, qkv, qkv, scores[b * H:], a_off=b * S * 3 * D, b_off=b * S * 3 * D + D)
            check(L.cg_b200_softmax(dt, p(scores), p(scores), B * H * S, S, st), "softmax")
            for b in range(B):
                gemm(d_pv, scores[b * H:], qkv, ctx[b * S:], b_off=b * S * 3 * D + 2 * D)
            return
        # scores[b, h] = Q_bh K_bh^T / sqrt(dh): Q, K are column blocks of the qkv rows (row stride 3D);
        # heads are the inner batch level (stride dh), sequences the outer one (stride S * 3D)
        d_qk = capi.make_gemm_desc(S, S, dh, dt, dt, epilogue="scale", alpha=scale, batch=B * H,
                                   b_transposed=1, lda=3 * D, ldb=3 * D, ldc=S, batch_inner=H,
                                   bsa=S * 3 * D, bsb=S * 3 * D, bsc=H * S * S, isa=dh, isb=dh, isc=S * S)
        gemm(d_qk, qkv, qkv, scores, b_off=D)
        check(L.cg_b200_softmax(dt, p(scores), p(scores), B * H * S, S, st), "softmax")
        # ctx[b, :, h*dh:(h+1)*dh] = P_bh V_bh, V_bh = qkv[b, :, 2D + h*dh : ...] ([S, dh], N contiguous)
        d_pv = capi.make_gemm_desc(S, dh, S, dt, dt, batch=B * H, lda=S, ldb=3 * D, ldc=D, batch_inner=H,
                                   bsa=H * S * S, bsb=S * 3 * D, bsc=S * D, isa=S * S, isb=dh, isc=dh)
        gemm(d_pv, scores, qkv, ctx, b_off=2 * D)

    @property
    def launches_per_forward(self):
        """16-bit types; an fp32 block launches 6 + 2 * batch kernels."""
        return 7 if self.fused_attention else 9
