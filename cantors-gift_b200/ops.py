"""Host-side calls of the C ABI on torch CUDA tensors and on host (NumPy / pinned) buffers.

PyTorch is used for device memory and streams only; every computation is a cg_b200_* call.
bf16 host arrays travel as uint16 bit patterns.
"""
import ctypes as C

import numpy as np
import torch

from . import capi
from .capi import BF16, F16, F32, check, lib

TORCH_DTYPE = {F32: torch.float32, BF16: torch.bfloat16, F16: torch.float16}
DTYPE_OF_TORCH = {v: k for k, v in TORCH_DTYPE.items()}


def _stream(stream=None):
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("cg_b200 ops take contiguous CUDA tensors")


def eltwise(desc, inputs, out, n=None, stream=None):
    _require_cuda(out, *inputs)
    n = out.numel() if n is None else n
    arr = (C.c_void_p * max(1, len(inputs)))(*[t.data_ptr() for t in inputs])
    check(lib().cg_b200_eltwise(C.byref(desc), arr, len(inputs), _ptr(out), n, _stream(stream)), "eltwise")
    return out


def softmax(x, out=None, stream=None):
    _require_cuda(x, out)
    out = torch.empty_like(x) if out is None else out
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    check(lib().cg_b200_softmax(DTYPE_OF_TORCH[x.dtype], _ptr(x), _ptr(out), rows, cols, _stream(stream)), "softmax")
    return out


def layernorm(x, gamma=None, beta=None, eps=1e-5, out=None, stream=None):
    _require_cuda(x, out, gamma, beta)
    out = torch.empty_like(x) if out is None else out
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    check(lib().cg_b200_layernorm(DTYPE_OF_TORCH[x.dtype], _ptr(x), _ptr(gamma), _ptr(beta), eps, _ptr(out),
                                  rows, cols, _stream(stream)), "layernorm")
    return out


def softmax_layernorm(x, gamma=None, beta=None, eps=1e-5, out=None, stream=None):
    _require_cuda(x, out, gamma, beta)
    out = torch.empty_like(x) if out is None else out
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    check(lib().cg_b200_softmax_layernorm(DTYPE_OF_TORCH[x.dtype], _ptr(x), _ptr(gamma), _ptr(beta), eps,
                                          _ptr(out), rows, cols, _stream(stream)), "softmax_layernorm")
    return out


def reduce_box(shape, axes):
    """(outer, reduce, inner) of a row-major tensor reduced over `axes`, or None when the axes are not a run of
    adjacent ones (no kernel then). Negative axes count from the end, as in the reference's shape inference."""
    rank = len(shape)
    ax = sorted({a + rank if a < 0 else a for a in axes})
    if not ax or ax[0] < 0 or ax[-1] >= rank or ax != list(range(ax[0], ax[-1] + 1)):
        return None
    outer = inner = red = 1
    for i, d in enumerate(shape):
        if i < ax[0]:
            outer *= d
        elif i > ax[-1]:
            inner *= d
        else:
            red *= d
    return outer, red, inner


def reduce(x, op, axes, keep_dims=False, out=None, stream=None):
    """reduce_sum / reduce_max / reduce_mean (op: "sum" | "max" | "mean") of a contiguous tensor over adjacent axes."""
    _require_cuda(x, out)
    box = reduce_box(tuple(x.shape), axes)
    if box is None or not x.is_contiguous():
        raise ValueError("reduce: the axes must be adjacent and the tensor contiguous")
    outer, red, inner = box
    rank = x.dim()
    ax = {a + rank if a < 0 else a for a in axes}
    shape = [1 if i in ax else d for i, d in enumerate(x.shape) if keep_dims or i not in ax]
    out = torch.empty(shape, dtype=x.dtype, device=x.device) if out is None else out
    check(lib().cg_b200_reduce(DTYPE_OF_TORCH[x.dtype], capi.REDUCE[op], _ptr(x), _ptr(out), outer, red, inner,
                               _stream(stream)), "reduce")
    return out


_workspaces = {}


def gemm_workspace(desc, device):
    need = C.c_size_t(0)
    check(lib().cg_b200_gemm_workspace_bytes(C.byref(desc), C.byref(need)), "gemm_workspace_bytes")
    if need.value == 0:
        return None, 0
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need.value:
        ws = torch.empty(need.value, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws, ws.numel()


def gemm(desc, A, B, C_out, bias=None, residual=None, workspace=None, stream=None, tuning=None):
    """`tuning`: a capi.GemmTuning (an autotuner's tile choice) or None for the library's heuristic."""
    _require_cuda(A, B, C_out, bias, residual)
    if workspace is None:
        workspace, ws_bytes = gemm_workspace(desc, A.device)
    else:
        ws_bytes = workspace.numel() * workspace.element_size()
    if tuning is None:
        check(lib().cg_b200_gemm(C.byref(desc), _ptr(A), _ptr(B), _ptr(bias), _ptr(residual), _ptr(C_out),
                                 _ptr(workspace), ws_bytes, _stream(stream)), "gemm")
    else:
        check(lib().cg_b200_gemm_tuned(C.byref(desc), C.byref(tuning), _ptr(A), _ptr(B), _ptr(bias), _ptr(residual),
                                       _ptr(C_out), _ptr(workspace), ws_bytes, _stream(stream)), "gemm_tuned")
    return C_out


def last_device_error(stream=None):
    w = C.c_uint32(0)
    check(lib().cg_b200_last_device_error(_stream(stream), C.byref(w)), "last_device_error")
    return w.value


# ---- host-buffer entry (the call a user of the reference's Runtime would make) ------------------
class HostRunner:
    """Runs one op with HOST inputs and outputs: H2D copies, the kernel, D2H copy, sync.

    Device buffers and pinned staging are allocated once through the C ABI and reused, as a
    bound executable would hold them.
    """

    def __init__(self):
        self._dev = {}
        self.stream = C.c_void_p()
        check(lib().cg_b200_stream_create(C.byref(self.stream)), "stream_create")

    def dev(self, name, nbytes):
        cur = self._dev.get(name)
        if cur is None or cur[1] < nbytes:
            if cur is not None:
                check(lib().cg_b200_free(cur[0]), "free")
            p = C.c_void_p()
            check(lib().cg_b200_malloc(C.byref(p), nbytes), "malloc")
            cur = (p, nbytes)
            self._dev[name] = cur
        return cur[0]

    def h2d(self, name, host):
        """host: pinned torch tensor or numpy array."""
        nbytes = host.numel() * host.element_size() if hasattr(host, "numel") else host.nbytes
        src = host.data_ptr() if hasattr(host, "data_ptr") else host.ctypes.data
        d = self.dev(name, nbytes)
        check(lib().cg_b200_memcpy_h2d(d, C.c_void_p(src), nbytes, self.stream), "memcpy_h2d")
        return d

    def d2h(self, host, dev, nbytes=None):
        n = (host.numel() * host.element_size() if hasattr(host, "numel") else host.nbytes) if nbytes is None else nbytes
        dst = host.data_ptr() if hasattr(host, "data_ptr") else host.ctypes.data
        check(lib().cg_b200_memcpy_d2h(C.c_void_p(dst), dev, n, self.stream), "memcpy_d2h")

    def sync(self):
        check(lib().cg_b200_stream_sync(self.stream), "stream_sync")

    # ---- slab pipeline: copy in, compute, copy out on three streams ------------------------------
    # PCIe moves data in both directions at once and the copy engines run beside the SMs, so a step
    # whose input splits into independent slabs (row blocks of A, sequences of a batch, ranges of an
    # elementwise array) costs about max(copy in, compute, copy out) instead of their sum.
    def _pipeline_streams(self):
        if not hasattr(self, "_s_compute"):
            self._s_compute, self._s_out = C.c_void_p(), C.c_void_p()
            check(lib().cg_b200_stream_create(C.byref(self._s_compute)), "stream_create")
            check(lib().cg_b200_stream_create(C.byref(self._s_out)), "stream_create")
            self._events = []
        return self._s_compute, self._s_out

    def _event(self, i):
        while len(self._events) <= i:
            e = C.c_void_p()
            check(lib().cg_b200_event_create(C.byref(e)), "event_create")
            self._events.append(e)
        return self._events[i]

    def run_slabs(self, n_slabs, copy_in, compute, copy_out):
        """copy_in(i, stream), compute(i, stream), copy_out(i, stream) enqueue slab i's work on the
        stream they are given; anything all slabs share (weights, B) is copied on self.stream by the
        caller before this. Returns after everything has finished."""
        s_in = self.stream
        s_compute, s_out = self._pipeline_streams()
        for i in range(n_slabs):
            copy_in(i, s_in)
            ev_in = self._event(2 * i)
            check(lib().cg_b200_event_record(ev_in, s_in), "event_record")
            check(lib().cg_b200_stream_wait_event(s_compute, ev_in), "stream_wait_event")
            compute(i, s_compute)
            ev_done = self._event(2 * i + 1)
            check(lib().cg_b200_event_record(ev_done, s_compute), "event_record")
            check(lib().cg_b200_stream_wait_event(s_out, ev_done), "stream_wait_event")
            copy_out(i, s_out)
        check(lib().cg_b200_stream_sync(s_out), "stream_sync")
        check(lib().cg_b200_stream_sync(s_compute), "stream_sync")
        check(lib().cg_b200_stream_sync(s_in), "stream_sync")

    def close(self):
        for p, _ in self._dev.values():
            lib().cg_b200_free(p)
        self._dev = {}
        for e in getattr(self, "_events", []):
            lib().cg_b200_event_destroy(e)
        self._events = []
        for name in ("_s_compute", "_s_out"):
            if hasattr(self, name):
                lib().cg_b200_stream_destroy(getattr(self, name))
                delattr(self, name)
        if self.stream:
            lib().cg_b200_stream_destroy(self.stream)
            self.stream = C.c_void_p()
