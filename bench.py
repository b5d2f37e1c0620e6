"""Benchmark of the B200 execution path for cantors-gift Executables.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm|eltwise|rowreduce|matmul_f32|block|attention]
                    [--impl ours|reference] [--no-also]

One JSON line on stdout (rank 0). The headline workload is the bf16 4096^3 GEMM with fused
bias + GELU(tanh) (TFLOP/s); the memory-bound kernels of the path (fused elementwise chain,
softmax -> layernorm; GB/s), the fp32 1024^3 matmul and the transformer encoder block (a Tensor-IR
graph lowered, compiled, bound and launched through the reference's own TensorToCodegenLowering /
NvidiaBackend / Runtime interfaces) are short entries under "also", repeated inside "roofline". With
N > 1 GPUs the GEMM is sharded along M and the block along the batch, the last GEMM's epilogue
stores into every rank's output (fused all-gather), "also" holds the block, and outside the timed
region every rank compares what it holds after the gather with the one-GPU result, bit for bit
("gather_check"). "library_baseline" is torch.matmul on the GEMM's operands. All inputs are seeded
synthetic data of the configured shapes.

Timing: W >= 3 warm-up steps, then K steps between two CUDA events on the launching stream,
bracketed by barrier + synchronize, max over ranks. Memory-bound workloads stream inputs larger
than L2 every step; the GEMMs rotate over buffer sets larger than L2. Tensor-bound fractions divide
by the measured burst peak when the timed region lasts under a second (sustained peak and nominal
2.25 PFLOP/s as side keys).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "fused bf16 GEMM TFLOP/s & elementwise/softmax GB/s vs roofline"
PROG_CHAIN = [("input", 0), ("input", 1), "mul", ("input", 2), "add", "relu", ("imm", 0.5), "mul"]

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (None until a capture exists for that kernel).
NCU_TRAFFIC_BYTES = {"gemm": 85168896, "eltwise": 1047363072, "rowreduce": 485570560, "matmul_f32": 8465408, "block": None,
                     "attention": None}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Samples taken before this call (start-up, warm-up) are left out of the summary."""
        self.first = len(self.lines)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines[getattr(self, "first", 0):]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---- workloads -----------------------------------------------------------------------------------
class Workload:
    """A step = one pass of the hot path over one batch of synthetic input."""
    name = ""
    unit = ""
    bound = ""
    dtype = ""
    launches_per_step = 1

    def setup(self, rank, world):
        raise NotImplementedError

    def step(self, i):
        raise NotImplementedError

    def work_per_step(self):            # in the metric's numerator unit (GB or TFLOP), whole job
        raise NotImplementedError

    def algorithmic_per_launch(self):   # bytes or flop of the dominant kernel, per launch, this rank
        raise NotImplementedError


class EltwiseWorkload(Workload):
    name, unit, bound, dtype = "eltwise", "GB/s", "hbm", "f32"
    n = 1 << 26

    def config(self, world):
        return {"workload": "cfg2: y=relu(a*b+c)*0.5 over 2^26 fp32 per GPU, one fused kernel",
                "elements_per_gpu": self.n, "l2": "inputs (768 MiB) larger than L2 every step",
                "parallelism": f"replicas x{world}"}

    def setup(self, rank, world):
        import torch
        from cantors_gift_b200 import capi
        self.world = world
        g = torch.Generator(device="cuda").manual_seed(1 + rank)
        self.ins = [torch.randn(self.n, device="cuda", generator=g) for _ in range(3)]
        self.out = torch.empty(self.n, device="cuda")
        self.desc = capi.make_eltwise_desc(capi.F32, PROG_CHAIN, ["full"] * 3)

    def step(self, i):
        from cantors_gift_b200 import ops
        ops.eltwise(self.desc, self.ins, self.out)

    def work_per_step(self):
        return 4 * 4 * self.n * self.world / 1e9

    def algorithmic_per_launch(self):
        return 4 * 4 * self.n

    # end to end: host buffers in, host buffer out
    def e2e_setup(self):
        import torch
        from cantors_gift_b200 import ops
        self.runner = ops.HostRunner()
        self.h_in = [t.cpu().pin_memory() for t in self.ins]
        self.h_out = torch.empty(self.n, dtype=torch.float32).pin_memory()
        return 3 * 4 * self.n, 4 * self.n

    def e2e_step(self):
        import ctypes as C
        from cantors_gift_b200 import capi
        # ranges of the arrays are independent: eight of them in flight on three streams
        r = self.runner
        L = capi.lib()
        d = [r.dev(f"in{k}", 4 * self.n) for k in range(3)]
        o = r.dev("out", 4 * self.n)
        slabs = 8
        per = self.n // slabs
        assert per * slabs == self.n and (per * 4) % 16 == 0
        nb = 4 * per
        hin, hout = [h.data_ptr() for h in self.h_in], self.h_out.data_ptr()

        def copy_in(i, s):
            for k in range(3):
                capi.check(L.cg_b200_memcpy_h2d(C.c_void_p(d[k].value + i * nb), C.c_void_p(hin[k] + i * nb), nb, s), "h2d")

        def compute(i, s):
            arr = (C.c_void_p * 3)(*[p.value + i * nb for p in d])
            capi.check(L.cg_b200_eltwise(C.byref(self.desc), arr, 3, C.c_void_p(o.value + i * nb), per, s), "eltwise")

        def copy_out(i, s):
            capi.check(L.cg_b200_memcpy_d2h(C.c_void_p(hout + i * nb), C.c_void_p(o.value + i * nb), nb, s), "d2h")

        r.run_slabs(slabs, copy_in, compute, copy_out)

    def cpu_baseline(self, budget_s, prefer_ref=True):
        from oracle import oracle as O
        n = self.n
        rng = np.random.default_rng(1)
        a, b, c = (rng.standard_normal(n, dtype=np.float32) for _ in range(3))
        out = np.empty_like(a)
        threads = os.cpu_count() or 1
        if prefer_ref and O.have_ref():
            kind = "reference"
            run = lambda: O.ref_fma_relu_scale(a, b, c, 0.5, threads=threads, out=out)  # noqa: E731
        else:
            kind = "port"
            O.set_num_threads(threads)
            d = O.make_eltwise_desc(O.F32, PROG_CHAIN, ["full"] * 3)
            run = lambda: O.eltwise(d, [a, b, c], n)  # noqa: E731
        run()
        t0 = time.perf_counter()
        reps = 0
        while reps < 3 or (time.perf_counter() - t0 < min(budget_s, 10.0) and reps < 200):
            run()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": 16 * n / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
                "sample": f"the full 2^26-element chain, {reps} repetitions"}, dt


class RowReduceWorkload(Workload):
    name, unit, bound, dtype = "rowreduce", "GB/s", "hbm", "bf16"
    rows, cols = 32768, 4096

    def config(self, world):
        return {"workload": "cfg4: layernorm(softmax(x)), bf16 [32768, 4096] per GPU, eps 1e-5, one fused kernel",
                "l2": "input + output (512 MiB) larger than L2 every step", "parallelism": f"replicas x{world}"}

    def setup(self, rank, world):
        import torch
        self.world = world
        g = torch.Generator(device="cuda").manual_seed(3 + rank)
        self.x = torch.randn(self.rows, self.cols, device="cuda", generator=g).to(torch.bfloat16)
        self.y = torch.empty_like(self.x)

    def step(self, i):
        from cantors_gift_b200 import ops
        ops.softmax_layernorm(self.x, eps=1e-5, out=self.y)

    def work_per_step(self):
        return 2 * 2 * self.rows * self.cols * self.world / 1e9

    def algorithmic_per_launch(self):
        return 2 * 2 * self.rows * self.cols

    def e2e_setup(self):
        import torch
        from cantors_gift_b200 import ops
        self.runner = ops.HostRunner()
        self.h_x = self.x.cpu().pin_memory()
        self.h_y = torch.empty_like(self.h_x).pin_memory()
        nb = 2 * self.rows * self.cols
        return nb, nb

    def e2e_step(self):
        # rows are independent: eight row blocks in flight on three streams
        import ctypes as C
        from cantors_gift_b200 import capi
        r = self.runner
        L = capi.lib()
        total = 2 * self.rows * self.cols
        d, o = r.dev("x", total), r.dev("y", total)
        slabs = 8
        per = self.rows // slabs
        assert per * slabs == self.rows
        nb = 2 * per * self.cols
        hx, hy = self.h_x.data_ptr(), self.h_y.data_ptr()

        def copy_in(i, s):
            capi.check(L.cg_b200_memcpy_h2d(C.c_void_p(d.value + i * nb), C.c_void_p(hx + i * nb), nb, s), "h2d")

        def compute(i, s):
            capi.check(L.cg_b200_softmax_layernorm(capi.BF16, C.c_void_p(d.value + i * nb), None, None, 1e-5,
                                                   C.c_void_p(o.value + i * nb), per, self.cols, s), "softmax_layernorm")

        def copy_out(i, s):
            capi.check(L.cg_b200_memcpy_d2h(C.c_void_p(hy + i * nb), C.c_void_p(o.value + i * nb), nb, s), "d2h")

        r.run_slabs(slabs, copy_in, compute, copy_out)

    def cpu_baseline(self, budget_s, prefer_ref=True):
        from oracle import oracle as O
        threads = os.cpu_count() or 1
        O.set_num_threads(threads)
        rows = 4096
        rng = np.random.default_rng(3)
        x = O.to_bf16(rng.standard_normal((rows, self.cols), dtype=np.float32))
        O.softmax_layernorm(x, O.BF16)
        t0 = time.perf_counter()
        reps = 0
        while reps < 2 or (time.perf_counter() - t0 < min(budget_s, 10.0) and reps < 100):
            O.softmax_layernorm(x, O.BF16)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": 4 * rows * self.cols / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                "sample": f"{rows} of {self.rows} rows, {reps} repetitions (the reference has no executable "
                          "softmax/layernorm)"}, dt * self.rows / rows


class GemmWorkload(Workload):
    """bf16 M=N=K=4096, C = gelu_tanh(A B + bias); M-sharded over the ranks, in-place all-gather."""
    name, unit, bound, dtype = "gemm", "TFLOP/s", "tensor", "bf16"
    M = N = K = 4096
    in_dtype_name, epilogue = "BF16", "bias_gelu_tanh"
    sets = 4

    def config(self, world):
        return {"workload": "cfg3: bf16 GEMM M=N=K=4096 + bias + GELU(tanh), fp32 accumulate",
                "M": self.M, "N": self.N, "K": self.K,
                "l2": f"rotating over {self.sets} (A, B, C) buffer sets, 384 MiB > L2",
                "parallelism": "1 GPU" if world == 1 else
                f"M-sharded x{world}; all-gather of C fused into the GEMM epilogue (peer stores over NVLink) + one barrier"
                if os.environ.get("CG_B200_BENCH_ALLGATHER", "fused") == "fused" else
                f"M-sharded x{world}, in-place NCCL all-gather of C"}

    def setup(self, rank, world):
        import ctypes as C
        import torch
        from cantors_gift_b200 import capi
        from cantors_gift_b200.sharding import padded_rows
        self.rank, self.world = rank, world
        self.Ms, padded = padded_rows(self.M, world)
        assert padded == self.M, "the benchmark shapes divide evenly over 1/2/4/8 ranks"
        in_dt = getattr(capi, self.in_dtype_name)
        tdt = {"BF16": torch.bfloat16, "F32": torch.float32}[self.in_dtype_name]
        g = torch.Generator(device="cuda").manual_seed(2)          # same data on every rank
        scale = 0.02 if self.in_dtype_name == "BF16" else 1.0
        self.A, self.B, self.C = [], [], []
        for _ in range(self.sets):
            if self.in_dtype_name == "BF16":
                A = (torch.randn(self.M, self.K, device="cuda", generator=g) * scale).to(tdt)
                B = (torch.randn(self.K, self.N, device="cuda", generator=g) * scale).to(tdt)
            else:
                A = torch.rand(self.M, self.K, device="cuda", generator=g) * 2 - 1
                B = torch.rand(self.K, self.N, device="cuda", generator=g) * 2 - 1
            if not self.A:
                self.A_full0 = A if world > 1 else None   # the gather check recomputes set 0 on one GPU
            self.A.append(A[rank * self.Ms:(rank + 1) * self.Ms].contiguous())
            self.B.append(B)
            self.C.append(torch.empty(self.M, self.N, device="cuda", dtype=tdt))
        self.bias = torch.randn(self.N, device="cuda", generator=g).to(tdt)
        self.desc = capi.make_gemm_desc(self.Ms, self.N, self.K, in_dt, in_dt, epilogue=self.epilogue)
        self.ws, self.ws_bytes = None, 0
        from cantors_gift_b200 import ops
        self.ws, self.ws_bytes = ops.gemm_workspace(self.desc, self.A[0].device)
        self.comm = None
        self.fused = world > 1 and os.environ.get("CG_B200_BENCH_ALLGATHER", "fused") == "fused"
        if world > 1:
            self.comm = make_comm(rank, world)
        if self.fused:
            # C buffers from the C ABI allocator (plain cudaMalloc, so they can be exported) and every
            # peer's copy mapped here: the GEMM epilogue stores its rows into all of them
            self.C_raw, self.peer_tables = share_buffers(rank, world, self.sets, self.M * self.N * self.C[0].element_size())
            _, flag_tables = share_buffers(rank, world, 1, 256)
            self.barrier = C.c_void_p()
            capi.check(capi.lib().cg_b200_peer_barrier_create(C.byref(self.barrier), flag_tables[0], world, rank),
                       "peer_barrier_create")
        self.launches_per_step = 1   # fp32 too: the tf32 hi / lo split happens inside the GEMM kernel

    def step(self, i):
        import ctypes as C
        from cantors_gift_b200 import capi, ops
        s = i % self.sets
        if self.fused:
            import torch
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            p = lambda t: None if t is None else C.c_void_p(t.data_ptr())  # noqa: E731
            capi.check(capi.lib().cg_b200_gemm_allgather(
                C.byref(self.desc), p(self.A[s]), p(self.B[s]), p(self.bias) if self.epilogue != "none" else None, None,
                self.C_raw[s], self.peer_tables[s], self.world, self.rank, p(self.ws), self.ws_bytes, st), "gemm_allgather")
            capi.check(capi.lib().cg_b200_peer_barrier(self.barrier, st), "peer_barrier")
            return
        c_shard = self.C[s][self.rank * self.Ms:(self.rank + 1) * self.Ms]
        ops.gemm(self.desc, self.A[s], self.B[s], c_shard, bias=self.bias if self.epilogue != "none" else None,
                 workspace=self.ws)
        if self.comm is not None:
            import torch
            shard_bytes = self.Ms * self.N * self.C[s].element_size()
            capi.check(capi.lib().cg_b200_allgather_inplace(self.comm, C.c_void_p(self.C[s].data_ptr()), shard_bytes,
                                                            C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                       "allgather_inplace")

    def flops(self):
        return 2.0 * self.M * self.N * self.K

    def work_per_step(self):
        return self.flops() / 1e12

    def algorithmic_per_launch(self):
        return self.flops() / self.world

    def gather_check(self):
        """Outside the timed region: one more sharded step on buffer set 0, then this rank compares the C it
        holds after the gather with the one-GPU kernel's result for the whole problem, bit for bit.
        Returns the number of differing elements on this rank."""
        import torch
        import torch.distributed as dist
        from cantors_gift_b200 import capi, ops
        self.step(0)
        torch.cuda.synchronize()
        dist.barrier()
        want = torch.empty(self.M, self.N, device="cuda", dtype=self.C[0].dtype)
        in_dt = getattr(capi, self.in_dtype_name)
        full = capi.make_gemm_desc(self.M, self.N, self.K, in_dt, in_dt, epilogue=self.epilogue)
        ws, _ = ops.gemm_workspace(full, want.device)
        ops.gemm(full, self.A_full0, self.B[0], want, bias=self.bias if self.epilogue != "none" else None, workspace=ws)
        torch.cuda.synchronize()
        got = device_bytes_to_host(self.C_raw[0], want.numel() * want.element_size()) if self.fused else \
            self.C[0].cpu().view(torch.uint8).flatten()
        diff = int((got.view(torch.int16) != want.cpu().view(torch.uint8).flatten().view(torch.int16)).sum().item())
        dist.barrier()
        return diff

    def library_baseline(self, steps):
        """torch.matmul (the library GEMM) on the same shape and buffer rotation, no epilogue."""
        import torch
        outs = [torch.empty_like(c) for c in self.C]
        for i in range(5):
            torch.matmul(self.A[i % self.sets], self.B[i % self.sets], out=outs[i % self.sets])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            torch.matmul(self.A[i % self.sets], self.B[i % self.sets], out=outs[i % self.sets])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"what": "torch.matmul on the same operands (library GEMM, no bias, no GELU)", "ms_per_step": ms,
                "value": self.flops() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}

    def e2e_setup(self):
        import torch
        from cantors_gift_b200 import ops
        self.runner = ops.HostRunner()
        self.h_A = self.A[0].cpu().pin_memory()
        self.h_B = self.B[0].cpu().pin_memory()
        self.h_bias = self.bias.cpu().pin_memory()
        self.h_C = torch.empty(self.Ms, self.N, dtype=self.A[0].dtype).pin_memory()
        es = self.h_A.element_size()
        if self.ws_bytes:
            self.runner.dev("ws", self.ws_bytes)
        return (self.h_A.numel() + self.h_B.numel() + self.h_bias.numel()) * es, self.h_C.numel() * es

    def e2e_step(self):
        # B and the bias go first; then row slabs of A are copied, multiplied and copied back on three
        # streams, so the step costs about the host-to-device time of A and B, not the sum of the copies
        # and the kernel (HostRunner.run_slabs).
        import ctypes as C
        from cantors_gift_b200 import capi
        r = self.runner
        L = capi.lib()
        es_in, es_out = self.h_A.element_size(), self.h_C.element_size()
        b, bias = r.h2d("B", self.h_B), r.h2d("bias", self.h_bias)
        a = r.dev("A", self.h_A.numel() * es_in)
        c = r.dev("C", self.h_C.numel() * es_out)
        ws = r.dev("ws", self.ws_bytes) if self.ws_bytes else None
        if self.ws_bytes:   # fp32: the operand split would run once per slab; one GEMM on one stream
            a = r.h2d("A", self.h_A)
            capi.check(L.cg_b200_gemm(C.byref(self.desc), a, b, bias if self.epilogue != "none" else None, None, c, ws,
                                      self.ws_bytes, r.stream), "gemm")
            r.d2h(self.h_C, c)
            r.sync()
            return
        slabs = max(1, min(4, self.Ms // 512))
        rows = self.Ms // slabs
        assert rows * slabs == self.Ms
        if getattr(self, "_slab_desc_rows", None) != rows:
            self._slab_desc = capi.make_gemm_desc(rows, self.N, self.K, self.desc.in_dtype, self.desc.out_dtype,
                                                  epilogue=self.epilogue)
            self._slab_desc_rows = rows
        a_bytes, c_bytes = rows * self.K * es_in, rows * self.N * es_out
        hA, hC = self.h_A.data_ptr(), self.h_C.data_ptr()

        def copy_in(i, s):
            capi.check(L.cg_b200_memcpy_h2d(C.c_void_p(a.value + i * a_bytes), C.c_void_p(hA + i * a_bytes), a_bytes, s), "h2d")

        def compute(i, s):
            capi.check(L.cg_b200_gemm(C.byref(self._slab_desc), C.c_void_p(a.value + i * a_bytes), b,
                                      bias if self.epilogue != "none" else None, None, C.c_void_p(c.value + i * c_bytes),
                                      ws, self.ws_bytes, s), "gemm")

        def copy_out(i, s):
            capi.check(L.cg_b200_memcpy_d2h(C.c_void_p(hC + i * c_bytes), C.c_void_p(c.value + i * c_bytes), c_bytes, s), "d2h")

        r.run_slabs(slabs, copy_in, compute, copy_out)

    def cpu_baseline(self, budget_s, prefer_ref=True):
        from oracle import oracle as O
        threads = os.cpu_count() or 1
        O.set_num_threads(threads)
        M, N, K = self.M, self.N, self.K
        rng = np.random.default_rng(2)
        if self.in_dtype_name == "BF16":
            dt = O.BF16
            A = O.to_bf16(rng.standard_normal((M, K), dtype=np.float32) * 0.02)
            B = O.to_bf16(rng.standard_normal((K, N), dtype=np.float32) * 0.02)
            bias = O.to_bf16(rng.standard_normal(N, dtype=np.float32))
        else:
            dt = O.F32
            A = (rng.random((M, K), dtype=np.float32) * 2 - 1).astype(np.float32)
            B = (rng.random((K, N), dtype=np.float32) * 2 - 1).astype(np.float32)
            bias = None
        d = O.make_gemm_desc(M, N, K, dt, dt, epilogue=self.epilogue)
        probe = np.arange(0, min(M, 4 * threads), dtype=np.int64)
        out = np.zeros(M * N, dtype=O.NP_OF[dt])
        t0 = time.perf_counter()
        O.gemm(d, A, B, bias=bias, rows=probe, out=out)
        per_row = (time.perf_counter() - t0) / probe.size
        n_rows = int(max(threads, min(M, budget_s / max(per_row, 1e-9))))
        rows = np.arange(0, n_rows, dtype=np.int64)
        t0 = time.perf_counter()
        O.gemm(d, A, B, bias=bias, rows=rows, out=out)
        dt_s = time.perf_counter() - t0
        return {"value": 2.0 * n_rows * N * K / dt_s / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"rows 0..{n_rows} of {M} (all N and K), sequential-k fp32 FMA chain as the reference's "
                          "scalar JIT matmul, vectorised over n; the reference has no bf16/epilogue code"}, dt_s * M / n_rows


class MatmulF32Workload(GemmWorkload):
    """fp32 M=N=K=1024 through the 3xTF32 split, done inside the GEMM kernel (about 2 GFLOP per launch: bound by
    the L2-to-SM operand traffic of 128 x 64 tiles and by launch latency, not by the tensor cores)."""
    name, dtype = "matmul_f32", "f32 (3xTF32)"
    M = N = K = 1024
    in_dtype_name, epilogue = "F32", "none"
    sets = 16

    def config(self, world):
        return {"workload": "cfg1: fp32 matmul M=N=K=1024 (3xTF32 split + tcgen05 kind::tf32)",
                "l2": f"rotating over {self.sets} buffer sets, 192 MiB > L2", "parallelism": f"x{world}"}


class BlockWorkload(Workload):
    """Pre-LN encoder block, bf16, batch 32 x seq 2048, d_model 1024, 16 heads, FFN 4096; batch-sharded
    over the ranks with one in-place all-gather of y."""
    name, unit, bound, dtype = "block", "TFLOP/s", "tensor", "bf16"
    B, S, D, H, F = 32, 2048, 1024, 16, 4096
    launches_per_step = 9

    def config(self, world):
        return {"workload": "cfg5: pre-LN transformer encoder block, bf16, batch 32, seq 2048, d_model 1024, 16 heads, "
                            "FFN 4096, GELU(tanh), weights ~N(0,0.02)",
                "l2": "activations (over 6 GiB per step) larger than L2",
                "parallelism": "1 GPU" if world == 1 else f"batch-sharded x{world}, y gathered by the last GEMM's peer stores",
                "driver": "Tensor-IR graph -> TensorToCodegenLowering -> NvidiaBackend -> Runtime.bind -> BoundExecutable.launch"
                if getattr(self, "graph", None) is not None else "C-ABI calls from cantors_gift_b200.transformer (host layer not built)"}

    def setup(self, rank, world):
        import torch
        from cantors_gift_b200.sharding import padded_rows
        from cantors_gift_b200.transformer import EncoderBlock
        self.rank, self.world = rank, world
        self.Bs, padded = padded_rows(self.B, world)
        assert padded == self.B
        g = torch.Generator(device="cuda").manual_seed(4)
        w = lambda *s: (torch.randn(*s, device="cuda", generator=g) * 0.02).to(torch.bfloat16)  # noqa: E731
        D, F = self.D, self.F
        self.block = EncoderBlock(D, self.H, F, w(D, 3 * D), w(D, D), w(D, F), w(F), w(F, D), w(D))
        g2 = torch.Generator(device="cuda").manual_seed(5)
        x = torch.randn(self.B, self.S, D, device="cuda", generator=g2).to(torch.bfloat16)
        self.x = x[rank * self.Bs:(rank + 1) * self.Bs].contiguous()
        self.x_full = x if world > 1 else None   # the gather check runs the whole batch on one GPU
        self.y = torch.empty(self.B, self.S, D, device="cuda", dtype=torch.bfloat16)
        self.comm, self.gather = None, None
        self.launches_per_step = self.block.launches_per_forward
        # The step goes through the reference's own interfaces when the host layer is built: the block as a
        # Tensor-IR graph -> TensorToCodegenLowering -> NvidiaBackend -> Runtime.bind -> BoundExecutable.launch.
        # Otherwise the same seven C-ABI calls are issued from cantors_gift_b200.transformer.
        self.graph = None
        try:
            self.graph = GraphBlock(self, torch.cuda.current_device())
        except ImportError as e:
            self.graph_unavailable = str(e).split(";")[0]
        if world > 1 and os.environ.get("CG_B200_BENCH_ALLGATHER", "fused") == "nccl":
            self.comm = make_comm(rank, world)
        elif world > 1:
            # y lives in a buffer every rank maps; the block's last GEMM stores its rows into all of them
            import ctypes as C
            from cantors_gift_b200 import capi
            raw, tables = share_buffers(rank, world, 1, self.B * self.S * D * 2)
            _, flag_tables = share_buffers(rank, world, 1, 256)
            self.barrier = C.c_void_p()
            capi.check(capi.lib().cg_b200_peer_barrier_create(C.byref(self.barrier), flag_tables[0], world, rank),
                       "peer_barrier_create")
            self.gather = (raw[0], tables[0], world, rank)
            self.launches_per_step += 1   # the flag barrier
            if self.graph is not None:
                self.graph.gather_into(raw[0].value, [tables[0][r] for r in range(world)], world, rank)

    def step(self, i):
        import ctypes as C
        import torch
        from cantors_gift_b200 import capi
        if self.gather is not None:
            if self.graph is not None:
                self.graph.launch(self.x, None)
            else:
                self.block.forward(self.x, gather=self.gather)
            capi.check(capi.lib().cg_b200_peer_barrier(self.barrier, C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                       "peer_barrier")
            return
        ys = self.y[self.rank * self.Bs:(self.rank + 1) * self.Bs]
        if self.graph is not None:
            self.graph.launch(self.x, ys)
        else:
            self.block.forward(self.x, out=ys)
        if self.comm is not None:
            capi.check(capi.lib().cg_b200_allgather_inplace(self.comm, C.c_void_p(self.y.data_ptr()), ys.numel() * 2,
                                                            C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                       "allgather_inplace")

    def gather_check(self):
        """Outside the timed region: one more sharded step, then the y this rank holds after the gather
        against the block run on the whole batch by this GPU alone, bit for bit."""
        import torch
        import torch.distributed as dist
        self.step(0)
        torch.cuda.synchronize()
        dist.barrier()
        if self.gather is not None:
            got = device_bytes_to_host(self.gather[0], self.y.numel() * 2)
        else:
            got = self.y.cpu().view(torch.uint8).flatten()
        want = self.block.forward(self.x_full)
        torch.cuda.synchronize()
        diff = int((got.view(torch.int16) != want.cpu().view(torch.uint8).flatten().view(torch.int16)).sum().item())
        dist.barrier()
        return diff

    def flops(self):
        from cantors_gift_b200.transformer import EncoderBlock
        return EncoderBlock.flops(self.B, self.S, self.D, self.H, self.F)

    def work_per_step(self):
        return self.flops() / 1e12

    def algorithmic_per_launch(self):   # per step here: seven launches make one pass of the block
        return self.flops() / self.world

    def e2e_setup(self):
        import torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_y = torch.empty_like(self.h_x).pin_memory()
        self.d_x = torch.empty_like(self.x)
        self.d_y = torch.empty_like(self.x)

        from cantors_gift_b200 import ops
        self.runner = ops.HostRunner()
        return self.h_x.numel() * 2, self.h_y.numel() * 2

    def e2e_step(self):
        # sequences are independent: slabs of the batch are copied in, run and copied out on three streams
        import ctypes as C
        import torch
        from cantors_gift_b200 import capi
        L = capi.lib()
        Bl = self.h_x.shape[0]
        slabs = max(1, min(8, Bl))
        per = Bl // slabs
        assert per * slabs == Bl
        nb = per * self.S * self.D * 2
        dx, dy, hx, hy = self.d_x.data_ptr(), self.d_y.data_ptr(), self.h_x.data_ptr(), self.h_y.data_ptr()

        def copy_in(i, s):
            capi.check(L.cg_b200_memcpy_h2d(C.c_void_p(dx + i * nb), C.c_void_p(hx + i * nb), nb, s), "h2d")

        def compute(i, s):
            if self.graph is not None:
                self.graph.launch(self.d_x[i * per:(i + 1) * per], self.d_y[i * per:(i + 1) * per],
                                  stream=torch.cuda.ExternalStream(s.value))
            else:
                self.block.forward(self.d_x[i * per:(i + 1) * per], out=self.d_y[i * per:(i + 1) * per],
                                   stream=torch.cuda.ExternalStream(s.value))

        def copy_out(i, s):
            capi.check(L.cg_b200_memcpy_d2h(C.c_void_p(hy + i * nb), C.c_void_p(dy + i * nb), nb, s), "d2h")

        self.runner.run_slabs(slabs, copy_in, compute, copy_out)

    def cpu_baseline(self, budget_s, prefer_ref=True):
        from oracle import oracle as O
        from oracle import transformer as T
        threads = os.cpu_count() or 1
        O.set_num_threads(threads)
        rng = np.random.default_rng(4)
        D, F, S = self.D, self.F, self.S
        w = lambda *s: O.to_bf16(rng.standard_normal(s, dtype=np.float32) * 0.02)  # noqa: E731
        ws = dict(w_qkv=w(D, 3 * D), w_o=w(D, D), w_1=w(D, F), b_1=w(F), w_2=w(F, D), b_2=w(D))
        x = O.to_bf16(rng.standard_normal((1, S, D), dtype=np.float32))
        t0 = time.perf_counter()
        T.encoder_block(x, n_heads=self.H, dtype=O.BF16, **ws)
        dt_s = time.perf_counter() - t0
        fl = self.flops() / self.B
        return {"value": fl / dt_s / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"1 of {self.B} sequences (sequences are independent); the reference compiles this graph "
                          "but never executes it"}, dt_s * self.B


class AttentionWorkload(Workload):
    """The fused attention kernel alone at the block's shape: bf16, 16 heads of 64, seq 2048, Q / K / V read in
    place from a packed [batch * seq, 3 * d_model] projection. $CG_B200_BENCH_ATTENTION_BATCH (default 32)
    shrinks the batch for profiler captures."""
    name, unit, bound, dtype = "attention", "TFLOP/s", "tensor", "bf16"
    S, D, H = 2048, 1024, 16

    def __init__(self):
        self.B = int(os.environ.get("CG_B200_BENCH_ATTENTION_BATCH", "32"))
        self.sets = 1 if self.B >= 32 else max(2, min(16, 32 // self.B))

    def config(self, world):
        return {"workload": f"fused attention softmax(Q K^T / 8) V, bf16, batch {self.B}, 16 heads, seq 2048, head_dim 64, "
                            "Q/K/V in place from the packed QKV projection",
                "l2": f"rotating over {self.sets} QKV buffers" if self.B < 32 else "QKV and output (537 MB) larger than L2",
                "parallelism": "1 GPU"}

    def setup(self, rank, world):
        import ctypes as C
        import math
        import torch
        from cantors_gift_b200 import capi
        assert world == 1, "the attention workload is a one-GPU measurement"
        B, S, D, H = self.B, self.S, self.D, self.H
        dh = D // H
        self.sets = 1 if B >= 32 else max(2, min(16, 32 // B))
        g = torch.Generator(device="cuda").manual_seed(6)
        self.qkv = [torch.randn(B * S, 3 * D, device="cuda", generator=g).to(torch.bfloat16) for _ in range(self.sets)]
        self.ctx = [torch.empty(B * S, D, device="cuda", dtype=torch.bfloat16) for _ in range(self.sets)]
        self.desc = capi.AttentionDesc(dtype=capi.BF16, head_dim=dh, batch=B, heads=H, seq_q=S, seq_kv=S, ldq=3 * D,
                                       ldk=3 * D, ldv=3 * D, ldo=D, head_stride_q=dh, head_stride_k=dh, head_stride_v=dh,
                                       head_stride_o=dh, batch_stride_q=S * 3 * D, batch_stride_k=S * 3 * D,
                                       batch_stride_v=S * 3 * D, batch_stride_o=S * D, scale=1.0 / math.sqrt(dh))
        self._C = C

    def step(self, i):
        import torch
        from cantors_gift_b200 import capi
        C = self._C
        q = self.qkv[i % self.sets]
        base, es = q.data_ptr(), 2
        capi.check(capi.lib().cg_b200_attention(
            C.byref(self.desc), C.c_void_p(base), C.c_void_p(base + self.D * es), C.c_void_p(base + 2 * self.D * es),
            C.c_void_p(self.ctx[i % self.sets].data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)), "attention")

    def flops(self):
        return 4.0 * self.B * self.H * self.S * self.S * (self.D // self.H)

    def work_per_step(self):
        return self.flops() / 1e12

    def algorithmic_per_launch(self):
        return self.flops()

    def library_baseline(self, steps):
        """torch's scaled_dot_product_attention (library kernel) on the same Q, K, V (strided views, no copy)."""
        import torch
        B, S, D, H = self.B, self.S, self.D, self.H
        views = []
        for q in self.qkv:
            t = q.view(B, S, 3, H, D // H)
            views.append(tuple(t[:, :, j].transpose(1, 2) for j in range(3)))
        f = torch.nn.functional.scaled_dot_product_attention
        for i in range(5):
            f(*views[i % self.sets])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            f(*views[i % self.sets])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"what": "torch scaled_dot_product_attention on the same Q, K, V", "ms_per_step": ms,
                "value": self.flops() / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}

    def cpu_baseline(self, budget_s, prefer_ref=True):
        from oracle import oracle as O
        threads = os.cpu_count() or 1
        O.set_num_threads(threads)
        rng = np.random.default_rng(6)
        dh = self.D // self.H
        q, k, v = (O.to_bf16(rng.standard_normal((1, 1, self.S, dh), dtype=np.float32)) for _ in range(3))
        t0 = time.perf_counter()
        O.attention(q, k, v, O.BF16, 1.0 / np.sqrt(dh))
        dt_s = time.perf_counter() - t0
        fl = self.flops() / (self.B * self.H)
        return {"value": fl / dt_s / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"1 of {self.B * self.H} (batch, head) pairs; the reference annotates this pattern and "
                          "executes nothing"}, dt_s * self.B * self.H


WORKLOADS = {"attention": AttentionWorkload, "block": BlockWorkload, "gemm": GemmWorkload, "eltwise": EltwiseWorkload, "rowreduce": RowReduceWorkload,
             "matmul_f32": MatmulF32Workload}


class GraphBlock:
    """The encoder block compiled from its Tensor-IR graph and bound through the reference's Runtime."""

    def __init__(self, w, device_index):
        import torch
        from cantors_gift_b200 import graphs
        cg, ext = graphs.host_modules()
        self.cg, self.ext, self.dev = cg, ext, device_index
        self.rt = cg.Runtime()
        if not ext.add_cuda_device(self.rt, device_index):
            raise RuntimeError("no usable sm_100 device for the host layer")
        self.w = w
        self.bound = {}
        blk = w.block
        # weights stored [out, in] and read through a transpose in the graph: the K-contiguous operand layout
        self.weights = [blk._wt["qkv"], blk._wt["o"], blk._wt["1"], blk.b_1, blk._wt["2"], blk.b_2]
        self.stream_of = {}
        self._t = lambda t: ext.Tensor.from_ptr(t.data_ptr(), list(t.shape), cg.DType.BF16, device_index)  # noqa: E731
        self.wt = [self._t(t) for t in self.weights]
        self.gather = None
        self._bind(w.Bs)
        torch.cuda.synchronize()

    def _bind(self, batch):
        from cantors_gift_b200 import graphs
        w = self.w
        exe = graphs.compile_for_b200(self.cg, self.ext, graphs.encoder_block_graph(
            self.cg, batch, w.S, w.D, w.H, w.F, self.cg.DType.BF16, weights_out_in=True))
        assert self.ext.plan_summary(exe) == ["layernorm", "gemm", "attention", "gemm", "layernorm", "gemm", "gemm"]
        b = self.ext.bind(self.rt, exe, self.dev)
        if b is None:
            raise RuntimeError("Runtime.bind returned None")
        self.bound[batch] = b
        return b

    def gather_into(self, y_full_ptr, peer_ptrs, world, rank):
        st = self.bound[self.w.Bs].set_output_gather([int(p) for p in peer_ptrs], world, rank)
        if st != 0:
            raise RuntimeError("set_output_gather: " + self.ext.status_string(st))
        self.gather = self.ext.Tensor.from_ptr(int(y_full_ptr), [self.w.B, self.w.S, self.w.D], self.cg.DType.BF16, self.dev)

    def launch(self, x, y, stream=None):
        """y: a torch tensor, or None: the full-size y of the fused gather (gather_into)."""
        import torch
        s = torch.cuda.current_stream() if stream is None else stream
        h = self.stream_of.get(s.cuda_stream)
        if h is None:
            h = self.stream_of[s.cuda_stream] = self.ext.wrap_stream(s.cuda_stream, self.dev)
        batch = x.shape[0]
        b = self.bound.get(batch) or self._bind(batch)
        out = self.gather if y is None else self._t(y)
        st = b.launch([self._t(x)] + self.wt, [out], h)
        if st != 0:
            raise RuntimeError("launch: " + self.ext.status_string(st))


def device_bytes_to_host(dev_ptr, nbytes):
    """A device buffer of the C ABI allocator as a host uint8 tensor."""
    import ctypes as C
    import torch
    from cantors_gift_b200 import capi
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    capi.check(capi.lib().cg_b200_memcpy_d2h(C.c_void_p(host.data_ptr()), dev_ptr, nbytes, None), "memcpy_d2h")
    capi.check(capi.lib().cg_b200_stream_sync(None), "stream_sync")
    return host


def share_buffers(rank, world, count, nbytes):
    """Allocates `count` buffers through the C ABI on every rank and maps every peer's copies here.
    Returns (local pointers, per-buffer tables of `world` pointers; entry `rank` is the local one)."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from cantors_gift_b200 import capi
    L = capi.lib()
    local, tables = [], []
    for _ in range(count):
        ptr = C.c_void_p()
        capi.check(L.cg_b200_malloc(C.byref(ptr), nbytes), "malloc")
        capi.check(L.cg_b200_memset(ptr, 0, nbytes, None), "memset")
        h = (C.c_char * capi.IPC_HANDLE_BYTES)()
        capi.check(L.cg_b200_ipc_export(ptr, h), "ipc_export")
        mine = torch.frombuffer(bytearray(bytes(h)), dtype=torch.uint8).cuda()
        allh = torch.empty(world * capi.IPC_HANDLE_BYTES, dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(allh, mine)
        allh = allh.cpu().numpy().tobytes()
        table = (C.c_void_p * world)()
        for r in range(world):
            if r == rank:
                table[r] = ptr.value
            else:
                peer = C.c_void_p()
                capi.check(L.cg_b200_ipc_open(allh[r * capi.IPC_HANDLE_BYTES:(r + 1) * capi.IPC_HANDLE_BYTES], C.byref(peer)),
                           "ipc_open")
                table[r] = peer.value
        local.append(ptr)
        tables.append(table)
    torch.cuda.synchronize()
    dist.barrier()
    return local, tables


def make_comm(rank, world):
    """One NCCL communicator through the C ABI; the id travels over torch.distributed."""
    import ctypes as C
    import torch
    import torch.distributed as dist
    from cantors_gift_b200 import capi
    idbuf = (C.c_char * capi.COMM_ID_BYTES)()
    if rank == 0:
        capi.check(capi.lib().cg_b200_comm_unique_id(idbuf), "comm_unique_id")
    t = torch.frombuffer(bytearray(bytes(idbuf)), dtype=torch.uint8).cuda()
    dist.broadcast(t, src=0)
    raw = bytes(t.cpu().numpy().tobytes())
    comm = C.c_void_p()
    capi.check(capi.lib().cg_b200_comm_init_rank(C.byref(comm), world, rank, raw), "comm_init_rank")
    return comm


def time_workload(w, steps, warmup, rank, world, sample_clocks):
    """Returns (seconds for `steps` steps, max over ranks; clocks dict)."""
    import torch
    import torch.distributed as dist
    # the clock sampler starts first so that its start-up pause does not idle the GPU between the
    # warm-up and the timed region
    sampler = ClockSampler(torch.cuda.current_device()) if sample_clocks else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    for i in range(warmup):
        w.step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark()
    e0.record()
    for i in range(steps):
        w.step(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    secs = e0.elapsed_time(e1) * 1e-3
    if world > 1:
        dist.barrier()
        t = torch.tensor([secs], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    if secs < 0.6:   # on every rank, sampling or not: the steps of a sharded workload meet in a barrier
        # nvidia-smi delivers a sample every 100 ms and the timed region of a 0.1 ms kernel is over in a few
        # milliseconds: the same steps run on, untimed, until the sampler has seen 0.6 s of this load
        # (every rank runs the same number, computed from the max-reduced time)
        extra = int(0.6 / max(secs / steps, 1e-7)) + 1
        for i in range(extra):
            w.step(warmup + steps + i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["window"] = "the timed steps and the same steps continued, untimed, to 0.6 s of load"
    return secs, clocks


def time_e2e(w, steps, warmup, world):
    import torch
    import torch.distributed as dist
    h2d, d2h = w.e2e_setup()
    for _ in range(max(1, min(warmup, 3))):
        w.e2e_step()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        w.e2e_step()
    secs = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([secs], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    w.runner.close()
    return secs, h2d, d2h


def run_workload(name, steps, warmup, rank, world, peaks, sample_clocks, with_cpu, cpu_budget, with_e2e=True):
    w = WORKLOADS[name]()
    w.setup(rank, world)
    secs, clocks = time_workload(w, steps, warmup, rank, world, sample_clocks)
    ms_per_step = secs / steps * 1e3
    value = w.work_per_step() * steps / secs
    e2e_steps = max(3, min(steps, 10))
    if with_e2e and hasattr(w, "e2e_setup"):
        e_secs, h2d, d2h = time_e2e(w, e2e_steps, warmup, world)
    else:
        e_secs, h2d, d2h = float("inf"), 0, 0
    e2e_work = w.work_per_step()
    if w.bound == "hbm":
        achieved = w.algorithmic_per_launch() / (secs / steps) / 1e9
        peak, unit = peaks["hbm_gbs"], "GB/s"
    else:
        achieved = w.algorithmic_per_launch() / (secs / steps) / 1e12
        # a timed region of under a second is a kernel timed alone: the burst figure is its denominator;
        # longer regions run under the power cap and are set against the sustained figure
        burst = secs < 1.0
        peak, unit = peaks["bf16_tflops" if burst else "bf16_tflops_sustained"], "TFLOP/s"
    res = {
        "metric": METRIC, "value": value, "unit": w.unit, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if name in ("gemm", "matmul_f32", "block", "attention") else "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic", "config": w.config(world),
        "e2e": {"value": e2e_work * e2e_steps / e_secs, "unit": w.unit, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "note": "host buffers through the C ABI: H2D copies, kernel, D2H copy, stream sync per step"},
        "gpu_launches": steps * w.launches_per_step,
        "roofline": {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_source": peaks["source"] +
                     ((" (burst cuBLAS bf16: the timed region lasts under a second)" if burst else " (sustained cuBLAS bf16)")
                      if w.bound == "tensor" else " (copy bandwidth)"),
                     "note": "per rank; achieved = algorithmic work per launch / mean step time on the device"
                             + (" (includes the all-gather)" if world > 1 and name in ("gemm", "matmul_f32", "block") else "")},
    }
    if w.bound == "tensor":
        res["roofline"]["peak_sustained"] = peaks["bf16_tflops_sustained"]
        res["roofline"]["frac_of_sustained"] = achieved / peaks["bf16_tflops_sustained"]
        res["roofline"]["frac_of_nominal_2250"] = achieved / 2250.0
    if world > 1 and hasattr(w, "gather_check"):
        import torch
        import torch.distributed as dist
        t = torch.tensor([w.gather_check()], device="cuda", dtype=torch.int64)
        dist.all_reduce(t)
        res["gather_check"] = "bit-identical" if int(t.item()) == 0 else f"{int(t.item())} elements differ over {world} ranks"
    if world == 1 and hasattr(w, "library_baseline") and name in ("gemm", "attention"):
        res["library_baseline"] = w.library_baseline(steps)
    if clocks is not None:
        res["clocks"] = clocks
    if with_cpu and rank == 0:
        cpu, _ = w.cpu_baseline(cpu_budget)
        res["cpu_baseline"] = cpu
    del w
    import torch
    torch.cuda.empty_cache()
    return res


def compact(r):
    """The few figures of a secondary workload's line."""
    rf = r["roofline"]
    out = {"value": round(r["value"], 2), "unit": r["unit"], "ms_per_step": round(r["ms_per_step"], 5),
           "frac": round(rf["frac"], 4), "peak": rf["peak"]}
    if rf.get("traffic"):
        out["traffic_over_algorithmic"] = round(rf["traffic"] / (rf["achieved"] * r["ms_per_step"] * 1e-3 *
                                                                 (1e9 if rf["unit"] == "GB/s" else 1e12)), 3) \
            if rf["unit"] == "GB/s" else None
    if r["e2e"]["value"] > 0:
        out["e2e"] = round(r["e2e"]["value"], 2)
    if "cpu_baseline" in r:
        out["cpu"] = round(r["cpu_baseline"]["value"], 4)
        out["cpu_kind"] = r["cpu_baseline"]["kind"]
    if "gather_check" in r:
        out["gather_check"] = r["gather_check"]
    if "clocks" in r and r["clocks"]:
        out["sm_mhz"] = r["clocks"].get("sm_mhz")
        out["reasons"] = r["clocks"].get("reasons")
    return out


def run_reference_arm(args, rank, world):
    """The reference's CPU implementation of the path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    w = WORKLOADS[args.workload]()
    w.world = 1
    budget = 4.0
    for _ in range(args.warmup):
        w.cpu_baseline(budget if args.workload != "gemm" else 1.0)
    vals, secs = [], []
    t_all = time.perf_counter()
    for _ in range(args.steps):
        cpu, full_secs = w.cpu_baseline(budget)
        vals.append(cpu["value"])
        secs.append(full_secs)
        if time.perf_counter() - t_all > 150:
            break
    v = float(np.median(vals))
    cpu["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": w.unit, "n_gpus": args.gpus,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": float(np.median(secs)) * 1e3,
            "higher_is_better": True, "scaling": "strong" if args.workload in ("gemm", "matmul_f32", "block", "attention") else "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic", "config": w.config(1),
            "cpu_baseline": cpu,
            "e2e": {"value": v, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "CPU arm: ms_per_step is the sample's time scaled to the full workload"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="gemm", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-also", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return 0

    import torch
    import torch.distributed as dist
    import cantors_gift_b200  # noqa: F401  (fails loudly if the CUDA library is missing)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    peaks = measured_peaks()

    line = run_workload(args.workload, args.steps, args.warmup, rank, world, peaks, sample_clocks=(rank == 0),
                        with_cpu=(world == 1 and not args.no_cpu), cpu_budget=12.0, with_e2e=not args.no_e2e)
    if not args.no_also:
        # one GPU: every other configuration of the path; several GPUs: the transformer block, the other
        # workload that is partitioned (batch-sharded, y gathered by its last GEMM)
        others = ("eltwise", "rowreduce", "matmul_f32", "block", "attention") if world == 1 else ("block",)
        also = {}
        for other in others:
            if other == args.workload:
                continue
            r = run_workload(other, args.steps, args.warmup, rank, world, peaks, sample_clocks=(rank == 0),
                             with_cpu=(world == 1 and not args.no_cpu), cpu_budget=5.0,
                             with_e2e=(world == 1 and not args.no_e2e))
            also[other] = compact(r)
        # short entries, also kept inside "roofline" (a key whose whole value is recorded)
        line["also"] = also
        line["roofline"]["also"] = also
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
