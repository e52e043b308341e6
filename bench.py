"""Benchmark of the dense-contraction path: fp16 two-layer MLP (MatrixMultiply forward + backward), batch-sharded.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (weak scaling, 8192 rows per GPU in the global batch): X rows x 4096, W1 4096x16384, ReLU, W2 16384x4096, upstream
gradient dY rows x 4096; fp16 storage, fp32 accumulation.  One step = H = X W1, A = relu(H), Y = A W2, then dA = dY W2^T,
dW2 = A^T dY, dH = relu'(H) dA, dX = dH W1^T, dW1 = X^T dH (six contractions of 2*8192*4096*16384 FLOP each on 8192 rows),
and for N > 1 the sum of dW1 and dW2 over the GPUs (peer-memory exchange, deep8_b200.dp.PeerAllReduce).  By default the two
ReLU passes run inside the epilogues of the contractions that produce their inputs and every gradient is written by its
first (here: only) contribution, so no zero fill is needed; `--unfused` runs the reference's call sequence instead (zero
every gradient, eight separate operator calls, += everywhere).  Both give bit-identical tensors
(tests/test_gpu_parity.py::test_fused_step_equals_unfused).  Inputs are seeded synthetic data (X N(0,1), weights N(0,0.02),
dY N(0,1)*0.01, seed 10, rank-offset for X and dY).  With several GPUs the global batch of N x 8192 rows is split by the
ranks' measured speeds (`--no-balance`: 8192 rows each).

Prints ONE JSON line.  `value` is the aggregate TFLOP/s over all GPUs with inputs resident in HBM, after `--preheat` seconds
of the same step, with NVML clock samples taken inside the timed region; `e2e` is the same metric with X and dY copied from
pinned host memory and Y copied back inside every step (plus the same copies without kernels, and the step through the C++
interface, with synchronous feed / fetch and with its copies on Deep8::CopyStream); `roofline` is for the contraction kernel (tensor bound) against the measured cuBLAS bf16 peak of this pool;
`contractions` and `ranks` say where the step's time went on every rank (measured in a short pass with events around every
contraction right after the timed region, which itself carries no events between kernels); `exchange_check` compares the exchanged gradients
with the sum of the ranks' partial gradients; `cpu_baseline` is the reference's own CPU code on a row slice of the same
workload; `aux` reports the four fp32 operator configurations (`--config 1..4`) and `hbm_kernels` the HBM-bound neighbours
(matrix-vector products, Linear, AdamUpdate) against the measured copy bandwidth.  `--impl reference` times only that CPU code.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_PER_GPU, D_IN, D_HID = 8192, 4096, 16384
FLOP_PER_GEMM = 2.0 * M_PER_GPU * D_IN * D_HID
FLOP_PER_STEP = 6.0 * FLOP_PER_GEMM
METRIC = "mlp_fwd_bwd_tflops"
UNIT = "TFLOP/s"
# nominal dense fp16 tensor peak of one B200, for the "fraction of nominal peak" the north star quotes
NOMINAL_FP16_TFLOPS = 2250.0
CPU_SAMPLE_ROWS = 256


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops_sustained"]), "measured (cuBLAS bf16, sustained)"
    return 1400.0, "fallback (sustained figure of an earlier measurement on this pool)"


# ------------------------------------------------------------------------------------------------ clocks
class NvmlSampler:
    """Reads SM clock, board power and the active clock-event reasons of one GPU through NVML (queries only) from a thread
    of this process every `period_s`; report(t0, t1) summarises the samples whose host time lies inside [t0, t1] - the
    timed region, bracketed by synchronisations on both sides - so the clock figure describes the region itself."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, torch, index, period_s=0.002):
        self.period_s, self.samples, self.stop_flag, self.thread, self.handle, self.nvml = period_s, [], False, None, None, None
        self.max_mhz, self.error = None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception as exc:
            self.handle, self.error = None, repr(exc)[:200]

    def available(self):
        return self.handle is not None

    def _loop(self):
        n, h = self.nvml, self.handle
        reasons_fn = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop_flag:
            try:
                mhz = n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)
            except Exception as exc:  # without the clock there is no sample; keep the reason for the report
                self.error = repr(exc)[:200]
                time.sleep(self.period_s)
                continue
            mask, watts = 0, None
            try:
                mask = int(reasons_fn(h))
            except Exception as exc:
                self.error = repr(exc)[:200]
            try:
                watts = n.nvmlDeviceGetPowerUsage(h) / 1000.0
            except Exception as exc:
                self.error = repr(exc)[:200]
            self.samples.append((time.perf_counter(), float(mhz), mask, watts))
            time.sleep(self.period_s)

    def start(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)

    def report(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no NVML sample inside the timed region"], "samples": 0,
                    "samples_outside": len(self.samples), "error": self.error}
        mhz = [s[1] for s in inside]
        mask = 0
        for s in inside:
            mask |= s[2]
        return {"sm_mhz": statistics.median(mhz), "sm_mhz_min": min(mhz), "sm_mhz_max": max(mhz), "sm_max_mhz": self.max_mhz,
                "reasons": [name for name, bit in self.REASONS if mask & bit], "samples": len(inside),
                "power_w_median": statistics.median([s[3] for s in inside if s[3] is not None] or [0.0]),
                "source": "NVML queries from this process every %g ms; only samples inside the timed region are counted" % (self.period_s * 1e3)}


class SmiSampler:
    """Fallback when NVML cannot be loaded or returns nothing: nvidia-smi asked for a line every 20 ms."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def report(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for t, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not (t0 <= t <= t1 + 0.1):
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi -lms 20 (the in-process NVML queries gave no sample)"}


# ------------------------------------------------------------------------------------------------ CPU reference arm
class CpuMlp:
    """One fwd+bwd step of the MLP on CPU_SAMPLE_ROWS rows through a CPU implementation's MatrixMultiply entry points,
    buffers allocated once (as the GPU arm does) so that the timed region is the reference's arithmetic."""

    def __init__(self, impl, x, w1, w2, dy):
        self.impl, self.x, self.w1, self.w2, self.dy = impl, x, w1, w2, dy
        r = x.shape[1]
        z = lambda *s: np.zeros(s, np.float32)
        self.h, self.a, self.y = z(1, r, D_HID), z(1, r, D_HID), z(1, r, D_IN)
        self.da, self.dh, self.dx = z(1, r, D_HID), z(1, r, D_HID), z(1, r, D_IN)
        self.dw1, self.dw2 = np.zeros_like(w1), np.zeros_like(w2)

    def step(self):
        m = self.impl._matmul
        for g in (self.da, self.dh, self.dx, self.dw1, self.dw2):
            g.fill(0)
        m(0, self.x, None, self.w1, None, self.h, None)
        np.maximum(self.h, 0, out=self.a)
        m(0, self.a, None, self.w2, None, self.y, None)
        m(1, self.a, self.da, self.w2, None, self.y, self.dy)
        m(2, self.a, None, self.w2, self.dw2, self.y, self.dy)
        np.multiply(self.da, self.h > 0, out=self.dh)
        m(1, self.x, self.dx, self.w1, None, self.h, self.dh)
        m(2, self.x, None, self.w1, self.dw1, self.h, self.dh)


def cpu_arm(steps, warmup):
    """The reference's own CPU path (oracle/_ref) if it was built, else the restated oracle; float32 (no CPU half in
    the reference, deep8/src/math/MatrixMultiply.cpp:126-129) on a row slice, FLOPs counted for that slice."""
    from oracle import pyoracle
    if pyoracle.Reference.available():
        impl = pyoracle.Reference()
        cores = 1  # Eigen dense Map product without OpenMP: MatrixMultiply runs on one thread in the reference
    else:
        impl = pyoracle.Restated()
        cores = impl.threads()
    rng = np.random.Generator(np.random.Philox(10))
    x = rng.standard_normal((1, CPU_SAMPLE_ROWS, D_IN)).astype(np.float32)
    w1 = (rng.standard_normal((1, D_IN, D_HID)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((1, D_HID, D_IN)) * 0.02).astype(np.float32)
    dy = (rng.standard_normal((1, CPU_SAMPLE_ROWS, D_IN)) * 0.01).astype(np.float32)
    mlp = CpuMlp(impl, x, w1, w2, dy)
    for _ in range(warmup):
        mlp.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        mlp.step()
    dt = (time.perf_counter() - t0) / steps
    flop = FLOP_PER_STEP * CPU_SAMPLE_ROWS / M_PER_GPU
    return {"value": flop / dt / 1e12, "unit": UNIT, "cores": cores, "kind": impl.kind,
            "sample": "%d of %d rows per step, float32, %d step(s) of %.1f s" % (CPU_SAMPLE_ROWS, M_PER_GPU, steps, dt)}, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))       # a step of the 256-row sample takes about 7 s on one core
    warmup = 1 if args.warmup > 0 else 0
    base, dt = cpu_arm(steps, warmup)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(args.gpus), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def exchange_name(n):
    if n == 1:
        return "single GPU: nothing to exchange"
    mode = os.environ.get("D8_BENCH_ALLREDUCE", "fused")
    return {"fused": "peer memory: the contraction's epilogue stores each row block in its owner's GPU (reduce-scatter inside the "
                     "kernel), fixed-order sum kernel, copy-engine all-gather on a side stream",
            "peer": "peer memory: copy-engine reduce-scatter/all-gather + fixed-order sum kernel on a side stream",
            "none": "NO exchange (diagnostic: independent replicas, gradients are not summed)",
            "end": "NCCL all-reduce after the last contraction"}.get(mode, "NCCL all-reduce started as each gradient completes")


def workload_config(n):
    return {"workload": "config 5: fp16 2-layer MLP fwd+bwd via MatrixMultiply, X %dx%d per GPU, W1 %dx%d, ReLU, W2 %dx%d" %
            (M_PER_GPU, D_IN, D_IN, D_HID, D_HID, D_IN), "rows_per_gpu": M_PER_GPU, "global_rows": M_PER_GPU * n,
            "parallelism": "batch-sharded x%d, weight gradients summed across GPUs (%s)" % (n, exchange_name(n)),
            "flop_per_gpu_step": FLOP_PER_STEP, "l2": "inputs exceed L2 (weights 2x128 MiB, activations 4x256 MiB per GPU)"}


# ------------------------------------------------------------------------------------------------ GPU arm
# the six contractions of one step, in the order the fused step launches them
CONTRACTIONS = ("H = X*W1 (+ReLU)", "Y = A*W2", "dW2 = A^T*dY", "dA = dY*W2^T (+ReLU grad)", "dW1 = X^T*dH", "dX = dH*W1^T")


class MlpStep:
    """The MLP step on one GPU through the d8k C ABI; buffers allocated once, as an executor would keep them.
    X, dY and Y are double-buffered so that the end-to-end loop can copy step i+1 in and step i-1 out while step i runs.

    With several GPUs the sums of dW1 and dW2 run on a side stream.  A step does not wait for its own exchange: the wait
    moves to the first point of the NEXT step that needs it - before the staging memory is rewritten (after the two
    forward contractions), or, with the trainer's step inside the exchange (sgd), before the first contraction, which reads
    the updated weights.  drain() waits for whatever is still pending; the timed regions end with it."""

    SGD = (1e-6, 1e-4)  # learning rate, weight decay of the optional trainer step (--sgd); small: the data are random every step

    def __init__(self, ctx, torch, device, rank, fused=True, exchange=None, scatter=False, sgd=False, rows=None):
        self.ctx, self.torch, self.fused, self.scatter, self.sgd = ctx, torch, fused, scatter, sgd
        M_PER_GPU = self.rows = rows if rows is not None else globals()["M_PER_GPU"]  # this rank's share of the batch
        self.ar1 = self.ar2 = None
        self.pending = False
        g = torch.Generator(device=device)
        g.manual_seed(10)
        h = torch.float16
        self.W1 = (torch.randn((1, D_IN, D_HID), device=device, generator=g) * 0.02).to(h)
        self.W2 = (torch.randn((1, D_HID, D_IN), device=device, generator=g) * 0.02).to(h)
        g.manual_seed(10 + 1000 * (rank + 1))
        e = lambda *s: torch.empty(s, device=device, dtype=h)
        self.X = [torch.randn((1, M_PER_GPU, D_IN), device=device, generator=g).to(h)]
        self.dY = [(torch.randn((1, M_PER_GPU, D_IN), device=device, generator=g) * 0.01).to(h)]
        self.X.append(self.X[0].clone())
        self.dY.append(self.dY[0].clone())
        self.Y = [e(1, M_PER_GPU, D_IN), e(1, M_PER_GPU, D_IN)]
        self.H, self.A = e(1, M_PER_GPU, D_HID), e(1, M_PER_GPU, D_HID)
        self.dA, self.dH = e(1, M_PER_GPU, D_HID), e(1, M_PER_GPU, D_HID)
        self.dX, self.dW1, self.dW2 = torch.empty_like(self.X[0]), torch.empty_like(self.W1), torch.empty_like(self.W2)
        if exchange is not None:
            # weight gradients live in memory the peers map; the sums arrive in ar.result
            self.ar1, self.ar2 = exchange(self.W1.numel(), D_IN), exchange(self.W2.numel(), D_HID)
            self.dW1, self.dW2 = self.ar1.partial.view(self.W1.shape), self.ar2.partial.view(self.W2.shape)
            if sgd:  # the weights move into peer memory: each rank updates the shard it sums and receives the rest
                self.ar1.weights.copy_(self.W1.view(-1))
                self.ar2.weights.copy_(self.W2.view(-1))
                self.W1, self.W2 = self.ar1.weights.view(self.W1.shape), self.ar2.weights.view(self.W2.shape)
        self.gemm_events = []
        self.tail_events = []  # around each wait of the main stream for the exchange

    def _reduce(self, which, dist, work, overlap):
        ar, grad = (self.ar1, self.dW1) if which == 1 else (self.ar2, self.dW2)
        if ar is not None:
            ar.start(sgd=self.SGD if self.sgd else None)
        elif dist is not None and overlap:
            work.append(dist.all_reduce(grad, async_op=True))

    def _gemm(self, fn, timed):
        if timed:
            a, b = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            self.gemm_events.append((a, b))
        else:
            fn()

    def drain(self, timed=False):
        """Main stream waits for the exchanges started by the last step (no-op when nothing is pending)."""
        if self.ar1 is None or not self.pending:
            return
        if timed:
            ev = (self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True))
            ev[0].record()
        self.ar2.finish()
        self.ar1.finish()
        if timed:
            ev[1].record()
            self.tail_events.append(ev)
        self.pending = False

    def step(self, dist=None, timed=False, buf=0):
        c = self.ctx
        X, dY, Y = self.X[buf], self.dY[buf], self.Y[buf]
        overlap = os.environ.get("D8_BENCH_ALLREDUCE", "fused") != "end"
        work = []
        if self.sgd:
            self.drain(timed)  # the forward pass reads the weights the previous step's exchange updates
        if self.fused:
            # Weight gradients are produced as early as their inputs allow, so that each exchange has contractions
            # still to run behind it: dW2 needs only A and dY, dW1 needs dH, and dX (no exchange) goes last.
            self._gemm(lambda: c.matmul_forward_relu(X, self.W1, self.H, self.A), timed)
            self._gemm(lambda: c.matmul_forward(self.A, self.W2, out=Y), timed)
            self.drain(timed)
            if self.ar1 is not None:
                self.ar2.before_write()
            if self.scatter:  # the contraction's epilogue stores each row block in its owner's memory
                self._gemm(lambda: self.ar2.scatter_grad_y(self.A, dY), timed)
            else:
                self._gemm(lambda: c.matmul_grad_y(self.A, self.W2, self.dW2, dY, accumulate=False), timed)
            if not self.sgd:
                self._reduce(2, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x_relu(self.A, self.dA, self.W2, dY, self.H, self.dH, False, False), timed)
            if self.sgd:  # the trainer's step rewrites W2: only after its last reader of this step (dA) is enqueued
                self._reduce(2, dist, work, overlap)
            if self.ar1 is not None:
                self.ar1.before_write()
            if self.scatter:
                self._gemm(lambda: self.ar1.scatter_grad_y(X, self.dH), timed)
            else:
                self._gemm(lambda: c.matmul_grad_y(X, self.W1, self.dW1, self.dH, accumulate=False), timed)
            if not self.sgd:
                self._reduce(1, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x(X, self.dX, self.W1, self.dH, accumulate=False), timed)
            if self.sgd:  # likewise W1 and dX
                self._reduce(1, dist, work, overlap)
        else:
            for t in (self.dA, self.dH, self.dX):
                c.zero(t)
            self._gemm(lambda: c.matmul_forward(X, self.W1, out=self.H), timed)
            c.relu_forward(self.H, out=self.A)
            self._gemm(lambda: c.matmul_forward(self.A, self.W2, out=Y), timed)
            self.drain(timed)
            if self.ar1 is not None:
                self.ar2.before_write()
                self.ar1.before_write()
            c.zero(self.dW2)
            c.zero(self.dW1)
            self._gemm(lambda: c.matmul_grad_y(self.A, self.W2, self.dW2, dY), timed)
            if not self.sgd:
                self._reduce(2, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x(self.A, self.dA, self.W2, dY), timed)
            if self.sgd:
                self._reduce(2, dist, work, overlap)
            c.relu_backward(self.H, self.dH, self.dA)
            self._gemm(lambda: c.matmul_grad_y(X, self.W1, self.dW1, self.dH), timed)
            if not self.sgd:
                self._reduce(1, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x(X, self.dX, self.W1, self.dH), timed)
            if self.sgd:
                self._reduce(1, dist, work, overlap)
        if self.ar1 is not None:
            self.pending = True
        elif dist is not None:
            if not overlap:
                work.append(dist.all_reduce(self.dW2, async_op=True))
                work.append(dist.all_reduce(self.dW1, async_op=True))
            for w in work:
                w.wait()
        if self.sgd and self.ar1 is None:  # SGDTrainer::update on the full gradients (one GPU, or after NCCL)
            from deep8_b200.dp import sgd_coefficients
            alpha, beta = sgd_coefficients(*self.SGD)
            c.axpby(self.dW2, alpha, self.W2, beta)
            c.axpby(self.dW1, alpha, self.W1, beta)


def bind_to_gpu_numa_node(torch, index):
    """Run this process (and place the pinned host buffers it allocates later) on the CPUs next to the GPU: with several
    ranks feeding their GPUs from host memory every step, buffers on the wrong socket halve the copy rate.  The GPU's
    NUMA node comes from sysfs; where a container hides it, from NVML's ideal-CPU mask (read only).  Returns what was
    used ("node 1", "nvml 48 cpus"), or None when neither is visible (then nothing changes)."""
    allowed = os.sched_getaffinity(0)
    try:
        prop = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bdf).read())
        if node >= 0:
            cpus = set()
            for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= allowed
            if cpus:
                os.sched_setaffinity(0, cpus)
                return "node %d" % node
    except (OSError, ValueError, AttributeError):
        pass
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(index).uuid)
        handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        words = (max(allowed) + 64) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (word >> b) & 1} & allowed
        if cpus and cpus != allowed:
            os.sched_setaffinity(0, cpus)
            return "nvml %d cpus" % len(cpus)
    except Exception:
        pass
    return None


def exchange_check(mlp, ctx, torch, dist, device, world, rank):
    """After the timed steps: is what the exchange delivered the sum of the ranks' partial gradients?  Each rank recomputes
    its partial dW2 and dW1 with the plain gradient entry point, a few 128-row slabs of them (the first and last of every
    owner's row block) travel over NCCL to every rank, are added there in rank order in fp32 and rounded once - the
    arithmetic of the sum kernel - and must equal the exchanged result bit for bit.  With the trainer's step inside the
    exchange a rank holds only the summed shard it owns, so it checks that one (and that the weights agree everywhere)."""
    part = torch.empty_like(mlp.W2)
    bad = 0
    slabs_checked = 0
    for ar, x, dz, rows, cols in ((mlp.ar2, mlp.A, mlp.dY[0], D_HID, D_IN), (mlp.ar1, mlp.X[0], mlp.dH, D_IN, D_HID)):
        w = part.view(1, rows, cols)
        ctx.matmul_grad_y(x, w, w, dz, accumulate=False)
        torch.cuda.synchronize()
        got_all = ar.result.view(rows, cols)
        br = ar.block_rows
        for owner in range(world):
            lo, hi = owner * br, min((owner + 1) * br, rows)
            if lo >= hi:
                continue
            for r0 in sorted({lo, max(lo, hi - 128)}):
                mine = w[0, r0:r0 + 128].contiguous()
                parts = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(parts, mine)
                acc = parts[0].float()
                for q in range(1, world):
                    acc += parts[q].float()
                want = acc.to(torch.float16)
                if mlp.sgd and owner != rank:
                    continue
                slabs_checked += 1
                if not torch.equal(got_all[r0:r0 + 128], want):
                    bad += 1
    if mlp.sgd:  # every rank must hold the same updated weights
        for wt in (mlp.W1, mlp.W2):
            probe = wt.view(-1)[:: max(1, wt.numel() // 65536)].contiguous()
            parts = [torch.empty_like(probe) for _ in range(world)]
            dist.all_gather(parts, probe)
            slabs_checked += 1
            if any(not torch.equal(parts[0], p) for p in parts[1:]):
                bad += 1
    t = torch.tensor([bad, slabs_checked], device=device, dtype=torch.int64)
    dist.all_reduce(t)
    return int(t[0].item()), int(t[1].item())


def filter_gradient_exchange(n_cfg, ctx, ctx_side, side, torch, dist, device, world, rank):
    """Benchmark configuration 3 (Conv2d) or 4 (DeConv2d) with the images sharded over the GPUs: each rank computes the
    filter gradient of its images, the partial gradients are summed through PeerAllReduce (copy-engine reduce-scatter,
    fixed-order sum kernel, copy-engine all-gather - the filter is far too small for row blocks per owner), and rank 0
    compares the result with the CPU oracle on the whole batch.  Returns (ms per gradient + exchange, max rel error)."""
    from deep8_b200.dp import PeerAllReduce, shard_range
    name, x, w, dz, kind, meta, _ = small_config_case(n_cfg)
    lo, hi = shard_range(x.shape[0], world, rank)
    X = torch.from_numpy(np.ascontiguousarray(x[lo:hi])).to(device)
    DZ = torch.from_numpy(np.ascontiguousarray(dz[lo:hi])).to(device)
    W = torch.from_numpy(w).to(device)
    ar = PeerAllReduce(ctx, ctx_side, side, W.numel(), torch.float32, device, timeout_ms=20000.0)
    DW = ar.partial.view(W.shape)
    grad = ctx.conv2d_grad_y if kind == "conv" else ctx.deconv2d_grad_y

    def one():
        ar.before_write()
        ctx.zero(DW)
        if hi > lo:
            grad(X, W, DW, DZ, *meta)
        ar.start()
        ar.finish()

    for _ in range(3):
        one()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 10
    e0.record()
    for _ in range(iters):
        one()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    got = ar.result.view(W.shape).cpu().numpy()
    # every rank must hold the same bits
    probe = ar.result.clone()
    parts = [torch.empty_like(probe) for _ in range(world)]
    dist.all_gather(parts, probe)
    same = all(torch.equal(parts[0], p) for p in parts[1:])
    err = None
    if rank == 0:
        from oracle import pyoracle
        oracle = pyoracle.Restated()
        want = oracle.conv2d_grad_y(x, w, dz, *meta) if kind == "conv" else oracle.deconv2d_grad_y(x, w, dz, *meta)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import cases
        err = cases.rel_max(got, want)
    dist.barrier()
    ar.close()
    return {"workload": name, "images_per_gpu": hi - lo, "filter_gradient_bytes": W.numel() * 4, "ms_gradient_plus_exchange": float(t.item()),
            "max_rel_err_vs_oracle_whole_batch": err, "same_bits_on_every_rank": bool(same),
            "path": "PeerAllReduce: partial gradient in peer-mapped memory, copy-engine pull of the owned shard, fixed-order sum kernel, "
                    "copy-engine push to every peer"}


def step_cost(rows, pairs=74):
    """Relative time of one step on `rows` rows: the paired kernel works in waves of `pairs` 256 x 256 tiles, each tile costing
    its contraction length.  Used to predict what moving rows between ranks does, wave quantisation included."""
    mt = -(-rows // 256)
    wide = -(-mt * (D_HID // 256) // pairs) * D_IN          # H = X W1 and dA = dY W2^T: rows x 16384 outputs, K = 4096
    narrow = -(-mt * (D_IN // 256) // pairs) * D_HID         # Y = A W2 and dX = dH W1^T: rows x 4096 outputs, K = 16384
    grads = -(-(D_HID // 256) * (D_IN // 256) // pairs) * rows  # dW1, dW2: fixed outputs, K = rows
    return 2.0 * (wide + narrow + grads)


def balance_rows(step_ms, total_rows, quantum=256):
    """Rows per rank (multiples of `quantum`, summing to total_rows) that minimise the slowest rank's predicted step, given
    each rank's measured step time on an equal share.  GPUs of one box differ by 5-20 % under the power limit, and a step
    that exchanges gradients runs at the pace of the slowest rank: the faster GPUs take more of the batch."""
    world = len(step_ms)
    equal = total_rows // world
    speed = [1.0 / t for t in step_ms]
    rows = [max(quantum, int(round(total_rows * sp / sum(speed) / quantum)) * quantum) for sp in speed]
    while sum(rows) > total_rows:
        rows[rows.index(max(rows))] -= quantum
    while sum(rows) < total_rows:
        rows[rows.index(min(rows))] += quantum
    predict = lambda r, k: step_ms[k] * step_cost(r) / step_cost(equal)
    for _ in range(4 * world * (equal // quantum)):  # move one quantum from the slowest predicted rank to the one that stays fastest
        times = [predict(rows[k], k) for k in range(world)]
        slow = times.index(max(times))
        if rows[slow] <= quantum:
            break
        best, best_t = None, times[slow]
        for k in range(world):
            if k == slow:
                continue
            t = max(predict(rows[k] + quantum, k), predict(rows[slow] - quantum, slow))
            if t < best_t - 1e-9:
                best, best_t = k, t
        if best is None:
            break
        rows[slow] -= quantum
        rows[best] += quantum
    return rows


def run_gpu_arm(args):
    import torch
    import deep8_b200

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torch.distributed.run --nproc-per-node %d" % (args.gpus, world, args.gpus))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    numa_node = bind_to_gpu_numa_node(torch, local_rank) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    ctx = deep8_b200.Context(local_rank)
    stream = torch.cuda.current_stream()
    ctx.use_stream(stream if stream.cuda_stream != 0 else None)
    exchange = None
    ctx_side = side = None
    mode = os.environ.get("D8_BENCH_ALLREDUCE", "fused")
    if world > 1 and mode in ("peer", "fused"):
        # gradient exchange through peer memory on a side stream (deep8_b200.dp.PeerAllReduce); D8_BENCH_ALLREDUCE=overlap
        # or =end selects NCCL all-reduce instead, started as each gradient completes or after the last contraction
        from deep8_b200.dp import PeerAllReduce
        side = torch.cuda.Stream(device=device)
        ctx_side = deep8_b200.Context(local_rank, scratch_bytes=1 << 20)
        ctx_side.use_stream(side)
        # waits between ranks give up after 20 s here (first steps include module loading on every rank); the default is 2 s
        exchange = lambda numel, rows: PeerAllReduce(ctx, ctx_side, side, numel, torch.float16, device, rows=rows, with_weights=args.sgd,
                                                     timeout_ms=20000.0, gather=os.environ.get("D8_BENCH_GATHER", "copy"))
    step_dist = None if mode == "none" else dist  # "none": the ranks run side by side and nothing is summed (diagnostic)
    # Shares of the batch.  The global batch is world x 8192 rows; each rank first times the step alone on an equal share
    # (no exchange, about a second, so that the GPUs are at their power-limited clocks), then the rows are split so that every
    # rank is predicted to need the same time.  --no-balance keeps 8192 rows everywhere.
    my_rows, balance = M_PER_GPU, None
    if dist is not None and not args.no_balance and not args.profile:
        cal = MlpStep(ctx, torch, device, rank, fused=not args.unfused)
        for _ in range(160):
            cal.step()
        torch.cuda.synchronize()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(40):
            cal.step()
        c1.record()
        torch.cuda.synchronize()
        mine = torch.tensor([c0.elapsed_time(c1) / 40], device=device, dtype=torch.float64)
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        alone_ms = [float(t.item()) for t in every]
        shares = balance_rows(alone_ms, M_PER_GPU * world)
        my_rows = shares[rank]
        balance = {"rows_per_gpu": shares, "step_ms_alone_on_equal_shares": alone_ms,
                   "rule": "rows in multiples of 256, chosen so that every rank's predicted step time (measured time x tile-wave count) is equal"}
        del cal
        torch.cuda.empty_cache()
    mlp = MlpStep(ctx, torch, device, rank, fused=not args.unfused, exchange=exchange,
                  scatter=exchange is not None and mode == "fused" and not args.unfused, sgd=args.sgd, rows=my_rows)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def status_ok():
        return ctx.status() == 0 and (ctx_side is None or ctx_side.status() == 0)

    barrier()
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record()
    for _ in range(args.warmup):
        mlp.step(step_dist)
    mlp.drain()
    w1.record()
    barrier()
    if not status_ok():
        raise SystemExit("kernel status non-zero after warm-up")
    # Pre-heat: the same step, untimed, for about `--preheat` seconds, so that the timed region runs at the clock the power
    # limit settles on rather than at the boost clock of a cold start.  Every rank runs the same number of steps.
    # The clock sampler starts before the pre-heat, so that it is known to deliver before the timed region begins.
    sampler = None
    if rank == 0 and not args.profile:
        sampler = NvmlSampler(torch, local_rank)
        sampler.start()
    preheat_steps, preheat_s = 0, 0.0
    if args.preheat > 0 and not args.profile:
        th = time.perf_counter()
        # a first chunk, timed, tells how many steps fill the rest of the pre-heat (the warm-up steps carry first-call costs)
        chunk = 20
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(chunk):
            mlp.step(step_dist)
        mlp.drain()
        c1.record()
        torch.cuda.synchronize()
        chunk_ms = max_over_ranks(c0.elapsed_time(c1) / chunk)
        preheat_steps = chunk + max(0, int(math.ceil(args.preheat * 1e3 / max(chunk_ms, 0.1))) - chunk)
        for _ in range(preheat_steps - chunk):
            mlp.step(step_dist)
        mlp.drain()
        barrier()
        preheat_s = time.perf_counter() - th
    fallback_sampler = None
    if sampler is not None and (not sampler.available() or (args.preheat > 0 and not sampler.samples)):
        fallback_sampler = SmiSampler(local_rank)  # NVML absent, or it delivered nothing during the pre-heat
        fallback_sampler.start()
        time.sleep(0.3)

    # ---- device-resident timed region
    launches0 = ctx.launch_count()
    barrier()
    host_t0 = time.perf_counter()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        mlp.step(step_dist)
    mlp.drain()
    t1.record()
    torch.cuda.synchronize()
    host_t1 = time.perf_counter()
    barrier()
    launches = ctx.launch_count() - launches0
    # ---- the same step with CUDA events around every contraction, right after and outside the timed region: where the time
    # goes on every rank.  (Inside the region the events cost 4-5 %: an event between two kernels keeps the next one's first CTAs
    # from starting while the previous one's last, partly filled wave of tiles drains.)
    inst_steps = max(1, min(args.steps, 10))
    i0, i1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    i0.record()
    for _ in range(inst_steps):
        mlp.step(step_dist, timed=True)
    mlp.drain(timed=True)
    i1.record()
    torch.cuda.synchronize()
    barrier()
    inst_ms = i0.elapsed_time(i1) / inst_steps
    clocks = None
    if sampler is not None:
        sampler.stop()
        clocks = sampler.report(host_t0, host_t1)
        if fallback_sampler is not None:
            fallback_sampler.stop()
            if not clocks.get("samples"):
                nvml_report = clocks
                clocks = fallback_sampler.report(host_t0, host_t1)
                clocks["nvml"] = {k: nvml_report.get(k) for k in ("samples_outside", "error")}
    my_ms = t0.elapsed_time(t1) / args.steps
    ms_step = max_over_ranks(t0.elapsed_time(t1)) / args.steps
    gemm_ms = [a.elapsed_time(b) for a, b in mlp.gemm_events]
    mlp.gemm_events = []
    per_gemm = [sum(gemm_ms[i::6]) / max(1, len(gemm_ms[i::6])) for i in range(6)]   # mean of each of the six contractions
    tail_ms = sum(a.elapsed_time(b) for a, b in mlp.tail_events) / inst_steps
    mlp.tail_events = []
    # every rank's step, contraction and exchange-wait times, so that the line shows the spread between GPUs
    mine = torch.tensor([my_ms, sum(gemm_ms) / inst_steps, tail_ms] + per_gemm, device=device, dtype=torch.float64)
    if dist is not None:
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        table = torch.stack(allr).cpu().numpy()
    else:
        table = mine.cpu().numpy()[None, :]
    if os.environ.get("D8_BENCH_DIAG"):  # per rank: where the step's time went
        print("rank %d: step %.3f ms, contractions %.3f ms (%s), waiting for the exchange %.3f ms" %
              (rank, my_ms, sum(gemm_ms) / inst_steps, " ".join("%.3f" % v for v in per_gemm), tail_ms), file=sys.stderr, flush=True)
    if not status_ok():
        raise SystemExit("kernel status non-zero after the timed region")

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms_step, "gpu_launches": launches}), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- correctness of the exchange, outside the timed region
    xcheck = None
    filt = None
    if dist is not None and exchange is not None:
        bad, slabs = exchange_check(mlp, ctx, torch, dist, device, world, rank)
        xcheck = {"result": "bit-exact" if bad == 0 else "MISMATCH", "slabs_compared": slabs, "mismatching": bad,
                  "what": "dW1 and dW2 after the last timed step against the rank-ordered fp32 sum of every rank's recomputed partial "
                          "gradient (first and last 128 rows of each owner's block, gathered over NCCL)"}
        if not args.no_aux:
            filt = {"config 3": filter_gradient_exchange(3, ctx, ctx_side, side, torch, dist, device, world, rank),
                    "config 4": filter_gradient_exchange(4, ctx, ctx_side, side, torch, dist, device, world, rank)}
        if not status_ok():
            raise SystemExit("kernel status non-zero after the exchange checks")

    # ---- end-to-end: X and dY from pinned host memory every step, Y back to the host.  Copies run on their own
    # streams into the other half of the double buffers, so step i computes while step i+1 arrives and step i-1 leaves.
    hX = torch.empty(mlp.X[0].shape, dtype=torch.float16).pin_memory()
    hdY = torch.empty(mlp.dY[0].shape, dtype=torch.float16).pin_memory()
    hY = [torch.empty(mlp.Y[0].shape, dtype=torch.float16).pin_memory() for _ in range(2)]
    hX.copy_(mlp.X[0])
    hdY.copy_(mlp.dY[0])
    e2e_steps = max(4, min(args.steps, 20))
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    main = torch.cuda.current_stream()

    def e2e_loop(n, compute=True):
        in_ready = [None, None]    # event: inputs of buffer b have arrived
        out_done = [None, None]    # event: Y of buffer b has left
        comp_done = [None, None]   # event: the step that used buffer b has finished

        def feed(i):
            b = i % 2
            with torch.cuda.stream(s_in):
                if comp_done[b] is not None:
                    s_in.wait_event(comp_done[b])       # the step that last read X[b], dY[b] is over
                mlp.X[b].copy_(hX, non_blocking=True)
                mlp.dY[b].copy_(hdY, non_blocking=True)
                in_ready[b] = torch.cuda.Event()
                in_ready[b].record(s_in)

        feed(0)
        for i in range(n):
            b = i % 2
            if i + 1 < n:
                feed(i + 1)
            main.wait_event(in_ready[b])
            if out_done[b] is not None:
                main.wait_event(out_done[b])            # Y[b] of two steps ago has been read
            if compute:
                mlp.step(step_dist, buf=b)
            comp_done[b] = torch.cuda.Event()
            comp_done[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                hY[b].copy_(mlp.Y[b], non_blocking=True)
                out_done[b] = torch.cuda.Event()
                out_done[b].record(s_out)
        if compute:
            mlp.drain()
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    def timed_loop(compute):
        # the compute leg is pre-heated like the device-resident region (the checks in between let the GPU cool, and a cold
        # start runs 8-10 % faster on boost clocks: not a sustained figure)
        heat = max(2, int(args.preheat * 1e3 / max(ms_step, 0.1))) if compute and not args.profile else 2
        e2e_loop(heat, compute)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_loop(e2e_steps, compute)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / e2e_steps

    e2e_ms = timed_loop(True)
    # the same copies on the same buffers and streams with no kernel in between: the host-link ceiling of this box at this N
    copy_ms = timed_loop(False)
    h2d = hX.numel() * 2 + hdY.numel() * 2
    d2h = hY[0].numel() * 2

    if rank == 0:
        peak, peak_src = measured_peaks()
        avg_gemm_ms = sum(gemm_ms) / len(gemm_ms)
        flop_per_launch = FLOP_PER_GEMM * my_rows / M_PER_GPU  # rank 0's contractions, on rank 0's share of the rows
        achieved = flop_per_launch / (avg_gemm_ms * 1e-3) / 1e12
        per_gpu = FLOP_PER_STEP / (ms_step * 1e-3) / 1e12
        sm_mhz = clocks.get("sm_mhz") if clocks else None
        contractions = [{"name": CONTRACTIONS[i] if not args.unfused else CONTRACTIONS[i].split(" (")[0], "ms_rank0": float(table[0, 3 + i]),
                         "ms_min_over_ranks": float(table[:, 3 + i].min()), "ms_max_over_ranks": float(table[:, 3 + i].max())} for i in range(6)]
        line = {
            "metric": METRIC, "value": per_gpu * world, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (f32 accumulate)",
            "data": "synthetic", "config": dict(workload_config(world), step=("fused epilogues, first-touch gradients" if not args.unfused
                                                  else "reference call sequence (zero fill, separate ReLU passes)") +
                                                  (" + SGD step (outside the metric's work)" if args.sgd else "")),
            "per_gpu_tflops": per_gpu, "frac_of_nominal_fp16_peak": per_gpu / NOMINAL_FP16_TFLOPS,
            "preheat_s": preheat_s, "preheat_steps": preheat_steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "kernel": "d8k_gemm_pair_kernel (TMA-fed fp16, CTA pairs on 256x256 tiles)",
                         "peak_source": peak_src, "flop_per_launch": flop_per_launch, "avg_launch_ms": avg_gemm_ms,
                         "mcycles_per_launch": (avg_gemm_ms * 1e-3 * sm_mhz) if sm_mhz else None,
                         "measured_in": "the instrumented pass right after the timed region (%d steps with CUDA events around every "
                                        "contraction: %.3f ms per step on rank 0)" % (inst_steps, inst_ms),
                         "gemm_share_of_step": sum(gemm_ms) / (inst_ms * inst_steps)},
            "contractions": contractions,
            "ranks": {"step_ms": [float(table[:, 0].min()), float(table[:, 0].max())],
                      "contractions_ms": [float(table[:, 1].min()), float(table[:, 1].max())],
                      "waiting_for_exchange_ms": [float(table[:, 2].min()), float(table[:, 2].max())],
                      "note": "[min, max] over ranks of each rank's own per-step means; step_ms from the timed region, the other two from the "
                              "instrumented pass after it; a step's exchange is waited for inside the next step"},
            "e2e": {"value": FLOP_PER_STEP * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "preheat_s": args.preheat,
                    "overlap": "copies on side streams, double-buffered inputs and outputs", "host_numa_node_rank0": numa_node,
                    "copy_only_ms": copy_ms, "copy_only_gbs_per_gpu": (h2d + d2h) / (copy_ms * 1e-3) / 1e9,
                    "copy_only_gbs_aggregate": world * (h2d + d2h) / (copy_ms * 1e-3) / 1e9,
                    "e2e_over_max_of_copy_and_compute": e2e_ms / max(copy_ms, ms_step)},
            "gpu_launches": launches, "clocks": clocks,
        }
        if balance is not None:
            line["config"]["rows_per_gpu"] = balance["rows_per_gpu"]
            line["config"]["batch_shares"] = balance
        if xcheck is not None:
            line["exchange_check"] = xcheck["result"]
            line["exchange_check_detail"] = xcheck
        if filt is not None:
            line["filter_gradient_exchange"] = filt
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _ = cpu_arm(1, 0)
        if world == 1 and not args.no_aux:
            # the same step through the C++ interface (Deep8::Variable::feed -> EagerExecutor -> fetch), in its own process
            exe = os.path.join(ROOT, "tests", "cpp", "bin", "bench_mlp_e2e")
            if os.path.exists(exe):
                del mlp
                torch.cuda.empty_cache()
                for key, extra in (("cpp_api", []), ("cpp_api_overlapped", ["overlap"])):
                    try:
                        # 200 steps (1 to 2 s): long enough for the power limit to set the clock, as in the legs above
                        r = subprocess.run([exe, "200", str(M_PER_GPU)] + extra, capture_output=True, text=True, timeout=300)
                        line["e2e"][key] = json.loads(r.stdout.strip().splitlines()[-1])
                    except Exception as exc:  # the figure is auxiliary: its absence must not cost the line
                        line["e2e"][key] = {"error": str(exc)[:200]}
        if world == 1 and not args.no_aux:
            # benchmark configurations 1-4 with their own inputs: an auxiliary report, outside the headline's timed region
            line["aux"] = [run_small(ctx, torch, device, n, steps=20, warmup=3, half=False, with_cpu=not args.no_cpu) for n in (1, 2, 3, 4)]
            line["hbm_kernels"] = run_hbm_kernels(ctx, torch, device)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        if xcheck is not None and xcheck["mismatching"]:
            dist.destroy_process_group()
            raise SystemExit("the exchanged gradients differ from the sum of the partial gradients")
        dist.destroy_process_group()


# DRAM bytes (read + write) of one contraction launch of this workload: mean over the six launches of one step captured with ncu
# (dram__bytes_read.sum + dram__bytes_write.sum); the algorithmic bytes are 0.45e9 to 0.96e9 depending on the fused epilogue.
TRAFFIC_BYTES_PER_LAUNCH = 1.31e9


# ------------------------------------------------------------------------------------------------ HBM-bound neighbours
def run_hbm_kernels(ctx, torch, dev, rows=16384, cols=16384):
    """The path's HBM-bound kernels on operands far larger than L2: MatrixMultiply with a single-column y (forward = matrix-vector
    product over rows, gradient of y = over columns, gradient of x = outer product) on a rows x cols matrix, and Linear /
    AdamUpdate on 2^27 elements.  Median of 10 launches (CUDA events), algorithmic bytes / time, and that as a fraction of the
    measured copy bandwidth."""
    import statistics
    peak, label = 6650.0, "of fallback copy bandwidth (an earlier measurement on this pool)"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak, label = float(json.load(f)["hbm_gbs"]), "of measured copy bandwidth"

    def gbs(fn, nbytes):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        v = nbytes / statistics.median(ts) / 1e9
        return {"gbs": round(v, 1), "frac": round(v / peak, 3)}

    out = {"peak_gbs": peak, "frac_is": label, "matrix": [rows, cols]}
    for dt, es, name in ((torch.float32, 4, "f32"), (torch.float16, 2, "f16")):
        X = torch.randn(1, rows, cols, device=dev, dtype=dt)
        y = torch.randn(1, cols, 1, device=dev, dtype=dt)
        z = torch.empty(1, rows, 1, device=dev, dtype=dt)
        dz = torch.randn(1, rows, 1, device=dev, dtype=dt)
        dX, dy = torch.zeros_like(X), torch.zeros_like(y)
        r = {}
        r["matvec_rows"] = gbs(lambda: ctx.matmul_forward(X, y, out=z), rows * cols * es)
        r["matvec_columns"] = gbs(lambda: ctx.matmul_grad_y(X, y, dy, dz), rows * cols * es)
        r["outer_product"] = gbs(lambda: ctx.matmul_grad_x(X, dX, y, dz), 2 * rows * cols * es)
        del X, dX
        n = 1 << 27
        a, b = torch.randn(n, device=dev, dtype=dt), torch.randn(n, device=dev, dtype=dt)
        m, v = torch.zeros(n, device=dev, dtype=dt), torch.zeros(n, device=dev, dtype=dt)
        r["linear_forward"] = gbs(lambda: ctx.linear_forward(a, 0.5, 1.0, out=b), 2 * n * es)
        r["linear_grad"] = gbs(lambda: ctx.linear_grad(b, 0.5, a), 3 * n * es)
        r["adam_update"] = gbs(lambda: ctx.adam_update(a, b, m, v, 0.9, 0.999, 1e-7, 1e-3, 0.0, 1), 8 * n * es)
        del a, b, m, v
        torch.cuda.empty_cache()
        out[name] = r
    return out


# ------------------------------------------------------------------------------------------------ configs 1-4 (fp32)
def small_config_case(n):
    """(name, x, w, dz, kind, meta, flop) of benchmark configuration n in 1..4, inputs drawn as the configuration states
    (numpy Philox streams named by the configuration's seeds; the second operand of configurations 1 and 2 uses seed + 10)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import cases
    if n == 1:
        return ("fp32 MatrixMultiply 256x512 * 512x128", cases.uniform(0, (1, 256, 512)), cases.uniform(10, (1, 512, 128)),
                cases.uniform(1, (1, 256, 128)), "matmul", None, 3 * 2.0 * 256 * 512 * 128)
    if n == 2:
        return ("fp32 MatrixMultiply batch 64 of 128x256 * batch 1 of 256x256", cases.normal(2, (64, 128, 256), 0.05),
                cases.normal(12, (1, 256, 256), 0.05), cases.normal(3, (64, 128, 256)), "matmul", None, 3 * 2.0 * 8192 * 256 * 256)
    if n == 3:
        return ("fp32 Conv2d 32x56x56x64, 3x3x64 -> 64, stride 1, covered", cases.uniform(4, (32, 56, 56, 64)),
                cases.normal(5, (64, 3, 3, 64), (2.0 / 576) ** 0.5), cases.normal(6, (32, 56, 56, 64)), "conv", (True, (1, 1), (1, 1)),
                3 * 2.0 * 100352 * 576 * 64)
    return ("fp32 DeConv2d 16x14x14x256, 4x4x256 -> 128, stride 2, covered (output 27x27)", cases.uniform(7, (16, 14, 14, 256)),
            cases.normal(8, (128, 4, 4, 256), 1.0 / 64), cases.normal(9, (16, 27, 27, 128)), "deconv", (True, (2, 2)),
            3 * 2.0 * 3136 * 256 * 2048)


def run_small(ctx, torch, dev, n, steps, warmup, half, with_cpu):
    """Benchmark configuration n in 1..4 (fp32, 3xTF32): forward + gradient of x + gradient of y of ONE operator on one GPU,
    timed with CUDA events with an L2 flush between iterations, checked against the oracle, with the reference's CPU
    code timed beside it.  Returns the report as a dict."""
    from oracle import pyoracle
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import cases

    name, x, w, dz, kind, meta, flop = small_config_case(n)
    tdtype, tol, label = torch.float32, 1e-5, "f32 (3xTF32)"
    if half:  # the same operator on fp16 storage (fp32 accumulation); the oracle sees the rounded inputs
        tdtype, tol, label = torch.float16, 2e-2, "f16 (f32 accumulate)"
        x, w, dz = (a.astype("float16").astype("float32") for a in (x, w, dz))
    X, W, DZ = (torch.from_numpy(a).to(dev).to(tdtype) for a in (x, w, dz))
    DX, DW = torch.zeros_like(X), torch.zeros_like(W)
    Z = torch.empty(tuple(dz.shape), device=dev, dtype=tdtype)
    paths = {}  # which kernel variant each contraction took (d8k_last_kernel)

    def step():
        ctx.zero(DX)
        ctx.zero(DW)
        if kind == "matmul":
            ctx.matmul_forward(X, W, out=Z)
            paths["forward"] = ctx.last_kernel()
            ctx.matmul_grad_x(X, DX, W, DZ)
            paths["grad_x"] = ctx.last_kernel()
            ctx.matmul_grad_y(X, W, DW, DZ)
        elif kind == "conv":
            ctx.conv2d_forward(X, W, *meta, out=Z)
            paths["forward"] = ctx.last_kernel()
            ctx.conv2d_grad_x(X, DX, W, DZ, *meta)
            paths["grad_x"] = ctx.last_kernel()
            ctx.conv2d_grad_y(X, W, DW, DZ, *meta)
        else:
            ctx.deconv2d_forward(X, W, *meta, out=Z)
            paths["forward"] = ctx.last_kernel()
            ctx.deconv2d_grad_x(X, DX, W, DZ, *meta)
            paths["grad_x"] = ctx.last_kernel()
            ctx.deconv2d_grad_y(X, W, DW, DZ, *meta)
        paths["grad_y"] = ctx.last_kernel()

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    if ctx.status() != 0:
        raise SystemExit("kernel status non-zero in configuration %d" % n)
    ms = statistics.median(times)
    line = {"report": "config %d" % n, "workload": name.replace("fp32", "fp16") if half else name, "dtype": label, "ms_per_step": ms,
            "tflops": flop / ms / 1e9,
            ("frac_of_fp16_peak" if half else "frac_of_tf32_peak_over_3"): flop / ms / 1e9 / (2250.0 if half else 1100.0 / 3),
            "l2": "flushed between iterations (256 MiB write)", "steps": steps, "kernels": dict(paths), "cpu": None}
    if not with_cpu:
        return line
    # parity against the oracle and the reference's CPU time
    oracle = pyoracle.Restated()
    ref = pyoracle.Reference() if pyoracle.Reference.available() else oracle

    def cpu(impl):
        if kind == "matmul":
            return impl.matmul_forward(x, w), impl.matmul_grad_x(x, w, dz), impl.matmul_grad_y(x, w, dz)
        if kind == "conv":
            return impl.conv2d_forward(x, w, *meta), impl.conv2d_grad_x(x, w, dz, *meta), impl.conv2d_grad_y(x, w, dz, *meta)
        return impl.deconv2d_forward(x, w, *meta), impl.deconv2d_grad_x(x, w, dz, *meta), impl.deconv2d_grad_y(x, w, dz, *meta)

    want = cpu(oracle)
    got = (Z.float().cpu().numpy(), DX.float().cpu().numpy(), DW.float().cpu().numpy())
    line["max_rel_err_vs_oracle"] = max(cases.rel_max(g, r) for g, r in zip(got, want))
    line["tolerance"] = tol
    cpu(ref)
    cpu_times = []
    for _ in range(3):
        t0 = time.perf_counter()
        cpu(ref)
        cpu_times.append(time.perf_counter() - t0)
    cpu_ms = min(cpu_times) * 1e3
    line["cpu"] = {"ms": cpu_ms, "kind": ref.kind, "threads": 1 if kind == "matmul" else ref.threads(), "gflops": flop / cpu_ms / 1e6}
    return line


def run_small_config(args):
    """`--config N` with N in 1..4: the auxiliary report of one configuration as its own JSON line."""
    import torch
    import deep8_b200
    ctx = deep8_b200.Context(0)
    print(json.dumps(run_small(ctx, torch, torch.device("cuda", 0), args.config, args.steps, args.warmup, args.half, not args.no_cpu)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=5, choices=[1, 2, 3, 4, 5], help="benchmark configuration; 5 (default) is the headline "
                    "line, 1-4 print an auxiliary fp32 report for one operator")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-aux", action="store_true", help="skip the auxiliary reports (configurations 1-4 on one GPU; the Conv2d/DeConv2d "
                    "filter-gradient exchange on several)")
    ap.add_argument("--no-balance", action="store_true", help="several GPUs: keep 8192 rows on every rank instead of giving the faster GPUs "
                    "a larger share of the global batch")
    ap.add_argument("--preheat", type=float, default=2.0, help="seconds of untimed steps before the timed region (0 = none)")
    ap.add_argument("--half", action="store_true", help="with --config: run the configuration's operator on fp16 storage")
    ap.add_argument("--sgd", action="store_true",
                    help="add the reference's SGD step on W1, W2 to every step (not part of the metric's forward + backward): "
                         "after the backward pass on one GPU, inside the gradient exchange's sum kernel on several")
    ap.add_argument("--unfused", action="store_true", help="the reference's call sequence: zero fill, separate ReLU passes, += everywhere")
    ap.add_argument("--profile", action="store_true", help="for runs under a profiler: no clock sampling, no end-to-end or CPU leg, "
                    "warm-up as given; the printed numbers are not benchmark values")
    args = ap.parse_args()
    if args.impl == "ours" and not args.profile:
        args.warmup = max(args.warmup, 3)  # timing rule: at least three untimed steps
    if args.config != 5 and args.impl == "ours":
        run_small_config(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
