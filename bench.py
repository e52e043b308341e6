"""Benchmark of the dense-contraction path: fp16 two-layer MLP (MatrixMultiply forward + backward), batch-sharded.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (per GPU, weak scaling): X 8192x4096, W1 4096x16384, ReLU, W2 16384x4096, upstream gradient dY 8192x4096;
fp16 storage, fp32 accumulation.  One step = H = X W1, A = relu(H), Y = A W2, then dA = dY W2^T, dW2 = A^T dY,
dH = relu'(H) dA, dX = dH W1^T, dW1 = X^T dH (six contractions of 2*8192*4096*16384 FLOP each), and for N > 1 the NCCL
all-reduce (sum) of dW1 and dW2.  By default the two ReLU passes run inside the epilogues of the contractions that
produce their inputs and every gradient is written by its first (here: only) contribution, so no zero fill is needed;
`--unfused` runs the reference's call sequence instead (zero every gradient, eight separate operator calls, += everywhere).
Both give bit-identical tensors (tests/test_gpu_parity.py::test_fused_step_equals_unfused).  Inputs are seeded synthetic
data (X N(0,1), weights N(0,0.02), dY N(0,1)*0.01, seed 10, rank-offset for X and dY).

Prints ONE JSON line.  `value` is the aggregate TFLOP/s over all GPUs with inputs resident in HBM; `e2e` is the same
metric with X and dY copied from pinned host memory and Y copied back inside every step; `roofline` is for the
contraction kernel (tensor bound) against the measured cuBLAS bf16 peak of this pool; `cpu_baseline` is the reference's
own CPU code on a row slice of the same workload.  `--impl reference` times only that CPU code.
"""
import argparse
import json
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
class ClockSampler:
    """Samples nvidia-smi while the timed region runs: SM clock, its maximum and the active throttle reasons."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
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
                "reasons": sorted(reasons), "samples": len(sm)}


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
    base, dt = cpu_arm(max(1, min(args.steps, 3)), 1 if args.warmup > 0 else 0)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
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
            "end": "NCCL all-reduce after the last contraction"}.get(mode, "NCCL all-reduce started as each gradient completes")


def workload_config(n):
    return {"workload": "config 5: fp16 2-layer MLP fwd+bwd via MatrixMultiply, X %dx%d per GPU, W1 %dx%d, ReLU, W2 %dx%d" %
            (M_PER_GPU, D_IN, D_IN, D_HID, D_HID, D_IN), "rows_per_gpu": M_PER_GPU, "global_rows": M_PER_GPU * n,
            "parallelism": "batch-sharded x%d, weight gradients summed across GPUs (%s)" % (n, exchange_name(n)),
            "flop_per_gpu_step": FLOP_PER_STEP, "l2": "inputs exceed L2 (weights 2x128 MiB, activations 4x256 MiB per GPU)"}


# ------------------------------------------------------------------------------------------------ GPU arm
class MlpStep:
    """The MLP step on one GPU through the d8k C ABI; buffers allocated once, as an executor would keep them.
    X, dY and Y are double-buffered so that the end-to-end loop can copy step i+1 in and step i-1 out while step i runs."""

    SGD = (1e-6, 1e-4)  # learning rate, weight decay of the optional trainer step (--sgd); small: the data are random every step

    def __init__(self, ctx, torch, device, rank, fused=True, exchange=None, scatter=False, sgd=False):
        self.ctx, self.torch, self.fused, self.scatter, self.sgd = ctx, torch, fused, scatter, sgd
        self.ar1 = self.ar2 = None
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
        self.tail_events = []  # (after the last contraction, after the exchange has been waited for)

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

    def step(self, dist=None, timed=False, buf=0):
        c = self.ctx
        X, dY, Y = self.X[buf], self.dY[buf], self.Y[buf]
        overlap = os.environ.get("D8_BENCH_ALLREDUCE", "fused") != "end"
        work = []
        if self.ar1 is not None:
            self.ar2.before_write()
            self.ar1.before_write()
        if self.fused:
            # Weight gradients are produced as early as their inputs allow, so that each exchange has contractions
            # still to run behind it: dW2 needs only A and dY, dW1 needs dH, and dX (no exchange) goes last.
            self._gemm(lambda: c.matmul_forward_relu(X, self.W1, self.H, self.A), timed)
            self._gemm(lambda: c.matmul_forward(self.A, self.W2, out=Y), timed)
            if self.scatter:  # the contraction's epilogue stores each row block in its owner's memory
                self._gemm(lambda: self.ar2.scatter_grad_y(self.A, dY), timed)
            else:
                self._gemm(lambda: c.matmul_grad_y(self.A, self.W2, self.dW2, dY, accumulate=False), timed)
            self._reduce(2, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x_relu(self.A, self.dA, self.W2, dY, self.H, self.dH, False, False), timed)
            if self.scatter:
                self._gemm(lambda: self.ar1.scatter_grad_y(X, self.dH), timed)
            else:
                self._gemm(lambda: c.matmul_grad_y(X, self.W1, self.dW1, self.dH, accumulate=False), timed)
            self._reduce(1, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x(X, self.dX, self.W1, self.dH, accumulate=False), timed)
        else:
            for t in (self.dA, self.dH, self.dX, self.dW1, self.dW2):
                c.zero(t)
            self._gemm(lambda: c.matmul_forward(X, self.W1, out=self.H), timed)
            c.relu_forward(self.H, out=self.A)
            self._gemm(lambda: c.matmul_forward(self.A, self.W2, out=Y), timed)
            self._gemm(lambda: c.matmul_grad_y(self.A, self.W2, self.dW2, dY), timed)
            self._reduce(2, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x(self.A, self.dA, self.W2, dY), timed)
            c.relu_backward(self.H, self.dH, self.dA)
            self._gemm(lambda: c.matmul_grad_y(X, self.W1, self.dW1, self.dH), timed)
            self._reduce(1, dist, work, overlap)
            self._gemm(lambda: c.matmul_grad_x(X, self.dX, self.W1, self.dH), timed)
        if self.ar1 is not None:
            if timed:
                self.tail_events.append((self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)))
                self.tail_events[-1][0].record()
            self.ar2.finish()
            self.ar1.finish()
            if timed:
                self.tail_events[-1][1].record()
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
    mlp = MlpStep(ctx, torch, device, rank, fused=not args.unfused, exchange=exchange,
                  scatter=exchange is not None and mode == "fused" and not args.unfused, sgd=args.sgd)

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

    for _ in range(args.warmup):
        mlp.step(dist)
    barrier()
    if ctx.status() != 0 or (exchange is not None and ctx_side.status() != 0):
        raise SystemExit("kernel status non-zero after warm-up")

    # ---- device-resident timed region
    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.profile:
        sampler.start()
        time.sleep(0.3)
    launches0 = ctx.launch_count()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        mlp.step(dist, timed=True)
    t1.record()
    barrier()
    launches = ctx.launch_count() - launches0
    clocks = sampler.stop() if (rank == 0 and not args.profile) else None
    ms_total = max_over_ranks(t0.elapsed_time(t1))
    ms_step = ms_total / args.steps
    gemm_ms = [a.elapsed_time(b) for a, b in mlp.gemm_events]
    mlp.gemm_events = []
    if os.environ.get("D8_BENCH_DIAG"):  # per rank: where the step's time went
        tail = [a.elapsed_time(b) for a, b in mlp.tail_events]
        print("rank %d: step %.3f ms, contractions %.3f ms, exchange left after the last contraction %.3f ms" %
              (rank, t0.elapsed_time(t1) / args.steps, sum(gemm_ms) / args.steps, sum(tail) / max(1, args.steps)), file=sys.stderr, flush=True)
    mlp.tail_events = []
    if ctx.status() != 0 or (exchange is not None and ctx_side.status() != 0):
        raise SystemExit("kernel status non-zero after the timed region")

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms_step, "gpu_launches": launches}), flush=True)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
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

    def e2e_loop(n):
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
            mlp.step(dist, buf=b)
            comp_done[b] = torch.cuda.Event()
            comp_done[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                hY[b].copy_(mlp.Y[b], non_blocking=True)
                out_done[b] = torch.cuda.Event()
                out_done[b].record(s_out)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    e2e_loop(2)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_loop(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    h2d = hX.numel() * 2 + hdY.numel() * 2
    d2h = hY[0].numel() * 2

    if rank == 0:
        peak, peak_src = measured_peaks()
        avg_gemm_ms = sum(gemm_ms) / len(gemm_ms)
        achieved = FLOP_PER_GEMM / (avg_gemm_ms * 1e-3) / 1e12
        per_gpu = FLOP_PER_STEP / (ms_step * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": per_gpu * world, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (f32 accumulate)",
            "data": "synthetic", "config": dict(workload_config(world), step=("fused epilogues, first-touch gradients" if not args.unfused
                                                  else "reference call sequence (zero fill, separate ReLU passes)") +
                                                  (" + SGD step (outside the metric's work)" if args.sgd else "")),
            "per_gpu_tflops": per_gpu, "frac_of_nominal_fp16_peak": per_gpu / NOMINAL_FP16_TFLOPS,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "kernel": "d8k_gemm_pair_kernel (TMA-fed fp16, CTA pairs on 256x256 tiles)",
                         "peak_source": peak_src, "flop_per_launch": FLOP_PER_GEMM, "avg_launch_ms": avg_gemm_ms,
                         "gemm_share_of_step": sum(gemm_ms) / (ms_step * args.steps)},
            "e2e": {"value": FLOP_PER_STEP * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "overlap": "copies on side streams, double-buffered inputs and outputs", "host_numa_node_rank0": numa_node},
            "gpu_launches": launches, "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _ = cpu_arm(1, 0)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes (read + write) of one contraction launch of this workload: mean of the three launches of the default step captured with ncu
# (profiles/d8k_gemm_pair_kernel_f16_mlp_config5.md); algorithmic bytes are 0.47e9.
TRAFFIC_BYTES_PER_LAUNCH = 1.28e9


# ------------------------------------------------------------------------------------------------ configs 1-4 (fp32)
def run_small_config(args):
    """BASELINE configurations 1-4 (fp32, 3xTF32): forward + gradient of x + gradient of y of ONE operator on one GPU,
    timed with CUDA events with an L2 flush between iterations, checked against the oracle, with the reference's CPU
    code timed beside it.  An auxiliary report (one JSON line), not the benchmark line of the default run."""
    import torch
    import deep8_b200
    from oracle import pyoracle
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import cases

    n = args.config
    dev = torch.device("cuda", 0)
    ctx = deep8_b200.Context(0)
    if n == 1:
        name = "fp32 MatrixMultiply 256x512 * 512x128"
        x, w = cases.uniform(0, (1, 256, 512)), cases.uniform(10, (1, 512, 128))
        dz = cases.uniform(1, (1, 256, 128))
        kind, meta, flop = "matmul", None, 3 * 2.0 * 256 * 512 * 128
    elif n == 2:
        name = "fp32 MatrixMultiply batch 64 of 128x256 * batch 1 of 256x256"
        x, w = cases.normal(2, (64, 128, 256), 0.05), cases.normal(12, (1, 256, 256), 0.05)
        dz = cases.normal(3, (64, 128, 256))
        kind, meta, flop = "matmul", None, 3 * 2.0 * 8192 * 256 * 256
    elif n == 3:
        name = "fp32 Conv2d 32x56x56x64, 3x3x64 -> 64, stride 1, covered"
        x, w = cases.uniform(4, (32, 56, 56, 64)), cases.normal(5, (64, 3, 3, 64), (2.0 / 576) ** 0.5)
        dz = cases.normal(6, (32, 56, 56, 64))
        kind, meta, flop = "conv", (True, (1, 1), (1, 1)), 3 * 2.0 * 100352 * 576 * 64
    else:
        name = "fp32 DeConv2d 16x14x14x256, 4x4x256 -> 128, stride 2, covered (output 27x27)"
        x, w = cases.uniform(7, (16, 14, 14, 256)), cases.normal(8, (128, 4, 4, 256), 1.0 / 64)
        dz = cases.normal(9, (16, 27, 27, 128))
        kind, meta, flop = "deconv", (True, (2, 2)), 3 * 2.0 * 3136 * 256 * 2048
    tdtype, tol, label = torch.float32, 1e-5, "f32 (3xTF32)"
    if args.half:  # the same operator on fp16 storage (fp32 accumulation); the oracle sees the rounded inputs
        tdtype, tol, label = torch.float16, 2e-2, "f16 (f32 accumulate)"
        x, w, dz = (a.astype("float16").astype("float32") for a in (x, w, dz))
    X, W, DZ = (torch.from_numpy(a).to(dev).to(tdtype) for a in (x, w, dz))
    DX, DW = torch.zeros_like(X), torch.zeros_like(W)

    paths = {}  # which kernel variant each contraction took (d8k_last_kernel)

    def step():
        ctx.zero(DX)
        ctx.zero(DW)
        if kind == "matmul":
            z = ctx.matmul_forward(X, W, out=Z)
            paths["forward"] = ctx.last_kernel()
            ctx.matmul_grad_x(X, DX, W, DZ)
            paths["grad_x"] = ctx.last_kernel()
            ctx.matmul_grad_y(X, W, DW, DZ)
        elif kind == "conv":
            z = ctx.conv2d_forward(X, W, *meta, out=Z)
            paths["forward"] = ctx.last_kernel()
            ctx.conv2d_grad_x(X, DX, W, DZ, *meta)
            paths["grad_x"] = ctx.last_kernel()
            ctx.conv2d_grad_y(X, W, DW, DZ, *meta)
        else:
            z = ctx.deconv2d_forward(X, W, *meta, out=Z)
            paths["forward"] = ctx.last_kernel()
            ctx.deconv2d_grad_x(X, DX, W, DZ, *meta)
            paths["grad_x"] = ctx.last_kernel()
            ctx.deconv2d_grad_y(X, W, DW, DZ, *meta)
        paths["grad_y"] = ctx.last_kernel()
        return z

    Z = torch.empty(tuple(dz.shape), device=dev, dtype=tdtype)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    assert ctx.status() == 0
    ms = statistics.median(times)
    # parity against the oracle and the reference's CPU time
    oracle = pyoracle.Restated()
    ref = pyoracle.Reference() if pyoracle.Reference.available() else oracle

    def cpu(impl):
        if kind == "matmul":
            return impl.matmul_forward(x, w), impl.matmul_grad_x(x, w, dz), impl.matmul_grad_y(x, w, dz)
        if kind == "conv":
            return impl.conv2d_forward(x, w, *meta), impl.conv2d_grad_x(x, w, dz, *meta), impl.conv2d_grad_y(x, w, dz, *meta)
        return impl.deconv2d_forward(x, w, *meta), impl.deconv2d_grad_x(x, w, dz, *meta), impl.deconv2d_grad_y(x, w, dz, *meta)

    if args.no_cpu:
        print(json.dumps({"report": "config %d" % n, "workload": name, "dtype": label, "ms_per_step": ms, "tflops": flop / ms / 1e9,
                          "steps": args.steps, "kernels": paths, "cpu": None}), flush=True)
        return
    want = cpu(oracle)
    got = (Z.float().cpu().numpy(), DX.float().cpu().numpy(), DW.float().cpu().numpy())
    err = max(cases.rel_max(g, r) for g, r in zip(got, want))
    cpu(ref)
    cpu_times = []
    for _ in range(3):
        t0 = time.perf_counter()
        cpu(ref)
        cpu_times.append(time.perf_counter() - t0)
    cpu_ms = min(cpu_times) * 1e3
    line = {"report": "config %d" % n, "workload": name.replace("fp32", "fp16") if args.half else name, "dtype": label, "ms_per_step": ms,
            "tflops": flop / ms / 1e9,
            ("frac_of_fp16_peak" if args.half else "frac_of_tf32_peak_over_3"): flop / ms / 1e9 / (2250.0 if args.half else 1100.0 / 3),
            "max_rel_err_vs_oracle": err, "tolerance": tol,
            "l2": "flushed between iterations (256 MiB write)", "steps": args.steps, "kernels": paths,
            "cpu": {"ms": cpu_ms, "kind": ref.kind, "threads": 1 if kind == "matmul" else ref.threads(),
                    "gflops": flop / cpu_ms / 1e6}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=5, choices=[1, 2, 3, 4, 5], help="BASELINE configuration; 5 (default) is the benchmark "
                    "line, 1-4 print an auxiliary fp32 report for one operator")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
