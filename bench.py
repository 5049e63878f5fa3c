"""Benchmark of the op-kernel hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-ops]

Headline (the line's `metric`/`value`): training throughput, in samples/s, of the data-parallel MLP
configuration -- 8 x Linear(4096, 4096) with Tanh between them, MSE loss against N(0,1) targets,
global batch 16384 of N(0,1) rows sharded over N ranks, SGD lr 1e-3, Kaiming-uniform init from seed
0, fp32 with 3xTF32 tensor-core products -- on synthetic data.  A step is forward + backward +
gradient all-reduce + update on one global batch.  `value` is measured with the batch resident in
HBM; `e2e` feeds every step's batch from pinned host memory (double-buffered host->device copies
inside the timed region) and reads the loss back to the host every step.

At N = 1 the same line also carries, under "ops", the per-op sweep of the other configurations
(elementwise and reductions in GB/s against the measured HBM copy rate, matmul in TFLOP/s), the
`roofline` of the dominant kernel of the step (the 3xTF32 GEMM) and `cpu_baseline`, the reference's
own CPU path timed on this box on a bounded sample.

`--impl reference` times the reference's CPU implementation of the same step (its native module
built into oracle/_ref, else the C restatement) on a bounded sample and prints the same line shape.

Under torchrun (N > 1) one process drives one GPU; torch.distributed (gloo) is used only for the
host-side rendezvous, barriers and the max-over-ranks of the device timings.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WIDTH, LAYERS, GLOBAL_BATCH, LR = 4096, 8, 16384, 1e-3
WORKLOAD = ("configs[4]: 8-layer MLP fp32 width 4096, tanh, MSE vs N(0,1) targets, global batch 16384 ~N(0,1) "
            "sharded data-parallel, SGD lr 1e-3, Kaiming-uniform init seed 0")


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def measure_gemm_peaks(seconds: float = 3.0) -> dict:
    """Denominators that MEASURED_PEAKS.json does not hold, taken the way it takes the bf16 one: cuBLAS
    through torch.matmul at 8192^3 on this GPU, CUDA events, best of 10 (burst) and back to back for a
    few seconds (sustained, under the power cap).  TF32: fp32 operands with TF32 products allowed -- the
    tensor-pipe peak the 3xTF32 kernel is measured against.  FP32: the same product with TF32 off --
    cuBLAS SGEMM on the CUDA cores, the denominator of the exact-mode SIMT kernel.  torch is only the
    way to reach cuBLAS here; nothing of it is on the product path."""
    import torch

    n = 8192
    flops = 2.0 * n ** 3
    a = torch.randn(n, n, device="cuda", dtype=torch.float32)
    b = torch.randn(n, n, device="cuda", dtype=torch.float32)
    c = torch.empty(n, n, device="cuda", dtype=torch.float32)
    out = {}
    for name, allow, budget in (("tf32", True, seconds), ("fp32", False, 1.0)):
        torch.backends.cuda.matmul.allow_tf32 = allow
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = 1e30
        for _ in range(10 if allow else 4):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        out[f"{name}_tflops"] = flops / best / 1e9
        iters = max(4, int(budget * 1e3 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            torch.matmul(a, b, out=c)
        e1.record()
        e1.synchronize()
        out[f"{name}_tflops_sustained"] = flops * iters / e0.elapsed_time(e1) / 1e9
    torch.backends.cuda.matmul.allow_tf32 = False
    del a, b, c
    torch.cuda.empty_cache()
    out["how"] = ("cuBLAS via torch.matmul, fp32 8192^3, CUDA events: best of 10 (burst) and back to back for ~3 s "
                  "(sustained); tf32 = allow_tf32 on, fp32 = off (SGEMM on the CUDA cores)")
    return out


# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.monotonic()] + [c.strip() for c in line.split(",")])

    def mark(self) -> float:
        return time.monotonic()

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0: float | None = None, t1: float | None = None) -> dict:
        """Samples that arrived in [t0, t1] (one sampling period of slack at the end); if the region was
        shorter than a period, the first sample after it started."""
        rows = [r[1:] for r in self.rows if t0 is None or (t0 <= r[0] <= (t1 or 1e30) + 0.25)]
        if not rows and t0 is not None:
            rows = [r[1:] for r in self.rows if r[0] >= t0][:1]
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
def reference_arm(args, rank: int) -> None:
    """The reference's CPU implementation of the step, on a bounded sample of the batch."""
    if rank != 0:
        return
    from oracle import oracle as O

    oracle = O.RefOracle() if O.ref_available() else O.PortOracle()
    t0 = time.perf_counter()
    stream = oracle.uniform(0, LAYERS * WIDTH * WIDTH)
    params = []
    for i in range(LAYERS):
        w = O.kaiming(oracle, stream[i * WIDTH * WIDTH:(i + 1) * WIDTH * WIDTH], WIDTH, WIDTH)
        params.append((w, np.zeros(WIDTH, np.float32)))
    del stream
    init_s = time.perf_counter() - t0
    batch = 2
    rng = np.random.default_rng(40)
    X = rng.standard_normal((batch, WIDTH)).astype(np.float32)
    Y = np.random.default_rng(41).standard_normal((batch, WIDTH)).astype(np.float32)
    limit_s = 150.0
    times = []
    total = args.warmup + args.steps
    for i in range(total):
        t = time.perf_counter()
        O.mlp_step(oracle, params, X, Y, LR, "tanh")
        dt = time.perf_counter() - t
        if i == 0 and dt * total > limit_s and batch > 1:
            batch = 1
            X, Y = X[:1], Y[:1]
        if i >= args.warmup:
            times.append((dt, X.shape[0]))
    seconds = sum(t for t, _ in times)
    samples = sum(b for _, b in times)
    value = samples / seconds
    cores = 1
    line = {
        "impl": "reference", "metric": "mlp_train_samples_per_s", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / len(times),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "width": WIDTH, "layers": LAYERS},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": oracle.kind,
                         "sample": f"batch of {times[-1][1]} of the 16384 rows through the full 8x4096^2 model, "
                                   f"forward+backward+SGD per step, single thread (the reference's CPU path has "
                                   f"no threading); init {init_s:.1f}s not counted; host has {os.cpu_count()} cores"},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    line["cpu_baseline"].update(extrapolated_full_batch(oracle))
    print(json.dumps(line))


def cpu_baseline_sample(limit_s: float = 20.0) -> dict:
    """Rank 0, N = 1: one step of the reference's CPU path on a batch of 2 rows of the workload."""
    from oracle import oracle as O

    oracle = O.RefOracle() if O.ref_available() else O.PortOracle()
    stream = oracle.uniform(0, LAYERS * WIDTH * WIDTH)
    params = []
    for i in range(LAYERS):
        w = O.kaiming(oracle, stream[i * WIDTH * WIDTH:(i + 1) * WIDTH * WIDTH], WIDTH, WIDTH)
        params.append((w, np.zeros(WIDTH, np.float32)))
    del stream
    batch = 2
    X = np.random.default_rng(40).standard_normal((batch, WIDTH)).astype(np.float32)
    Y = np.random.default_rng(41).standard_normal((batch, WIDTH)).astype(np.float32)
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 and (time.perf_counter() - t_start) < limit_s:
        t = time.perf_counter()
        O.mlp_step(oracle, params, X, Y, LR, "tanh")
        times.append(time.perf_counter() - t)
    best = min(times)
    out = {"value": batch / best, "unit": "samples/s", "cores": 1, "kind": oracle.kind,
           "sample": f"best of {len(times)} steps on a batch of {batch} of the 16384 rows through the full "
                     f"8x4096^2 model (forward+backward+SGD), single thread: the reference's CPU path has no "
                     f"threading; host has {os.cpu_count()} cores"}
    out.update(extrapolated_full_batch(oracle))
    return out


def extrapolated_full_batch(oracle, rows: int = 48) -> dict:
    """One full-size layer product of the step (activations x 4096^2 weights) on the reference's CPU path,
    timed on `rows` of the 16384 rows; the full-batch step is 23 such products over all rows (the
    elementwise work is three orders of magnitude smaller), so its rate follows by proportion.  Labelled
    as extrapolated: nobody ran the ~10-hour step."""
    A = np.random.default_rng(40).standard_normal((rows, WIDTH)).astype(np.float32)
    W = np.random.default_rng(31).uniform(-0.04, 0.04, (WIDTH, WIDTH)).astype(np.float32)
    t = time.perf_counter()
    oracle.matmul(A, W)
    dt = time.perf_counter() - t
    gflops = 2.0 * rows * WIDTH * WIDTH / dt / 1e9
    step_s = 2.0 * GLOBAL_BATCH * WIDTH * WIDTH * 23 / (gflops * 1e9)
    return {"full_size_layer_product_gflops": round(gflops, 3), "layer_product_sample": f"{rows} of 16384 rows x 4096 x 4096",
            "extrapolated_full_batch_value": GLOBAL_BATCH / step_s, "extrapolated_full_batch_seconds_per_step": round(step_s, 1),
            "extrapolated": True}


# ---------------------------------------------------------------------------------------------
def build_model(nt, nn):
    nt.manual_seed(0)
    layers = []
    for i in range(LAYERS):
        layers.append(nn.Linear(WIDTH, WIDTH, device="cuda"))
        if i < LAYERS - 1:
            layers.append(nn.Tanh())
    return nn.Sequential(*layers)


def pinned(nt, array: np.ndarray):
    """Copy `array` into a pinned host storage; returns (storage, numpy view)."""
    s = nt._C.Storage.allocate(array.size, nt.float32, nt.Device.Cpu)
    view = np.frombuffer(memoryview(s), dtype=np.float32)
    view[:] = array.reshape(-1)
    return s, view


def time_ops(nt, peaks: dict) -> dict:
    """Per-op sweep of the elementwise / reduction / matmul configurations at N = 1.

    HBM-bound ops are timed as `iters` back-to-back launches through the `_C` boundary (prebuilt
    views, so the host issues faster than the device drains) between one pair of events.  Launch i
    works on buffer set i mod n, with n chosen so that the sets together exceed 4x the L2 (inputs and
    the last n outputs are all distinct allocations): nothing a launch touches is still cached from
    the previous pass over the same set.  Matmuls (milliseconds each) are timed one launch at a time
    with the L2 flushed by a 512 MB fill in between.
    """
    _C = nt._C
    F32, CUDA = nt.float32, nt.Device.Cuda
    r = np.random.default_rng
    hbm = peaks["hbm_gbs"]
    out: dict = {}
    L2_BYTES = 126 * 1024 * 1024

    def dev(a):
        return nt.Tensor.from_numpy(a, "cuda")

    def copies(t, n):
        return [t] + [t.clone() for _ in range(n - 1)]

    def stream_time(calls, iters=40):
        n = len(calls)
        ring = [c() for c in calls]
        ring = [c() for c in calls]
        _C.cuda_sync()
        e0 = _C.Event().record()
        for i in range(iters):
            ring[i % n] = calls[i % n]()
        e1 = _C.Event().record()
        ms = e0.elapsed_ms(e1) / iters
        del ring
        return ms

    def record(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        out[name] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_of_measured_hbm": round(gbs / hbm, 3)}

    def nsets(nbytes):
        return max(3, -(-4 * L2_BYTES // nbytes))

    N = 4096
    numel = N * N
    host = {"a": r(10).uniform(-1, 1, (N, N)), "b": r(11).uniform(-1, 1, (N, N)), "d": r(12).uniform(0.5, 2, (N, N)),
            "n": r(14).standard_normal((N, N)), "p": r(15).uniform(0.1, 10, (N, N)), "G": r(16).standard_normal((N, N))}
    v_ = dev(r(13).uniform(-1, 1, (N,)).astype(np.float32))
    dv_ = dev(r(17).uniform(0.5, 2, (N,)).astype(np.float32))

    # each op is timed as itself: tanh / tanh_backward without the TF32 planes they add for a following
    # product (8 more bytes written per element); the rows named "+planes" time that form
    _C.set_producer_planes(False)
    with nt.no_grad():
        # ---- binary forward: contiguous, row broadcast, transposed operand
        k = nsets(3 * numel * 4)
        A = copies(dev(host["a"].astype(np.float32)), k)
        B = copies(dev(host["b"].astype(np.float32)), k)
        D = copies(dev(host["d"].astype(np.float32)), k)
        for name, kern in (("add", _C.add), ("sub", _C.subtract), ("mul", _C.multiply), ("truediv", _C.divide)):
            Y, yv = (D, dv_) if name == "truediv" else (B, v_)
            va = [t._C_view for t in A]
            record(f"{name}.contiguous", stream_time([lambda i=i: kern(va[i], Y[i]._C_view) for i in range(k)]),
                   3 * numel * 4)
            vrow = yv.expand(N, N)._C_view
            record(f"{name}.broadcast_row", stream_time([lambda i=i: kern(va[i], vrow) for i in range(k)]),
                   (2 * numel + N) * 4)
            vt = [t.T._C_view for t in Y]
            record(f"{name}.transposed", stream_time([lambda i=i: kern(va[i], vt[i]) for i in range(k)]), 3 * numel * 4)
        del B, D
        # ---- unary forward
        k = nsets(2 * numel * 4)
        Nn = copies(dev(host["n"].astype(np.float32)), k)
        Pp = copies(dev(host["p"].astype(np.float32)), k)
        A = A[:k] + [A[0].clone() for _ in range(max(0, k - len(A)))]
        for name, kern, src in (("pow2", lambda v: _C.pow(v, 2.0), A), ("exp", _C.exp, Nn), ("neg", _C.neg, Nn),
                                ("relu", _C.relu, Nn), ("tanh", _C.tanh, Nn), ("sigmoid", _C.sigmoid, Nn),
                                ("log", _C.log, Pp), ("sqrt", _C.sqrt, Pp)):
            views = [t._C_view for t in src]
            record(f"{name}.forward", stream_time([lambda i=i: kern(views[i]) for i in range(k)]), 2 * numel * 4)
        # ---- fused backward kernels: upstream gradient + saved tensor -> input gradient
        k = nsets(3 * numel * 4)
        G = copies(dev(host["G"].astype(np.float32)), k)
        gv = [t._C_view for t in G]
        saved = {"relu": [nt.relu(t) for t in Nn[:k]], "tanh": [nt.tanh(t) for t in Nn[:k]],
                 "sigmoid": [nt.sigmoid(t) for t in Nn[:k]], "exp": [t.exp() for t in Nn[:k]], "log": Pp[:k],
                 "sqrt": [nt.sqrt(t) for t in Pp[:k]]}
        kernels = {"relu": _C.relu_backward, "tanh": _C.tanh_backward, "sigmoid": _C.sigmoid_backward,
                   "exp": _C.exp_backward, "log": _C.log_backward, "sqrt": _C.sqrt_backward}
        for name, kern in kernels.items():
            sv = [t._C_view for t in saved[name]]
            record(f"{name}.backward", stream_time([lambda i=i: kern(gv[i], sv[i]) for i in range(k)]), 3 * numel * 4)
            saved[name] = None
        _C.set_producer_planes(True)
        tsv = [nt.tanh(t) for t in Nn[:k]]
        record("tanh.forward+planes", stream_time([lambda i=i: _C.tanh(Nn[i]._C_view) for i in range(k)]), 4 * numel * 4)
        record("tanh.backward+planes", stream_time([lambda i=i: _C.tanh_backward(gv[i], tsv[i]._C_view) for i in range(k)]),
               5 * numel * 4)
        _C.set_producer_planes(False)
        del tsv
        av = [t._C_view for t in A[:k]]
        record("pow2.backward", stream_time([lambda i=i: _C.pow_backward(gv[i], av[i], 2.0) for i in range(k)]),
               3 * numel * 4)
        # binary backward, one launch: mul' = (x2*g, x1*g), div' = (g/x2, ((-x1)/x2^2)*g): g, x1, x2 -> dx1, dx2 = 5 N floats
        Bk = copies(dev(host["b"].astype(np.float32)), k)
        Dk = copies(dev(host["d"].astype(np.float32)), k)
        bv, dv2 = [t._C_view for t in Bk], [t._C_view for t in Dk]
        record("mul.backward", stream_time([lambda i=i: _C.mul_backward(gv[i], av[i], bv[i]) for i in range(k)]), 5 * numel * 4)
        record("truediv.backward", stream_time([lambda i=i: _C.div_backward(gv[i], av[i], dv2[i]) for i in range(k)]),
               5 * numel * 4)
        # one operand seen through a transposed view: its gradient x1*g is written in x2's own (transposed) order
        bt = [t.T._C_view for t in Bk]
        record("mul.transposed.backward", stream_time(
            [lambda i=i: (_C.multiply(bt[i], gv[i]), _C.multiply(av[i], gv[i])) for i in range(k)]), 5 * numel * 4)
        # row-broadcast operand [N] against [N,N]: dx1 = v*g, dv = column sums of x1*g (the unbroadcast):
        # g, x1 -> dx1, tmp -> dv.  5 N + (N + C) floats by the per-op byte accounting of the reference (mem_bytes)
        vrow = v_.expand(N, N)._C_view

        def mul_bcast_backward(i):
            dx1 = _C.multiply(vrow, gv[i])
            tmp = _C.multiply(av[i], gv[i])
            return dx1, _C.sum(_C.TensorView(tmp, (N, N), (N, 1), 0), [0], F32)

        record("mul.broadcast_row.backward", stream_time([lambda i=i: mul_bcast_backward(i) for i in range(k)]),
               (6 * numel + N) * 4)
        record("add.broadcast_row.grad_of_row", stream_time([lambda i=i: _C.sum(gv[i], [0], F32) for i in range(k)]),
               (numel + N) * 4)
        # pow through the strided paths
        at = [t.T._C_view for t in A[:k]]
        record("pow2.transposed", stream_time([lambda i=i: _C.pow(at[i], 2.0) for i in range(k)]), 2 * numel * 4)
        record("pow2.broadcast_row", stream_time([lambda: _C.pow(vrow, 2.0)] * 3), (numel + N) * 4)
        del A, Nn, Pp, G, saved, gv, av, Bk, Dk, bv, dv2, bt, at

        # ---- reductions
        M = 8192
        k = 3
        X = copies(dev(r(20).standard_normal((M, M)).astype(np.float32)), k)
        xv = [t._C_view for t in X]
        y3 = dev(r(21).standard_normal((64, 1, 16384)).astype(np.float32))
        count = {(0,): M, (1,): M, (0, 1): M * M}
        for label, axes in (("dim0", (0,)), ("dim1", (1,)), ("full", (0, 1))):
            ax = list(axes)
            record(f"sum.{label}", stream_time([lambda i=i: _C.sum(xv[i], ax, F32) for i in range(k)]), M * M * 4)
            record(f"max.{label}", stream_time([lambda i=i: _C.max(xv[i], ax) for i in range(k)]), M * M * 4)
            record(f"min.{label}", stream_time([lambda i=i: _C.min(xv[i], ax) for i in range(k)]), M * M * 4)
            cnt = count[axes]  # MeanOp.forward: the sum divided by the count where the reduction finishes
            record(f"mean.{label}", stream_time([lambda i=i: _C.mean_f32(xv[i], ax, cnt) for i in range(k)]), M * M * 4)
        y3v = y3._C_view
        for op, kern in (("sum", lambda v: _C.sum(v, [2], F32)), ("max", lambda v: _C.max(v, [2])),
                         ("min", lambda v: _C.min(v, [2]))):
            record(f"{op}.[64,1,16384].last", stream_time([lambda: kern(y3v)] * 3, iters=100), y3.numel * 4)
        # backward: the reference's sum backward is a stride-0 view (0 bytes); the materialised broadcast
        # and the mean / max backward kernels are what moves data
        ones_row = dev(np.ones((M,), np.float32))
        row_view = ones_row.expand(M, M)._C_view
        record("sum.backward_materialised", stream_time([lambda: _C.clone_contiguous_view_from(row_view)] * 3), M * M * 4)
        # mean backward: the kept elements are divided once, the quotient is expanded as a stride-0 view;
        # a consumer that needs it dense pays the materialising broadcast
        denom_row = _C.TensorView(_C.full(1, float(M), F32, CUDA), (M,), (0,), 0)

        def mean_backward():
            q = _C.divide(ones_row._C_view, denom_row)
            return _C.clone_contiguous_view_from(_C.TensorView(q, (M, M), (0, 1), 0))

        record("mean.backward_materialised", stream_time([mean_backward] * 3), M * M * 4)
        m1 = [t.max((1,)) for t in X]
        g_full = ones_row.reshape(M, 1).expand(M, M)._C_view
        m_full = [m.reshape(M, 1).expand(M, M)._C_view for m in m1]
        record("max.backward", stream_time([lambda i=i: _C.extremum_backward(g_full, xv[i], m_full[i], [1])
                                            for i in range(k)], iters=20), 2 * M * M * 4)
        del m1, m_full
        # max / min backward over the leading dim and over the whole tensor: two launches over x (count the
        # positions equal to the extremum with integer atomics, then write g * unique-mask), read x + write dx
        for label, axes, kept in (("dim0", [0], (1, M)), ("full", [0, 1], (1, 1))):
            for op in ("max", "min"):
                mm = [getattr(t, op)(tuple(axes)) for t in X]
                mf = [m.reshape(*kept).expand(M, M)._C_view for m in mm]
                gk = dev(np.ones(kept, np.float32)).expand(M, M)._C_view
                record(f"{op}.backward.{label}", stream_time(
                    [lambda i=i: _C.extremum_backward(gk, xv[i], mf[i], axes) for i in range(k)], iters=20), 2 * M * M * 4)
                del mm, mf
        # ---- index-array gather / scatter of whole rows by a permutation (read + write = 8 bytes/element)
        perm_view = [dev(r(22).permutation(M).astype(np.int64))._C_view]
        plan = dict(fancy_dims_in_src=[0], fancy_dims_data=perm_view, out_axis_is_fancy=[True, False],
                    out_axis_target=[0, 1], checked=True)
        record("gather.rows_permuted", stream_time(
            [lambda i=i: _C.gather_from_axes(x=xv[i], new_shape=[M, M], **plan) for i in range(k)], iters=20), 2 * M * M * 4)
        T_ = [t.clone() for t in X]
        tv = [t._C_view for t in T_]
        record("scatter.rows_permuted", stream_time(
            [lambda i=i: _C.scatter_to_axes(src=xv[i], out=tv[i], unique=True, **plan) for i in range(k)], iters=20),
            2 * M * M * 4)
        record("scatter.rows_permuted.ordered", stream_time(
            [lambda i=i: _C.scatter_to_axes(src=xv[i], out=tv[i], unique=False, **plan) for i in range(k)], iters=20),
            2 * M * M * 4)
        del X, xv, T_, tv

        # ---- matmul
        def flush():
            _C.zeros(128 * 1024 * 1024, F32, CUDA)  # 512 MB written: larger than L2

        def timed(fn, iters, warm=2):
            for _ in range(warm):
                fn()
            ms = []
            for _ in range(iters):
                flush()
                e0 = _C.Event().record()
                fn()
                e1 = _C.Event().record()
                ms.append(e0.elapsed_ms(e1))
            return statistics.median(ms)

        tf32_peak = peaks["tf32_tflops"]      # burst figure: these launches are timed alone
        fp32_peak = peaks["fp32_tflops"]
        for label, (m, kk, n, bt) in {"4096x4096x4096": (4096, 4096, 4096, 1), "8192x1024x4096": (8192, 1024, 4096, 1),
                                      "32x512x512x512": (512, 512, 512, 32)}.items():
            shape_a = (bt, m, kk) if bt > 1 else (m, kk)
            shape_b = (bt, kk, n) if bt > 1 else (kk, n)
            shape_c = (bt, m, n) if bt > 1 else (m, n)
            Am = dev(r(30).uniform(-1, 1, shape_a).astype(np.float32))
            Bm = dev(r(31).uniform(-1, 1, shape_b).astype(np.float32))
            Gc = dev(r(32).uniform(-1, 1, shape_c).astype(np.float32))
            flops = 2.0 * bt * m * n * kk
            va, vb, vg = Am._C_view, Bm._C_view, Gc._C_view
            vat, vbt = Am.transpose(-2, -1)._C_view, Bm.transpose(-2, -1)._C_view
            for mode, mname in ((1, "3xtf32"), (0, "fp32_simt")):
                _C.set_matmul_mode(mode)
                try:
                    res = {}
                    for which, fn in (("forward", lambda: _C.matmul(va, vb)), ("grad_a", lambda: _C.matmul(vg, vbt)),
                                      ("grad_b", lambda: _C.matmul(vat, vg))):
                        _C.matmul_profile_enable(True)
                        ms = timed(fn, iters=5 if mode == 0 else 10)
                        total, launches = _C.matmul_profile_read()
                        _C.matmul_profile_enable(False)
                        res[which] = {"ms": round(ms, 4), "TFLOP/s": round(flops / ms / 1e9, 2)}
                        if mode == 0:
                            res[which]["frac_of_fp32_sgemm_peak"] = round(flops / ms / 1e9 / fp32_peak, 3)
                        if mode == 1:
                            res[which]["frac_of_tf32_peak"] = round(flops / ms / 1e9 / tf32_peak, 3)
                            kms = total / max(launches, 1)
                            res[which]["gemm_kernel_ms"] = round(kms, 4)
                            res[which]["tensor_TFLOP/s_3_products"] = round(3 * flops / ms / 1e9, 1)
                            res[which]["tensor_frac_of_tf32_peak"] = round(3 * flops / ms / 1e9 / tf32_peak, 3)
                            res[which]["gemm_kernel_tensor_frac_of_tf32_peak"] = round(3 * flops / kms / 1e9 / tf32_peak, 3)
                    out[f"matmul.{label}.{mname}"] = res
                finally:
                    _C.set_matmul_mode(1)
            del Am, Bm, Gc
    _C.set_producer_planes(True)
    out["mlp_784_256_10"] = time_config_1(nt)
    out["_notes"] = ("HBM-bound ops: back-to-back launches through the _C boundary over rotating buffer sets larger "
                     "than 4x L2, one event pair around 40 launches; bytes are the reference's mem_bytes() accounting "
                     "(sum/max/min count the input only); matmul: L2 flushed by a 512 MB fill between single timed "
                     "launches, `ms` includes the operand split kernels, gemm_kernel_ms is the tcgen05 kernel alone; "
                     "TF32 and FP32 peaks are cuBLAS rates measured in this run (burst)")
    return out


def time_config_1(nt) -> dict:
    """configs[0]: Linear(784,256)-ReLU-Linear(256,10), MSE, batch 256, seed-0 init, SGD lr 0.01 -- a step is
    ~40 small launches, so it is issue-bound: timed eagerly (launches issued from Python) and as one
    CUDA-graph replay per step."""
    import nanotorch_b200.nn as nn

    _C = nt._C
    nt.manual_seed(0)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10)).to("cuda")
    X = nt.Tensor.from_numpy(np.random.default_rng(1).standard_normal((256, 784)).astype(np.float32), "cuda")
    Y = nt.Tensor.from_numpy(np.random.default_rng(2).standard_normal((256, 10)).astype(np.float32), "cuda")
    opt = nn.GradientDescent(model.parameters(), lr=0.01)

    def step():
        loss = nt.mean((model(X) - Y) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss

    for _ in range(10):
        loss = step()
    first = float(loss.numpy())
    steps = 100
    l0 = _C.launch_count()
    e0 = _C.Event().record()
    for _ in range(steps):
        loss = step()
    e1 = _C.Event().record()
    ms_eager = e0.elapsed_ms(e1) / steps
    launches = (_C.launch_count() - l0) // steps
    graph = _C.Graph()
    with graph.capture():
        gl = step()
    for _ in range(5):
        graph.replay()
    _C.cuda_sync()
    e0 = _C.Event().record()
    for _ in range(steps):
        graph.replay()
    e1 = _C.Event().record()
    ms_graph = e0.elapsed_ms(e1) / steps
    last = float(gl.numpy())
    graph.close()
    return {"samples/s_eager": round(256 / ms_eager * 1e3, 1), "samples/s_graph": round(256 / ms_graph * 1e3, 1),
            "ms_per_step_eager": round(ms_eager, 4), "ms_per_step_graph": round(ms_graph, 4), "launches_per_step": launches,
            "loss_after_10_steps": first, "loss_after_215_steps": last}


def compact_ops(ops: dict) -> dict:
    """name -> [GB/s, fraction of the measured HBM copy rate] for the HBM-bound rows,
    name.pass -> [TFLOP/s, fraction] for the matmul rows (3xtf32: of the measured TF32 peak, algorithmic
    2MNK flops, the 3 tensor products per fp32 product not counted; fp32_simt: of the measured SGEMM rate)."""
    out = {}
    for name, row in ops.items():
        if name.startswith("_"):
            continue
        if "GB/s" in row:
            out[name] = [row["GB/s"], row["frac_of_measured_hbm"]]
        elif name.startswith("matmul."):
            for which, r in row.items():
                frac = r.get("frac_of_tf32_peak", r.get("frac_of_fp32_sgemm_peak"))
                out[f"{name}.{which}"] = [r["TFLOP/s"], frac]
        elif name == "mlp_784_256_10":
            out[name] = row
    return out


def reference_cuda_column() -> dict:
    """Optional comparison column (--ref-cuda): the reference's OWN generic CUDA kernels, compiled for
    sm_100 into oracle/_ref by oracle/Makefile, on this GPU through the reference's `_C` API.  Timed the
    way the reference times itself (scripts/profile_ops.py:61-89): perf_counter around the call plus a
    device sync, best of 5 after a warm-up.  Not part of the default run."""
    from oracle import oracle as O

    if not O.ref_available():
        return {"unavailable": "oracle/_ref is not built"}
    m = O.load_ref_module()
    if not m.is_cuda_available():
        return {"unavailable": "no CUDA device"}
    F32, CPU, CUDA = m.Dtype.Float32, m.Device.Cpu, m.Device.Cuda
    r = np.random.default_rng

    def dev(a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        s_ = m.Storage.allocate(a.size, F32, CPU)
        np.asarray(memoryview(s_))[:] = a.reshape(-1)
        return s_.to(CUDA), a.shape

    def view(st, shape, strides=None, offset=0):
        if strides is None:
            strides, acc = [], 1
            for e in reversed(shape):
                strides.insert(0, acc)
                acc *= e
        return m.TensorView(st, list(shape), list(strides), offset)

    def best(fn, reps=5):
        fn()
        m.cuda_sync()
        ts = []
        for _ in range(reps):
            t = time.perf_counter()
            fn()
            m.cuda_sync()
            ts.append(time.perf_counter() - t)
        return min(ts) * 1e3

    out = {}
    N = 4096
    a, _ = dev(r(10).uniform(-1, 1, (N, N)))
    b, _ = dev(r(11).uniform(-1, 1, (N, N)))
    v, _ = dev(r(13).uniform(-1, 1, (N,)))
    n_, _ = dev(r(14).standard_normal((N, N)))
    va, vb = view(a, (N, N)), view(b, (N, N))
    for name, fn, nbytes in (
            ("add.contiguous", lambda: m.add(va, vb), 3 * N * N * 4),
            ("add.broadcast_row", lambda: m.add(va, view(v, (N, N), (0, 1))), (2 * N * N + N) * 4),
            ("add.transposed", lambda: m.add(va, view(b, (N, N), (1, N))), 3 * N * N * 4),
            ("exp.forward", lambda: m.exp(view(n_, (N, N))), 2 * N * N * 4),
            ("tanh.forward", lambda: m.tanh(view(n_, (N, N))), 2 * N * N * 4)):
        ms = best(fn)
        out[name] = {"ms": round(ms, 4), "GB/s": round(nbytes / ms / 1e6, 1)}
    M = 8192
    x, _ = dev(r(20).standard_normal((M, M)))
    vx = view(x, (M, M))
    for name, fn in (("sum.dim0", lambda: m.sum(vx, [0], F32)), ("sum.dim1", lambda: m.sum(vx, [1], F32)),
                     ("sum.full", lambda: m.sum(vx, [0, 1], F32)), ("max.dim1", lambda: m.max(vx, [1]))):
        ms = best(fn)
        out[name] = {"ms": round(ms, 4), "GB/s": round(M * M * 4 / ms / 1e6, 1)}
    flops = 2.0 * N * N * N
    ms = best(lambda: m.matmul(va, vb), reps=3)
    out["matmul.4096x4096x4096.forward"] = {"ms": round(ms, 3), "TFLOP/s": round(flops / ms / 1e9, 2)}
    # both gradients multiply by a transposed VIEW and drop to the one-thread-per-output kernel
    ms = best(lambda: m.matmul(va, view(b, (N, N), (1, N))), reps=1)
    out["matmul.4096x4096x4096.grad_a"] = {"ms": round(ms, 3), "TFLOP/s": round(flops / ms / 1e9, 2)}
    compact = {k: v.get("GB/s", v.get("TFLOP/s")) for k, v in out.items()}
    compact["_units"] = ("GB/s (TFLOP/s for matmul): the reference's own generic CUDA kernels recompiled with "
                         "-gencode arch=compute_100,code=sm_100, perf_counter + device sync per call, best of 5")
    return compact


def reference_cpu_column(limit_s: float = 90.0) -> dict:
    """Optional comparison column (--ref-cpu): the reference's own CPU kernels (oracle/_ref) on the per-op
    configurations, single thread as the reference runs them, operands already in its storages, best of 2
    after a warm-up, perf_counter around the native call.  Elementwise and reductions at full size; each
    matmul on a bounded sample of its rows (the full 4096^3 product takes minutes).  Needs no GPU."""
    from oracle import oracle as O

    if not O.ref_available():
        return {"unavailable": "oracle/_ref is not built"}
    o = O.RefOracle()
    m = o.m
    r = np.random.default_rng
    t_start = time.perf_counter()

    def best(fn, reps=2):
        fn()
        ts = []
        for _ in range(reps):
            t = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t)
        return min(ts) * 1e3

    def view(array):
        return o._tv(np.ascontiguousarray(array, dtype=np.float32))  # (TensorView, storage kept alive)

    out: dict = {}
    N = 4096
    (va, sa), (vb, sb) = view(r(10).uniform(-1, 1, (N, N))), view(r(11).uniform(-1, 1, (N, N)))
    (vn, sn), (vp, sp_) = view(r(14).standard_normal((N, N))), view(r(15).uniform(0.1, 10, (N, N)))
    _, sv = view(r(13).uniform(-1, 1, (N,)))
    v_row = m.TensorView(sv, [N, N], [0, 1], 0)       # row broadcast: stride 0
    vb_t = m.TensorView(sb, [N, N], [1, N], 0)        # transposed view
    ew = [("add.contiguous", lambda: m.add(va, vb), 3), ("truediv.contiguous", lambda: m.divide(va, vp), 3),
          ("add.broadcast_row", lambda: m.add(va, v_row), 2), ("add.transposed", lambda: m.add(va, vb_t), 3),
          ("exp.forward", lambda: m.exp(vn), 2), ("tanh.forward", lambda: m.tanh(vn), 2),
          ("sigmoid.forward", lambda: m.sigmoid(vn), 2), ("relu.forward", lambda: m.relu(vn), 2),
          ("log.forward", lambda: m.log(vp), 2), ("pow2.forward", lambda: m.pow(va, 2.0), 2)]
    for name, fn, streams in ew:
        if time.perf_counter() - t_start > limit_s:
            break
        ms = best(fn)
        out[name] = {"ms": round(ms, 2), "GB/s": round(streams * N * N * 4 / ms / 1e6, 2)}
    M = 8192
    vx, sx = view(r(20).standard_normal((M, M)))
    F32 = o.F32
    for name, fn in (("sum.dim0", lambda: m.sum(vx, [0], F32)), ("sum.dim1", lambda: m.sum(vx, [1], F32)),
                     ("sum.full", lambda: m.sum(vx, [0, 1], F32)), ("max.dim1", lambda: m.max(vx, [1]))):
        if time.perf_counter() - t_start > limit_s:
            break
        ms = best(fn, reps=1)
        out[name] = {"ms": round(ms, 2), "GB/s": round(M * M * 4 / ms / 1e6, 2)}
    rows = 64  # of the left operand's rows
    for label, (m_, k_, n_) in {"4096x4096x4096": (4096, 4096, 4096), "8192x1024x4096": (8192, 1024, 4096)}.items():
        if time.perf_counter() - t_start > limit_s:
            break
        (vA, sA), (vB, sB) = view(r(30).uniform(-1, 1, (rows, k_))), view(r(31).uniform(-1, 1, (k_, n_)))
        ms = best(lambda: m.matmul(vA, vB), reps=1)
        out[f"matmul.{label}.forward"] = {"sample": f"{rows} of {m_} rows", "ms_sample": round(ms, 1),
                                          "GFLOP/s": round(2.0 * rows * k_ * n_ / ms / 1e6, 2)}
    out["_notes"] = (f"the reference's CPU kernels, 1 thread of {os.cpu_count()} (it has no threading), perf_counter "
                     "around the native call, best of 2 after a warm-up; bytes as in the GPU sweep; matmul on a row sample")
    return out


def product_arm(args, rank: int, local_rank: int, world: int) -> None:
    import nanotorch_b200 as nt
    import nanotorch_b200.nn as nn
    from nanotorch_b200.dp import Communicator, DataParallelSGD, shard_bounds

    _C = nt._C
    _C.set_device(local_rank)
    if not nt.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path in the product)")
    dist = None
    if world > 1:
        import torch.distributed as dist  # host-side plumbing only (gloo): rendezvous, barrier, max of timings

        dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world)

    def exchange_id(uid):
        box = [uid]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def barrier():
        _C.cuda_sync()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch

        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    comm = Communicator(rank, world, exchange_id, timeout_s=300.0)
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank).__enter__()  # runs for the whole benchmark; regions are cut out by time
    lo, hi = shard_bounds(GLOBAL_BATCH, rank, world)
    local = hi - lo

    def all_mean(values):
        """Mean over ranks of per-rank values (equal shards: the global-batch loss from the shard losses)."""
        if dist is None:
            return [float(v) for v in values]
        import torch

        t = torch.tensor([float(v) for v in values], dtype=torch.float64)
        dist.all_reduce(t)
        return (t / world).tolist()

    # ---------------- cross-world parity: 5 steps from the seed-0 state, global-batch loss and a checksum of
    # the first layer's weights; identical at every N up to the summation order of the gradient exchange
    model = build_model(nt, nn)
    opt = DataParallelSGD(model.parameters(), LR, comm)
    Xg = np.random.default_rng(40).standard_normal((GLOBAL_BATCH, WIDTH), dtype=np.float32)
    Yg = np.random.default_rng(41).standard_normal((GLOBAL_BATCH, WIDTH), dtype=np.float32)
    Xp, Yp = nt.Tensor.from_numpy(Xg[lo:hi], "cuda"), nt.Tensor.from_numpy(Yg[lo:hi], "cuda")
    del Xg, Yg
    parity_losses = []
    for _ in range(5):
        loss = nt.mean((model(Xp) - Yp) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        parity_losses.append(float(loss.numpy()))
    global_loss = all_mean(parity_losses)
    w0 = model.parameters()[0].numpy().astype(np.float64)
    w0_checksum, w0_abs_checksum = float(w0.sum()), float(np.abs(w0).sum())
    del Xp, Yp, w0, loss
    opt.detach()
    del model, opt

    model = build_model(nt, nn)   # seed 0 again: the timed part starts from the initial state
    opt = DataParallelSGD(model.parameters(), LR, comm)
    # two synthetic global batches (alternated by the end-to-end loop); this rank's rows only
    host = []
    for seed in (40, 42):
        Xg = np.random.default_rng(seed).standard_normal((GLOBAL_BATCH, WIDTH), dtype=np.float32)
        Yg = np.random.default_rng(seed + 1).standard_normal((GLOBAL_BATCH, WIDTH), dtype=np.float32)
        host.append((pinned(nt, Xg[lo:hi]), pinned(nt, Yg[lo:hi])))
        del Xg, Yg
    Xd = [nt.Tensor._new_contiguous(_C.Storage.allocate(local * WIDTH, nt.float32, nt.Device.Cuda), (local, WIDTH))
          for _ in range(2)]
    Yd = [nt.Tensor._new_contiguous(_C.Storage.allocate(local * WIDTH, nt.float32, nt.Device.Cuda), (local, WIDTH))
          for _ in range(2)]
    nbytes = local * WIDTH * 4

    def step(X, Y):
        loss = nt.mean((model(X) - Y) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss

    # ---------------- resident: batch already in HBM
    Xd[0].storage.upload(host[0][0][1].ctypes.data, nbytes)
    Yd[0].storage.upload(host[0][1][1].ctypes.data, nbytes)
    for _ in range(args.warmup):
        step(Xd[0], Yd[0])
    barrier()
    launches0 = _C.launch_count()
    _C.matmul_profile_enable(True)
    t_eager0 = sampler.mark()
    e0 = _C.Event().record()
    for _ in range(args.steps):
        loss = step(Xd[0], Yd[0])
    e1 = _C.Event().record()
    ms_resident = e0.elapsed_ms(e1)
    t_eager1 = sampler.mark()
    barrier()
    _C.matmul_profile_enable(False)
    gemm_ms, gemm_launches = _C.matmul_profile_read()
    launches = _C.launch_count() - launches0
    last_loss = float(loss.numpy())
    ms_eager = max_over_ranks(ms_resident)

    # ---------------- the same step captured once into a CUDA graph and replayed
    graph = _C.Graph()
    with graph.capture():
        graph_loss = step(Xd[0], Yd[0])
    for _ in range(args.warmup):
        graph.replay()
    barrier()
    launches0 = _C.launch_count()
    t_graph0 = sampler.mark()
    e0 = _C.Event().record()
    for _ in range(args.steps):
        graph.replay()
    e1 = _C.Event().record()
    ms_graph = e0.elapsed_ms(e1)
    t_graph1 = sampler.mark()
    barrier()
    graph_launches = _C.launch_count() - launches0
    last_loss = float(graph_loss.numpy())
    ms_graph = max_over_ranks(ms_graph)

    # ---------------- N > 1: the same captured step without the collectives (everything else alike: buckets,
    # updates on the side stream, 1/world scale).  The difference to the real step is what the exchange costs:
    # its exposed tail plus the SMs NCCL takes from the backward GEMMs while it runs.
    ms_no_exchange = None
    if world > 1:
        opt.detach()
        quiet = Communicator(0, 1, None)
        opt_q = DataParallelSGD(model.parameters(), LR, quiet)
        opt_q._grad_scale = 1.0 / world

        def step_q():
            loss_q = nt.mean((model(Xd[0]) - Yd[0]) ** 2)
            opt_q.zero_grad()
            loss_q.backward()
            opt_q.step()
            return loss_q

        step_q()
        gq = _C.Graph()
        with gq.capture():
            step_q()
        for _ in range(args.warmup):
            gq.replay()
        barrier()
        e0 = _C.Event().record()
        for _ in range(args.steps):
            gq.replay()
        e1 = _C.Event().record()
        ms_no_exchange = max_over_ranks(e0.elapsed_ms(e1)) / args.steps
        barrier()
        gq.close()
        opt_q.detach()
        for p in model.parameters():   # the real optimizer's hooks again
            from nanotorch_b200.autograd import leaf_grad_hooks
            leaf_grad_hooks[id(p)] = opt._on_grad
    use_graph = ms_graph <= ms_eager
    ms_resident = ms_graph if use_graph else ms_eager
    clock_window = (t_graph0, t_graph1) if use_graph else (t_eager0, t_eager1)

    # ---------------- end to end: every step's batch comes from pinned host memory
    def feed(i):
        hx, hy = host[i % 2]
        _C.upload_async(Xd[i % 2].storage, hx[1].ctypes.data, nbytes)
        _C.upload_async(Yd[i % 2].storage, hy[1].ctypes.data, nbytes)

    graphs = None
    if not use_graph:
        # eager collectives issued while a graph that captured collectives is alive were measured 3x
        # slower (NCCL keeps switching between its persistent and eager plans): never mix the two
        graph.close()
    if use_graph:  # one captured step per input buffer of the double-buffered feed
        g1 = _C.Graph()
        with g1.capture():
            loss1 = step(Xd[1], Yd[1])
        graphs = [(graph, graph_loss), (g1, loss1)]

    def e2e_loop(n, first):
        result = None
        for i in range(first, first + n):
            _C.upload_fence()      # compute waits for batch i
            feed(i + 1)            # batch i+1 streams in while step i computes
            if graphs is None:
                out = step(Xd[i % 2], Yd[i % 2])
            else:
                graphs[i % 2][0].replay()
                out = graphs[i % 2][1]
            result = float(out.numpy())  # device->host read of the loss, every step
        return result

    feed(0)
    e2e_loop(args.warmup, 0)
    barrier()
    e0 = _C.Event().record()
    t_wall = time.perf_counter()
    e2e_loop(args.steps, args.warmup)
    e1 = _C.Event().record()
    ms_e2e = max(e0.elapsed_ms(e1), 1e3 * (time.perf_counter() - t_wall))
    barrier()
    ms_e2e = max_over_ranks(ms_e2e)

    try:  # the TF32 / FP32 denominators, measured on this GPU after the timed regions (every rank alike), so
    # that seconds of full-power cuBLAS work cannot warm the part up under the headline numbers
        import torch

        torch.cuda.set_device(local_rank)
        peaks.update(measure_gemm_peaks())
        peaks["gemm_peaks_source"] = "measured in this run"
    except Exception as e:  # noqa: BLE001 -- no torch, or no room: fall back to the stated cross-check
        peaks.update({"tf32_tflops": peaks["bf16_tflops"] / 2, "tf32_tflops_sustained": peaks["bf16_tflops_sustained"] / 2,
                      "fp32_tflops": 74.0, "fp32_tflops_sustained": 74.0,
                      "gemm_peaks_source": f"not measured ({type(e).__name__}); TF32 taken as measured bf16 / 2, FP32 as the "
                                           f"nominal 148 SMs x 128 lanes x 2 x 1.965 GHz"})
    samples = GLOBAL_BATCH * args.steps
    value = samples / (ms_resident / 1e3)
    e2e_value = samples / (ms_e2e / 1e3)

    if rank == 0:
        m, k, n = local, WIDTH, WIDTH
        flops_per_launch = 2.0 * m * n * k            # algorithmic: one fp32 multiply-add per (m, n, k)
        avg_ms = gemm_ms / max(gemm_launches, 1)
        tf32_peak = peaks["tf32_tflops_sustained"]    # the kernel is timed inside a long, power-capped step
        achieved = flops_per_launch / avg_ms / 1e9 if gemm_launches else None
        full = local == GLOBAL_BATCH and _C.get_matmul_mode() == 1
        line = {
            "metric": "mlp_train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_resident / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_rank_batch": local, "width": WIDTH,
                       "layers": LAYERS, "matmul_mode": "3xTF32 (tcgen05)" if _C.get_matmul_mode() == 1 else "fp32",
                       "parallelism": f"dp{world}", "l2": "inputs larger than L2 (weights 537 MB, activations 268 MB each)",
                       # cross-world parity: the global-batch loss of the first 5 steps from the seed-0 state and
                       # the fp64 sum (and sum of magnitudes) of the first layer's weights after them; they agree
                       # between N = 1, 2, 4, 8 up to the summation order of the gradient exchange (rel 1e-5)
                       "global_loss": global_loss, "w0_checksum_after_5_steps": w0_checksum,
                       "w0_abs_checksum_after_5_steps": w0_abs_checksum,
                       "rank0_local_loss_after_timed_steps": last_loss,
                       "step_issue": "one CUDA-graph replay per step" if use_graph else "eager launches",
                       "ms_per_step_eager": ms_eager / args.steps, "ms_per_step_graph": ms_graph / args.steps,
                       "value_eager": samples / (ms_eager / 1e3), "value_graph": samples / (ms_graph / 1e3),
                       "ms_per_step_graph_without_exchange": ms_no_exchange,
                       "exchange_cost_ms_per_step": (ms_graph / args.steps - ms_no_exchange) if ms_no_exchange else None,
                       "kernels_per_step": launches // args.steps, "graph_replays_timed": graph_launches},
            "e2e": {"value": e2e_value, "unit": "samples/s", "h2d_bytes_per_step": 2 * nbytes * world,
                    "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches,
            "clocks": sampler.summary(*clock_window),
            "roofline": {
                "kernel": "gemm_3xtf32 (tcgen05.mma kind::tf32; fp32 product = 3 TF32 products)",
                "bound": "tensor", "unit": "TFLOP/s",
                # algorithmic work 2*M*N*K per launch over the average launch time, against the TF32 rate
                # cuBLAS sustains on this GPU; a 3xTF32 product issues three tensor-core products per
                # multiply-add, so 1/3 is the ceiling of this fraction
                "achieved": achieved, "peak": tf32_peak, "frac": (achieved / tf32_peak) if achieved else None,
                "frac_ceiling_3_products": 1.0 / 3.0,
                "tensor_pipe": {"achieved": 3 * achieved if achieved else None, "peak": tf32_peak,
                                "frac": (3 * achieved / tf32_peak) if achieved else None,
                                "what": "TF32 tensor FLOP/s actually issued (3 per algorithmic one) over the same peak"},
                "peak_source": f"{peaks['gemm_peaks_source']}: cuBLAS TF32 8192^3 sustained {peaks['tf32_tflops_sustained']:.0f}, "
                               f"burst {peaks['tf32_tflops']:.0f}; cross-check bf16/2 from MEASURED_PEAKS.json "
                               f"({peaks['source']}) = {peaks['bf16_tflops_sustained'] / 2:.0f} sustained / "
                               f"{peaks['bf16_tflops'] / 2:.0f} burst; cuBLAS SGEMM (no tensor cores) {peaks['fp32_tflops']:.0f}",
                "launches": gemm_launches, "avg_launch_ms": avg_ms,
                "flops_per_launch": flops_per_launch,
                # DRAM bytes of one launch, from the ncu capture of the step's two GEMM shapes at the full
                # per-GPU batch, weighted 15 : 8 as in one step; none for other shapes (re-reads do not scale)
                "traffic": GEMM_TRAFFIC_BYTES_PER_LAUNCH if full else None,
                "traffic_unit": "bytes/launch (dram__bytes_read.sum + dram__bytes_write.sum)",
                "traffic_source": GEMM_TRAFFIC_SOURCE if full else None,
                "algorithmic_bytes_per_launch": GEMM_ALGORITHMIC_BYTES_PER_LAUNCH if full else None,
            },
        }
        if world == 1 and not args.no_ops:
            ops = time_ops(nt, peaks)
            line["roofline"]["per_op"] = compact_ops(ops)
            line["roofline"]["hbm_peak_gbs"] = peaks["hbm_gbs"]
            line["cpu_baseline"] = cpu_baseline_sample()
            if not args.no_ref_cuda:
                line["roofline"]["reference_cuda_kernels_on_this_gpu"] = reference_cuda_column()
            if args.ops_detail:
                Path(args.ops_detail).write_text(json.dumps(ops, indent=1))
        print(json.dumps(line), flush=True)
    barrier()
    # graphs that captured collectives go before the communicator they use
    if graphs is not None:
        for g, _ in graphs:
            g.close()
    opt.detach()
    comm.close()
    sampler.__exit__(None, None, None)
    if dist is not None:
        dist.destroy_process_group()


# (15 * 2882.6 MB + 8 * 3027.4 MB) / 23: forward / input-gradient shape and weight-gradient shape of the step
GEMM_TRAFFIC_BYTES_PER_LAUNCH = 2.422e9
GEMM_TRAFFIC_SOURCE = "profiles/gemm_3xtf32_step_shapes_dram_traffic.md (ncu, third capture: one launch per shape)"
# fp32 operands read once, hi/lo planes written and read once, output written once, same 15 : 8 weighting
GEMM_ALGORITHMIC_BYTES_PER_LAUNCH = (15 * 939.5e6 + 8 * 1140.9e6) / 23

PROFILE_CASES = ("gemm4096", "add4096", "add4096_transposed", "pow2_4096_transposed", "add4096_broadcast", "tanh4096", "tanh4096_exact", "exp4096",
                 "sigmoid4096", "sum8192_dim0", "sum8192_dim1", "sum8192_full", "max_backward8192", "gather8192_rows", "gemm_step_shapes",
                 "sgemm4096", "max_backward8192_dim0", "sum_short_rows", "sgd4096", "cast4096", "scatter8192_ordered", "add_sliced_3d",
                 "mean8192_dim1", "mlp_step_16384", "mlp_step_2048", "mul_backward4096")


def profile_case(name: str, launches: int = 3) -> None:
    """One small, fixed case for an `ncu` capture: a warm-up launch, then `launches` launches of one op
    on inputs larger than L2 (at most ~0.5 GB on the device), then exit."""
    import nanotorch_b200 as nt

    _C = nt._C
    r = np.random.default_rng
    dev = lambda a: nt.Tensor.from_numpy(a.astype(np.float32), "cuda")  # noqa: E731
    if name == "gemm4096":
        a, b = dev(r(30).uniform(-1, 1, (4096, 4096))), dev(r(31).uniform(-1, 1, (4096, 4096)))
        fn = lambda: _C.matmul(a._C_view, b._C_view)  # noqa: E731
    elif name == "gemm_step_shapes":
        # the two GEMM shapes of the benchmark's training step: activation @ weight (forward and input
        # gradient, 16384 x 4096 x 4096) and activation^T @ gradient (weight gradient, 4096 x 4096 x 16384)
        x, w = dev(r(40).standard_normal((16384, 4096))), dev(r(31).uniform(-0.04, 0.04, (4096, 4096)))
        g = dev(r(32).standard_normal((16384, 4096)))
        launches = 1

        def fn():
            return _C.matmul(x._C_view, w._C_view), _C.matmul(x.T._C_view, g._C_view)
    elif name.startswith("add4096"):
        a, b = dev(r(10).uniform(-1, 1, (4096, 4096))), dev(r(11).uniform(-1, 1, (4096, 4096)))
        v = dev(r(13).uniform(-1, 1, (4096,)))
        other = {"add4096": b, "add4096_transposed": b.T, "add4096_broadcast": v.expand(4096, 4096)}[name]
        fn = lambda: _C.add(a._C_view, other._C_view)  # noqa: E731
    elif name == "pow2_4096_transposed":
        a = dev(r(10).uniform(-1, 1, (4096, 4096)))
        fn = lambda: _C.pow(a.T._C_view, 2.0)  # noqa: E731
    elif name == "max_backward8192":
        x = dev(r(20).standard_normal((8192, 8192)))
        m = x.max((1,)).reshape(8192, 1).expand(8192, 8192)
        g = dev(np.ones((8192,))).reshape(8192, 1).expand(8192, 8192)
        fn = lambda: _C.extremum_backward(g._C_view, x._C_view, m._C_view, [1])  # noqa: E731
    elif name in ("tanh4096", "tanh4096_exact", "exp4096", "sigmoid4096"):
        x = dev(r(14).standard_normal((4096, 4096)))
        if name == "tanh4096_exact":
            _C.set_tanh_mode(_C.TANH_BIT_EXACT_LIBM)
        kern = {"tanh4096": _C.tanh, "tanh4096_exact": _C.tanh, "exp4096": _C.exp, "sigmoid4096": _C.sigmoid}[name]
        fn = lambda: kern(x._C_view)  # noqa: E731
    elif name == "gather8192_rows":
        x = dev(r(20).standard_normal((8192, 8192)))
        perm = nt.Tensor.from_numpy(r(22).permutation(8192).astype(np.int64), "cuda")
        fn = lambda: _C.gather_from_axes(  # noqa: E731
            x=x._C_view, new_shape=[8192, 8192], fancy_dims_in_src=[0], fancy_dims_data=[perm._C_view],
            out_axis_is_fancy=[True, False], out_axis_target=[0, 1], checked=True)
    elif name in ("mlp_step_16384", "mlp_step_2048"):
        # the benchmark's training step at the 1-GPU batch and at the per-rank batch of the 8-GPU run
        # (one rank, no collective): two warm-up steps, then `launches` steps for the profiler's launch list
        import nanotorch_b200.nn as nn
        from nanotorch_b200.dp import Communicator, DataParallelSGD

        rows = int(name.rsplit("_", 1)[1])
        model = build_model(nt, nn)
        opt = DataParallelSGD(model.parameters(), LR, Communicator(0, 1, None))
        X, Y = dev(r(40).standard_normal((rows, WIDTH))), dev(r(41).standard_normal((rows, WIDTH)))
        launches = 1

        def fn():
            loss = nt.mean((model(X) - Y) ** 2)
            opt.zero_grad()
            loss.backward()
            opt.step()
            return loss

        fn()
    elif name == "sgemm4096":  # the exact-FP32 SIMT kernel (matmul mode 0)
        a, b = dev(r(30).uniform(-1, 1, (4096, 4096))), dev(r(31).uniform(-1, 1, (4096, 4096)))
        _C.set_matmul_mode(0)
        launches = 2
        fn = lambda: _C.matmul(a._C_view, b._C_view)  # noqa: E731
    elif name == "max_backward8192_dim0":  # two launches over x: extremum_count_*, extremum_apply*
        x = dev(r(20).standard_normal((8192, 8192)))
        m = x.max((0,)).reshape(1, 8192).expand(8192, 8192)
        g = dev(np.ones((8192,))).reshape(1, 8192).expand(8192, 8192)
        fn = lambda: _C.extremum_backward(g._C_view, x._C_view, m._C_view, [0])  # noqa: E731
    elif name == "sum_short_rows":  # one warp per row (reduce_rows_warp)
        x = dev(r(20).standard_normal((262144, 256)))
        fn = lambda: _C.sum(x._C_view, [1], nt.float32)  # noqa: E731
    elif name == "mean8192_dim1":  # the sum kernel with the division in its finish
        x = dev(r(20).standard_normal((8192, 8192)))
        fn = lambda: _C.mean_f32(x._C_view, [1], 8192)  # noqa: E731
    elif name == "mul_backward4096":  # both gradients of a product in one launch (ew_contig_two)
        a, b = dev(r(10).uniform(-1, 1, (4096, 4096))), dev(r(11).uniform(-1, 1, (4096, 4096)))
        g = dev(r(16).standard_normal((4096, 4096)))
        fn = lambda: _C.mul_backward(g._C_view, a._C_view, b._C_view)  # noqa: E731
    elif name == "sgd4096":
        p_, g_ = dev(r(31).uniform(-0.04, 0.04, (4096, 4096))), dev(r(32).standard_normal((4096, 4096)))
        fn = lambda: _C.sgd_update(p_._C_view, g_._C_view, 1e-3, 0.125)  # noqa: E731
    elif name == "cast4096":
        x = dev(r(14).standard_normal((4096, 4096)) * 100)
        fn = lambda: _C.cast(x.storage, nt.int32)  # noqa: E731
    elif name == "scatter8192_ordered":
        x = dev(r(20).standard_normal((8192, 8192)))
        tgt = x.clone()
        perm = nt.Tensor.from_numpy(r(22).permutation(8192).astype(np.int64), "cuda")
        fn = lambda: _C.scatter_to_axes(  # noqa: E731
            src=x._C_view, out=tgt._C_view, fancy_dims_in_src=[0], fancy_dims_data=[perm._C_view],
            out_axis_is_fancy=[True, False], out_axis_target=[0, 1], checked=True, unique=False)
    elif name == "add_sliced_3d":  # a view that does not collapse: the general index-math path of ew_strided
        a = dev(r(10).uniform(-1, 1, (64, 520, 520)))
        b = dev(r(11).uniform(-1, 1, (64, 520, 520)))
        av, bv = a[:, 3:515, 1:513], b[:, 5:517, 7:519]
        fn = lambda: _C.add(av._C_view, bv._C_view)  # noqa: E731
    elif name.startswith("sum8192"):
        x = dev(r(20).standard_normal((8192, 8192)))
        axes = {"sum8192_dim0": [0], "sum8192_dim1": [1], "sum8192_full": [0, 1]}[name]
        fn = lambda: _C.sum(x._C_view, axes, nt.float32)  # noqa: E731
    else:
        raise SystemExit(f"unknown case {name}; one of {PROFILE_CASES}")
    keep = [fn()]
    for _ in range(launches):
        keep.append(fn())
    _C.cuda_sync()
    print(f"{name}: {launches + 1} launches done")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op sweep and the CPU baseline sample")
    ap.add_argument("--no-ref-cuda", action="store_true",
                    help="skip the comparison column: the reference's own CUDA kernels (oracle/_ref) on this GPU")
    ap.add_argument("--ops-detail", default=None, help="write the full per-op table (all fields) to this JSON file")
    ap.add_argument("--ref-cpu", action="store_true",
                    help="time the reference's CPU kernels on the per-op configurations (needs no GPU), print JSON, exit")
    ap.add_argument("--case", default=None, help=f"run one small case for a profiler capture and exit: {PROFILE_CASES}")
    args = ap.parse_args()
    if args.case:
        profile_case(args.case)
        return
    if args.ref_cpu:
        print(json.dumps({"impl": "reference", "ops_cpu": reference_cpu_column()}), flush=True)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    product_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
