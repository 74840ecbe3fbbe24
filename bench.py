#!/usr/bin/env python
"""
Benchmark of the KANLinear hot path: forward + backward of sum(y^2) for one
KANLinear 1024 -> 1024 (G = 5, k = 3, fp32), batch 65536 rows, batch-sharded
over the GPUs of one node with an NCCL all-reduce of the parameter gradients.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference            # CPU arm: numpy port of the reference backend

Prints ONE JSON line (rank 0).  `value` = samples/s with inputs resident in
HBM; `e2e` = the same step through the public module API with the inputs
copied from pinned host memory and the loss read back, every step.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

IN_F, OUT_F, GRID, ORDER, BATCH = 1024, 1024, 5, 3, 65536
CPU_SAMPLE_ROWS = 4096
METRIC = "KANLinear fwd+bwd samples/s (1024->1024, G=5, k=3, fp32)"


def algorithmic_flops(rows: int, need_x: bool = False) -> float:
    """2 N O I (R+1) per pass; forward + parameter backward (+ input backward)."""
    per_pass = 2.0 * rows * OUT_F * IN_F * (GRID + ORDER + 1)
    return per_pass * (3 if need_x else 2)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops_sustained"]), float(d["hbm_gbs"]), "measured"
    return 1400.0, 6650.0, "fallback"


# ---------------------------------------------------------------------------
# CPU arm: the numpy oracle (a port of the reference's pure-PyTorch backend)
# ---------------------------------------------------------------------------
def cpu_step(rows: int, reps: int, warmup: int):
    """Median seconds of one forward + backward of sum(y^2) on `rows` rows, on the host cores, with
    the multi-threaded PyTorch restatement of the reference's CPU path (oracle/kan_oracle_torch.py)."""
    import torch
    from oracle import kan_oracle as ko
    from oracle import kan_oracle_torch as kt
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, IN_F, generator=g).clamp_(-1, 1)
    grid = torch.from_numpy(ko.uniform_grid(IN_F, GRID, ORDER))
    R = GRID + ORDER
    bw = (torch.rand(OUT_F, IN_F, generator=g) * 2 - 1) / IN_F ** 0.5
    sw = (torch.rand(OUT_F, IN_F, R, generator=g) * 2 - 1) * 0.1 / R ** 0.5
    sc = torch.ones(OUT_F, IN_F)
    times = []
    for it in range(warmup + reps):
        t0 = time.perf_counter()
        kt.layer_step_sum_sq(x, grid, bw, sw, sc, ORDER, need_x=False)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return statistics.median(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    sec = cpu_step(CPU_SAMPLE_ROWS, steps, warmup)
    val = CPU_SAMPLE_ROWS / sec
    cores = os.cpu_count() or 1
    sample = f"{CPU_SAMPLE_ROWS} rows of the {BATCH}-row batch per step, PyTorch-CPU restatement of the reference backend (oracle/kan_oracle_torch.py), median of {steps}"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "KANLinear 1024->1024 G=5 k=3 fp32, fwd+bwd of sum(y^2), x without grad",
                   "global_batch": BATCH},
        "cpu_baseline": {"value": val, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.file.read().splitlines():
            cols = [c.strip() for c in row.split(",")]
            if len(cols) < 9:
                continue
            try:
                sm.append(float(cols[1]))
                mx.append(float(cols[2]))
            except ValueError:
                continue
            for name, col in zip(names, cols[5:9]):
                if col.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import torchsplinekan_b200 as sk
    from torchsplinekan_b200 import _native, _C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the hot path has no CPU implementation; "
                         "use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.mode:
        _C.set_mma_mode(args.mode)

    torch.manual_seed(0)
    layer = sk.KANLinear(IN_F, OUT_F, grid_size=GRID, spline_order=ORDER, backend="cuda").to(dev)
    r0, r1 = sk.shard_rows(args.batch, world, rank)
    rows = r1 - r0
    gen = torch.Generator().manual_seed(0)
    x_host = torch.randn(args.batch, IN_F, generator=gen).clamp_(-1, 1)[r0:r1].contiguous().pin_memory()
    x_dev = x_host.to(dev)
    if args.need_x:
        x_dev.requires_grad_(True)
    bucket = sk.GradientBucket([layer], direct=True) if world > 1 else None

    class SumSquares(torch.autograd.Function):
        """sum(y^2) with one pass over y in each direction (one reduction forward, dY = 2 g y backward)
        instead of the four elementwise passes of ``y.square().sum()``."""

        @staticmethod
        def forward(ctx, y):
            ctx.save_for_backward(y)
            return torch.linalg.vector_norm(y).square()

        @staticmethod
        def backward(ctx, g):
            (y,) = ctx.saved_tensors
            return y * (2.0 * g)

    def step_resident():
        if bucket is not None:
            bucket.zero_grad()
        else:
            for p in layer.parameters():
                p.grad = None
        x_dev.grad = None
        y = layer(x_dev)
        loss = SumSquares.apply(y)
        loss.backward()
        if bucket is not None:
            bucket.finish()
        return loss

    # End to end: every step copies one batch from pinned host memory (the next step's, on a side
    # stream while this step computes) and reads the loss back.
    prefetch = sk.HostBatchPrefetcher(x_host.shape, x_host.dtype, dev)
    prefetch.submit(x_host)
    # the loss of every step is copied to pinned host memory; the host reads it one step later, so
    # that it queues the next step while the GPU still works on this one
    loss_host = [torch.zeros(1).pin_memory(), torch.zeros(1).pin_memory()]
    loss_ready = [None, None]
    e2e_state = {"k": 0, "last": None}

    def read_loss(slot):
        if loss_ready[slot] is not None:
            loss_ready[slot].synchronize()
            loss_ready[slot] = None
            e2e_state["last"] = float(loss_host[slot][0])

    def step_e2e():
        k = e2e_state["k"]
        e2e_state["k"] = k + 1
        read_loss((k + 1) % 2)                        # result of the previous step
        prefetch.submit(x_host)
        x_stage = prefetch.next()
        if args.need_x:
            x_stage = x_stage.detach().requires_grad_(True)
        if bucket is not None:
            bucket.zero_grad()
        else:
            for p in layer.parameters():
                p.grad = None
        y = layer(x_stage)
        loss = SumSquares.apply(y)
        loss.backward()
        if bucket is not None:
            bucket.finish()
        loss_host[k % 2].copy_(loss.detach().reshape(1), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
        loss_ready[k % 2] = ev

    def flush_e2e():
        read_loss(0)
        read_loss(1)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local) if rank == 0 else None          # samples every 20 ms from here on
    for _ in range(max(args.warmup, 3)):
        step_resident()
    step_e2e()
    _native.EVENT_LOG = []
    ms_total = timed(step_resident, args.steps)
    log, _native.EVENT_LOG = _native.EVENT_LOG, None
    # keep the same load running (untimed) until the clock sampler has seen about half a second
    # of it; the count is derived from the all-reduced time, so every rank does the same steps
    extra = int(min(2000, max(0, 500.0 / max(ms_total / args.steps, 1e-3) - args.steps)))
    for _ in range(extra):
        step_resident()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop() if sampler else None
    flush_e2e()
    barrier()
    e2e_start, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_start.record()
    for _ in range(args.steps):
        step_e2e()
    flush_e2e()                                                      # the last result is read inside the timed region
    e2e_end.record()
    barrier()
    ms_t = torch.tensor([e2e_start.elapsed_time(e2e_end)], device=dev)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_e2e = float(ms_t.item())
    assert e2e_state["last"] is not None and math.isfinite(e2e_state["last"])

    for buf in list(_native._ws_cache.values()):
        _native.check_status(buf)
    if bucket is not None:
        bucket.check()

    per = {}
    for name, a, b in log:
        per.setdefault(name, []).append(a.elapsed_time(b))
    kernel_ms = {k: sum(v) / len(v) for k, v in per.items()}

    # this library's kernels per step: forward = table + weight image + contraction; parameter
    # backward = table + dY image + contraction + finalize (once per range of output rows when the
    # gradients go straight into the all-reduce bucket); input gradient = weight image + contraction
    # (+ table and dY image when it is a call of its own); one all-reduce kernel per range on NVLink
    if bucket is not None and bucket._sinks:
        n_ranges = len(bucket._sinks[0].row_ranges(OUT_F))
        launches_per_step = 3 + 4 * n_ranges + (4 if args.need_x else 0)
        if bucket.transport.startswith("nvlink"):
            launches_per_step += n_ranges
    else:
        launches_per_step = 7 + (2 if args.need_x else 0)
        if bucket is not None and bucket.transport.startswith("nvlink"):
            launches_per_step += 1

    if rank == 0:
        bf16_peak, hbm_peak, peak_src = measured_peaks()
        ms_step = ms_total / args.steps
        value = args.batch / (ms_step * 1e-3)
        dom = max(kernel_ms, key=kernel_ms.get) if kernel_ms else None
        pass_flops = algorithmic_flops(rows) / 2 * (2 if (args.need_x and dom == "backward") else 1)
        achieved = pass_flops / (kernel_ms[dom] * 1e-3) / 1e12 if dom else None
        mode = _C.get_mma_mode()
        terms = 1 if mode == "bf16x1" else 3
        line = {
            "metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "KANLinear 1024->1024 G=5 k=3 fp32, fwd+bwd of sum(y^2), x "
                                   + ("with grad (input gradient computed)" if args.need_x else "without grad"),
                       "global_batch": args.batch, "rows_per_gpu": rows,
                       "parallelism": f"dp{world} batch shards + all-reduce of parameter gradients ("
                                      + ((bucket.transport + (", gradients written into the bucket by ranges of output rows, "
                                                             "all-reduce of a range overlaps the next"
                                                             if bucket._sinks else ""))
                                         if bucket is not None else "single rank") + ")",
                       "mma_mode": "bf16x3 (hi/lo split operands, fp32-level accuracy)" if terms == 3 else mode,
                       "l2": "inputs larger than L2 (x and dY are 268 MB each at 65536 rows)",
                       "e2e_pipeline": "each step copies the next step's batch from pinned host memory on a side "
                                       "stream (two device staging buffers) and copies its loss to pinned host "
                                       "memory, which the host reads one step later (the last one before the clock stops)"},
            "e2e": {"value": args.batch / (ms_e2e / args.steps * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": rows * IN_F * 4, "d2h_bytes_per_step": 4},
            "gpu_launches": launches_per_step * args.steps,
            "kernel_ms": kernel_ms,
            "roofline": {"bound": "tensor", "kernel": f"{dom} (tcgen05 contraction + operand producers)",
                         "achieved": achieved, "peak": bf16_peak, "unit": "TFLOP/s",
                         "frac": achieved / bf16_peak if achieved else None,
                         "frac_of_issued_mma": terms * achieved / bf16_peak if achieved else None,
                         "peak_source": f"bf16 sustained, of {peak_src}",
                         # DRAM bytes per launch of the dominant kernel: ncu capture at 16 384 rows
                         # (dram__bytes_read.sum + dram__bytes_write.sum), the part that grows with the
                         # rows (x and the dY image / y) scaled to this run's rows, the rest (weight
                         # image, tables, slab) kept
                         "traffic": ncu_traffic_bytes(dom, rows),
                         "note": "flops counted once: 2*N*O*I*(R+1) per pass; the split mode issues 3 bf16 MMAs "
                                 "per product, so frac is capped at 1/3"},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            sec = cpu_step(CPU_SAMPLE_ROWS, 3, 1)
            line["cpu_baseline"] = {"value": CPU_SAMPLE_ROWS / sec, "unit": "samples/s",
                                    "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": f"{CPU_SAMPLE_ROWS} rows of the batch per step, PyTorch-CPU "
                                              "restatement of the reference backend, all host threads, median of 3"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def ncu_traffic_bytes(kernel, rows):
    """DRAM traffic per launch of the two contraction kernels, from the ncu capture summarised in
    profiles/tc_kernels_rows16384_full.md: forward 145.8 MB read + 41.5 MB written, parameter
    backward 134.9 MB + 6.2 MB at 16 384 rows.  Of that, x, y and the dY image grow with the rows
    (forward 67 + 67 MB, backward 67 + 67 MB at 16 384 rows); the remainder does not."""
    if kernel not in ("forward", "backward"):
        return None
    total = {"forward": 187.3e6, "backward": 141.1e6}[kernel]
    per_16k = 134.2e6
    return per_16k * rows / 16384.0 + (total - per_16k)


def run_micro(args):
    """Times the secondary kernels of the path one by one (CUDA events, inputs larger than L2) and
    prints one JSON line per kernel: achieved GB/s against the measured HBM peak for the
    bandwidth-bound ones, achieved GFLOP/s for the FMA-bound ones.  Not the headline benchmark."""
    import torch
    from torchsplinekan_b200 import _native as nat
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    _, hbm_peak, src = measured_peaks()
    g = torch.Generator(device="cuda").manual_seed(0)

    def timeit(fn, reps=args.steps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        ev[0].record()
        for r in range(reps):
            fn()
            ev[r + 1].record()
        torch.cuda.synchronize()
        return statistics.median(ev[r].elapsed_time(ev[r + 1]) for r in range(reps))

    def emit(name, ms, bytes_=None, flops=None, **extra):
        line = {"kernel": name, "ms": ms}
        if bytes_ is not None:
            line.update(bound="hbm", achieved=bytes_ / ms / 1e6, peak=hbm_peak, unit="GB/s",
                        frac=bytes_ / ms / 1e6 / hbm_peak, peak_source=f"of {src}")
        if flops is not None:
            line.update(gflops=flops / ms / 1e6)
        line.update(extra)
        print(json.dumps(line), flush=True)

    # standalone basis / basis gradient: N x I x (R+1) elements, fp32, c1 feature count
    N, I, G, k = args.micro_rows, 1024, 5, 3
    R = G + k
    x = torch.randn(N, I, device=dev, generator=g).clamp_(-1, 1)
    grid = ((torch.arange(G + 2 * k + 1, device=dev, dtype=torch.float32) - k) * (2.0 / G) - 1.0)[None] \
        .expand(I, -1).contiguous()
    ms = timeit(lambda: nat.basis(x, grid, k))
    emit("basis_kernel<float,3>", ms, bytes_=4.0 * N * I * (R + 1), rows=N, I=I)
    gH = torch.randn(N, I, R, device=dev, generator=g)
    ms = timeit(lambda: nat.basis_grad(x, grid, k, gH))
    emit("basis_grad_kernel<float,3>", ms, bytes_=4.0 * N * I * (R + 2), rows=N, I=I)
    del gH

    # edge statistic on the first layer of the 784-256-256-10 network (8192 rows)
    Ne, Ie, Oe = 8192, 784, 256
    H = torch.rand(Ne, Ie, R, device=dev, generator=g)
    s = torch.randn(Ne, Ie, device=dev, generator=g)
    bw = torch.randn(Oe, Ie, device=dev, generator=g)
    W = torch.randn(Oe, Ie, R, device=dev, generator=g)
    ga = torch.rand(Oe, Ie, device=dev, generator=g)
    fl = 2.0 * Ne * Oe * Ie * (R + 1)
    ms = timeit(lambda: nat.edge_abs_mean(s, H, bw, W))
    emit("edge_param_kernel<forward>", ms, flops=fl, bytes_moved_GB=4e-9 * (Ne * Ie * (R + 1) + Oe * Ie * (R + 2)))
    ms = timeit(lambda: nat.edge_abs_mean_backward(ga, s, H, bw, W, False, False, True, True))
    emit("edge_param_kernel<grad> + sum_slabs", ms, flops=2 * fl)
    ms = timeit(lambda: nat.edge_abs_mean_backward(ga, s, H, bw, W, True, True, False, False))
    emit("edge_input_kernel", ms, flops=2 * fl)
    del H, s, W

    # float64 SIMT layer (PINN-style 64 -> 64, G = 8)
    Nd, Id, Od, Gd = 131072, 64, 64, 8
    xd = torch.rand(Nd, Id, device=dev, dtype=torch.float64, generator=g) * 2 - 1
    gd = ((torch.arange(Gd + 2 * k + 1, device=dev, dtype=torch.float64) - k) * (2.0 / Gd) - 1.0)[None] \
        .expand(Id, -1).contiguous()
    bwd_ = torch.randn(Od, Id, device=dev, dtype=torch.float64, generator=g)
    swd = torch.randn(Od, Id, Gd + k, device=dev, dtype=torch.float64, generator=g)
    scd = torch.randn(Od, Id, device=dev, dtype=torch.float64, generator=g)
    ms = timeit(lambda: nat.forward(xd, gd, bwd_, swd, scd, k, nat.MODE_SIMT))
    emit("fwd_simt_kernel<double,3>", ms, flops=2.0 * Nd * Od * Id * (k + 2), note="useful flops: k+2 terms per edge")
    D = torch.randn(Nd, Od, device=dev, dtype=torch.float64, generator=g)
    ms = timeit(lambda: nat.backward(D, xd, gd, bwd_, swd, scd, k, True, True, True, True, nat.MODE_SIMT))
    emit("bwd_simt (param + input)<double,3>", ms, flops=4.0 * Nd * Od * Id * (k + 2))


def run_config(args):
    """Times one training step of the other benchmark configurations (1 GPU, CUDA-event median):
    0 = KAN[16,32,8] MSE, 2 = KAN[784,256,256,10] cross-entropy + fused regulariser on update_grid
    knots, 3 = KANLinear 512->512 G=64 on update_grid knots, 4 = float64 KAN[2,64,64,1] PINN loss.
    Synthetic seeded inputs with the shapes and value distributions of those configurations."""
    import math
    import torch
    import torchsplinekan_b200 as sk
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    c = args.config
    if c == 0:
        net = sk.KAN([16, 32, 8], backend="cuda").to(dev)
        x = (torch.rand(1024, 16, generator=g) * 2 - 1).to(dev)
        tgt = torch.randn(1024, 8, generator=torch.Generator().manual_seed(1)).to(dev)
        loss_fn = lambda: torch.nn.functional.mse_loss(net(x), tgt)
        name, rows = "c0 KAN[16,32,8] N=1024 fp32, MSE", 1024
    elif c == 2:
        net = sk.KAN([784, 256, 256, 10], backend="cuda").to(dev)
        x = (torch.rand(8192, 784, generator=g) * 2 - 1).to(dev)
        labels = torch.randint(0, 10, (8192,), generator=torch.Generator().manual_seed(1)).to(dev)
        t0 = time.perf_counter()
        net.update_grid(x[:4096])
        torch.cuda.synchronize()
        upd = time.perf_counter() - t0

        def loss_fn():
            y, r = net.forward_with_regularization(x, 1e-2, 1e-2)
            return torch.nn.functional.cross_entropy(y, labels) + r
        name, rows = f"c2 KAN[784,256,256,10] N=8192 fp32, CE + fused reg, update_grid(4096 rows) took {upd:.2f} s", 8192
    elif c == 3:
        net = sk.KANLinear(512, 512, grid_size=64, backend="cuda").to(dev)
        x = torch.where(torch.rand(16384, 512, generator=g) < 0.5, -0.5, 0.5) + 0.15 * torch.randn(16384, 512, generator=g)
        x = x.clamp_(-1, 1).to(dev)
        net.update_grid(x)
        if args.need_x:
            x.requires_grad_(True)
        loss_fn = lambda: net(x).square().sum()
        name, rows = "c3 KANLinear 512->512 G=64 N=16384 fp32, update_grid knots" + \
            (", input gradient computed" if args.need_x else ""), 16384
    elif c == 4:
        net = sk.KAN([2, 64, 64, 1], grid_size=8, backend="cuda").to(dev, torch.float64)
        x = (torch.rand(131072, 2, generator=g, dtype=torch.float64) * 2 - 1).to(dev)
        ref = torch.sin(math.pi * x[:, 0]) * torch.sin(math.pi * x[:, 1])
        loss_fn = lambda: (net(x).squeeze(-1) - ref).square().mean()
        name, rows = "c4 KAN[2,64,64,1] G=8 N=131072 fp64 PINN loss (SIMT kernels)", 131072
    else:
        raise SystemExit("--config must be 0, 2, 3 or 4 (1 is the default benchmark)")

    def step():
        for p in net.parameters():
            p.grad = None
        loss_fn().backward()

    run = step
    if args.graph:
        # the whole step (forward, loss, backward) captured once and replayed: one launch per step
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run = graph.replay
        name += ", CUDA graph replay"
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    print(json.dumps({"config": name, "ms_per_step": ms, "samples_per_s": rows / ms * 1e3, "steps": args.steps,
                      "backends": [getattr(l, "last_backend", None) for l in getattr(net, "layers", [net])]}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--mode", default=None, choices=[None, "auto", "simt", "bf16x3", "bf16x1"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--need-x", action="store_true", help="also compute the input gradient (x.requires_grad)")
    ap.add_argument("--micro", action="store_true", help="time the secondary kernels instead of the training step")
    ap.add_argument("--micro-rows", type=int, default=16384)
    ap.add_argument("--config", type=int, default=None, help="time one of the other benchmark configurations")
    ap.add_argument("--graph", action="store_true", help="with --config: capture the step in a CUDA graph")
    args = ap.parse_args()
    if args.config is not None:
        run_config(args)
    elif args.micro:
        run_micro(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
