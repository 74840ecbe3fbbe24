#!/usr/bin/env python
"""
Benchmark of the KANLinear hot path: forward + backward of sum(y^2) for one
KANLinear 1024 -> 1024 (G = 5, k = 3, fp32), batch 65536 rows, batch-sharded
over the GPUs of one node with an NCCL all-reduce of the parameter gradients.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference            # CPU arm: the reference's own backend (baseline/_ref) on the host cores
    python bench.py --impl reference-cuda       # informational: the reference's own CUDA backend on this GPU

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
# Reference arms.  They import the UNMODIFIED reference package from baseline/_ref (installed there by
# __graft_entry__.build(); git-ignored) and never this repository's package: both register the
# torch.ops namespace "spline_kan", so they cannot share a process.
# ---------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
CPU_CHUNK_ROWS = 8192


def _import_reference():
    """The reference's `spline_kan` from baseline/_ref, or None when it is not installed."""
    if not os.path.isdir(os.path.join(REF_DIR, "spline_kan")):
        return None
    if "torchsplinekan_b200" in sys.modules:
        raise RuntimeError("the reference package cannot be imported beside torchsplinekan_b200")
    sys.path.insert(0, REF_DIR)
    import spline_kan                                   # noqa: F401  (the reference, not the alias of this repo)
    assert os.path.realpath(os.path.dirname(spline_kan.__file__)).startswith(os.path.realpath(REF_DIR))
    return spline_kan


def _c1_batch(torch, rows=BATCH):
    gen = torch.Generator().manual_seed(0)
    return torch.randn(BATCH, IN_F, generator=gen).clamp_(-1, 1)[:rows].contiguous()


def cpu_reference_step(chunks: int, reps: int, warmup: int, native: bool = False):
    """Median seconds of forward + backward of sum(y^2) over `chunks` chunks of 8192 rows with
    gradient accumulation, on the host cores: the reference's KANLinear(backend="reference") (pure
    PyTorch), or with `native` its C++ CPU kernels (csrc/kan_cpu.cpp through _C.kan_apply on CPU
    tensors).  Returns (seconds, kind) -- kind "port" when baseline/_ref is absent and the PyTorch
    restatement under oracle/ is timed instead."""
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    ref = _import_reference()
    x = _c1_batch(torch, chunks * CPU_CHUNK_ROWS)
    if ref is None:
        if native:
            return None, "unavailable"
        from oracle import kan_oracle as ko
        from oracle import kan_oracle_torch as kt
        g = torch.Generator().manual_seed(0)
        grid = torch.from_numpy(ko.uniform_grid(IN_F, GRID, ORDER))
        R = GRID + ORDER
        bw = (torch.rand(OUT_F, IN_F, generator=g) * 2 - 1) / IN_F ** 0.5
        sw = (torch.rand(OUT_F, IN_F, R, generator=g) * 2 - 1) * 0.1 / R ** 0.5
        sc = torch.ones(OUT_F, IN_F)

        def step():
            for c in range(chunks):
                kt.layer_step_sum_sq(x[c * CPU_CHUNK_ROWS:(c + 1) * CPU_CHUNK_ROWS], grid, bw, sw, sc, ORDER,
                                     need_x=False)
        kind = "port"
    else:
        torch.manual_seed(0)
        layer = ref.KANLinear(IN_F, OUT_F, grid_size=GRID, spline_order=ORDER, backend="reference")
        if native:
            from spline_kan import kan_linear as ref_kl
            if not ref_kl._CUDA_EXT_LOADED:
                return None, "unavailable"
            ext = ref_kl._C

            def fwd(xc):
                return ext.kan_apply(xc, layer.grid, layer.base_weight, layer.spline_weight, layer.spline_scaler,
                                     ORDER, True)
        else:
            fwd = layer

        def step():
            for p in layer.parameters():
                p.grad = None
            for c in range(chunks):
                fwd(x[c * CPU_CHUNK_ROWS:(c + 1) * CPU_CHUNK_ROWS]).square().sum().backward()
        kind = "reference"
    times = []
    for it in range(warmup + reps):
        t0 = time.perf_counter()
        step()
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return statistics.median(times), kind


def cpu_baseline_record(chunks: int, reps: int, warmup: int):
    """`cpu_baseline` object of the bench line (run in a child process: see _import_reference)."""
    sec, kind = cpu_reference_step(chunks, reps, warmup)
    rows = chunks * CPU_CHUNK_ROWS
    what = ("the reference's KANLinear(backend='reference') on CPU tensors" if kind == "reference"
            else "PyTorch-CPU restatement of the reference backend (oracle/kan_oracle_torch.py; baseline/_ref absent)")
    rec = {"value": rows / sec, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": kind,
           "sample": f"{chunks} chunk(s) of {CPU_CHUNK_ROWS} rows of the {BATCH}-row batch per step with gradient "
                     f"accumulation, {what}, torch.set_num_threads({os.cpu_count()}), median of {reps} after "
                     f"{warmup} warm-up"}
    if kind == "reference":
        sec2, kind2 = cpu_reference_step(1, max(1, min(reps, 2)), 1, native=True)
        if sec2 is not None:
            rec["kan_cpu_cpp"] = {"value": CPU_CHUNK_ROWS / sec2, "unit": "samples/s",
                                  "sample": f"1 chunk of {CPU_CHUNK_ROWS} rows, the reference's C++ CPU kernels "
                                            "(csrc/kan_cpu.cpp via _C.kan_apply on CPU tensors)"}
    return rec, sec * (BATCH / rows)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
    rec, sec_full = cpu_baseline_record(args.cpu_chunks, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": rec["value"], "unit": "samples/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec_full * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "KANLinear 1024->1024 G=5 k=3 fp32, fwd+bwd of sum(y^2), x without grad",
                   "global_batch": BATCH},
        "cpu_baseline": rec,
        "e2e": {"value": rec["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_reference_cuda_arm(args):
    """Informational: the reference's OWN CUDA backend (csrc/kan_cuda.cu: SIMT basis kernels + cuBLAS;
    csrc/kan_reg_cuda.cu) rebuilt for sm_100 in baseline/_ref, timed on this GPU at the benchmark's
    configuration with TF32 matmul off (its published setting) and on, plus its fused regulariser on
    the first layer of the 784-256-256-10 network."""
    import torch
    ref = _import_reference()
    out = {"impl": "reference-cuda"}
    if ref is None:
        out["unavailable"] = "baseline/_ref is not installed"
        print(json.dumps(out), flush=True)
        return
    from spline_kan import kan_linear as ref_kl
    if not (ref_kl._CUDA_EXT_LOADED and torch.cuda.is_available()):
        out["unavailable"] = "the reference's extension did not load or there is no GPU"
        print(json.dumps(out), flush=True)
        return
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    layer = ref.KANLinear(IN_F, OUT_F, grid_size=GRID, spline_order=ORDER, backend="cuda").to(dev)
    x = _c1_batch(torch).to(dev)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts)

    def step():
        for p in layer.parameters():
            p.grad = None
        layer(x).square().sum().backward()

    for tf32 in (False, True):
        torch.backends.cuda.matmul.allow_tf32 = tf32
        torch.backends.cudnn.allow_tf32 = tf32
        ms = timed(step, max(3, min(args.steps, 10)))
        out["c1_tf32_on" if tf32 else "c1_tf32_off"] = {"ms_per_step": ms, "samples_per_s": BATCH / ms * 1e3}
    torch.backends.cuda.matmul.allow_tf32 = False
    assert layer.last_backend == "cuda"
    # fused regulariser, first layer of KAN[784,256,256,10], 8192 rows
    torch.manual_seed(0)
    l0 = ref.KANLinear(784, 256, grid_size=GRID, spline_order=ORDER, backend="cuda").to(dev)
    x2 = (torch.rand(8192, 784, generator=torch.Generator().manual_seed(0)) * 2 - 1).to(dev)

    def reg_step():
        for p in l0.parameters():
            p.grad = None
        y, r = l0.forward_with_regularization(x2, 1e-2, 1e-2, reg_impl="fused")
        (y.square().mean() + r).backward()
    ms = timed(reg_step, max(3, min(args.steps, 10)))
    out["c2_layer0_fwr_fused"] = {"ms_per_step": ms, "rows": 8192}
    out["gpu"] = torch.cuda.get_device_name(0)
    print(json.dumps(out), flush=True)


def _child_json(argv, timeout):
    """Runs this script with `argv` in a child process and returns the last JSON line it printed."""
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__)] + argv, capture_output=True, text=True,
                           timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"timed out after {timeout} s"}
    for row in reversed(r.stdout.splitlines()):
        row = row.strip()
        if row.startswith("{"):
            try:
                return json.loads(row)
            except ValueError:
                continue
    return {"unavailable": f"exit code {r.returncode}: {r.stderr.strip()[-300:]}"}


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


def multi_gpu_grad_check(torch, dist, layer, x, bucket, step, world):
    """One extra step after the timed region: the bucket's all-reduced gradients against a plain NCCL
    all-reduce of this rank's shard gradients (recomputed through autograd outside the bucket), and
    whether every rank holds the same bits."""
    from torchsplinekan_b200 import _C
    step()
    torch.cuda.synchronize()
    reduced = torch.cat([b.detach().clone().flatten() for b in bucket.buckets])
    params = [p for _, ps in bucket._buckets for p in ps]
    with _C.no_grad_sinks():
        grads = torch.autograd.grad(layer(x.detach()).square().sum(), params)
    local = torch.cat([g.flatten() for g in grads])
    dist.all_reduce(local, op=dist.ReduceOp.SUM)
    den = float(local.abs().max())
    max_rel = float((reduced - local).abs().max()) / max(den, 1e-30)
    words = reduced.view(torch.int32).to(torch.int64)
    weights = torch.arange(1, words.numel() + 1, device=words.device) % 65521
    checksum = torch.stack([words.sum(), (words * weights).sum()])
    gathered = [torch.empty_like(checksum) for _ in range(world)]
    dist.all_gather(gathered, checksum)
    identical = all(bool((g == gathered[0]).all()) for g in gathered)
    return {"max_rel": max_rel, "ranks_bit_identical": identical, "ok": bool(max_rel < 1e-5 and identical),
            "note": "bucket after the timed path's all-reduce vs NCCL all-reduce of the shard gradients recomputed "
                    "outside the bucket; tolerance 1e-5 of max|gradient|; bit identity by checksums of the raw words"}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    import torchsplinekan_b200 as sk
    from torchsplinekan_b200 import _C

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
    # Timing hygiene: the input of a timed step must not sit in L2 (126 MB) from the step before.  A
    # rank's shard of x is 268 MB at one GPU; from four GPUs on it is smaller than L2, so the timed
    # steps then rotate over enough device copies of the shard to exceed 160 MB.
    x_bytes = rows * IN_F * 4
    n_rot = 1 if x_bytes >= 160e6 else int(math.ceil(160e6 / max(x_bytes, 1)))
    x_rot = [x_dev] + [x_dev.detach().clone().requires_grad_(args.need_x) for _ in range(n_rot - 1)]
    rot_state = {"k": 0}
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
        xin = x_rot[rot_state["k"] % n_rot]
        rot_state["k"] += 1
        xin.grad = None
        y = layer(xin)
        loss = SumSquares.apply(y)
        loss.backward()
        if bucket is not None:
            bucket.finish()
        return loss

    # End to end: every step copies one batch from pinned host memory (the next step's, on a side
    # stream while this step computes) and copies its loss to pinned host memory.  The host reads the
    # loss of step t only after it has queued step t+2 (three pinned slots), so it is always at least
    # one full step ahead of the GPU and the device never waits for the host.
    prefetch = sk.HostBatchPrefetcher(x_host.shape, x_host.dtype, dev)
    prefetch.submit(x_host)
    LAG = 2
    loss_host = [torch.zeros(1).pin_memory() for _ in range(LAG + 1)]
    loss_ready = [None] * (LAG + 1)
    e2e_state = {"k": 0, "last": None}

    def read_loss(slot):
        if loss_ready[slot] is not None:
            loss_ready[slot].synchronize()
            loss_ready[slot] = None
            e2e_state["last"] = float(loss_host[slot][0])

    def step_e2e():
        k = e2e_state["k"]
        e2e_state["k"] = k + 1
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
        slot = k % (LAG + 1)
        loss_host[slot].copy_(loss.detach().reshape(1), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
        loss_ready[slot] = ev
        read_loss((k + 1) % (LAG + 1))                # the slot step k+1 will write: result of step k-LAG

    def flush_e2e():
        k = e2e_state["k"]
        for j in range(LAG + 1):
            read_loss((k + 1 + j) % (LAG + 1))        # oldest first

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
    _C.take_event_log()
    _C.set_event_log(True)
    ms_total = timed(step_resident, args.steps)
    _C.set_event_log(False)
    log = _C.take_event_log()
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

    # the same resident step with single bf16 operands (one MMA per product instead of three): a
    # second, lower-precision data point beside the headline
    x1_line = None
    if world == 1 and not args.mode:
        with torch.no_grad():
            y3 = layer(x_dev)
        prev_mode = _C.get_mma_mode()
        _C.set_mma_mode("bf16x1")
        try:
            for _ in range(3):
                step_resident()
            n1 = min(args.steps, 10)
            ms1 = timed(step_resident, n1) / n1
            with torch.no_grad():
                y1 = layer(x_dev)
            x1_line = {"value": args.batch / (ms1 * 1e-3), "unit": "samples/s", "ms_per_step": ms1,
                       "stated_tolerance": 1e-2,
                       "max_error_vs_bf16x3_rel_to_max": float((y1 - y3).abs().max() / y3.abs().max())}
        finally:
            _C.set_mma_mode(prev_mode)

    _C.check_status()
    if bucket is not None:
        bucket.check()
    grad_check = multi_gpu_grad_check(torch, dist, layer, x_dev, bucket, step_resident, world) if world > 1 else None

    per = {}
    for name, ms in log:
        per.setdefault(name, []).append(ms)
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
                       "l2": (f"inputs larger than L2: x and dY are {x_bytes / 1e6:.0f} MB each per rank" if n_rot == 1 else
                              f"inputs larger than L2: the timed steps rotate over {n_rot} device copies of the rank's "
                              f"{x_bytes / 1e6:.0f} MB shard of x ({n_rot * x_bytes / 1e6:.0f} MB)"),
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
        line["config"]["loss"] = ("sum(y^2) as one fused autograd function (one reduction pass forward, dY = 2 g y "
                                  "backward) instead of the four elementwise passes of y.square().sum(); same maths")
        if grad_check is not None:
            line["grad_check"] = grad_check
        if x1_line is not None:
            line["bf16x1"] = x1_line
        if world == 1 and not args.no_cpu_baseline:
            # the reference itself, in child processes (it cannot be imported beside this package)
            child = _child_json(["--impl", "reference", "--steps", "2", "--warmup", "1",
                                 "--cpu-chunks", str(args.cpu_chunks)], timeout=900)
            line["cpu_baseline"] = child.get("cpu_baseline") or {"unavailable": child.get("unavailable", "no output")}
            line["reference_cuda"] = _child_json(["--impl", "reference-cuda", "--steps", "5"], timeout=600)
        print(json.dumps(line), flush=True)
    if grad_check is not None and not grad_check["ok"]:
        if world > 1:
            dist.destroy_process_group()
        raise SystemExit("bench.py: the all-reduced gradients differ from the sum of the shard gradients")
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
            pk = extra.pop("fma_peak_tflops", None)
            if pk:
                line.update(fma_peak_tflops=pk, frac_of_fma_peak=flops / ms / 1e9 / pk)
        line.update(extra)
        print(json.dumps(line), flush=True)

    # FMA-pipe peaks (register-only loop of 16 independent chains per thread, 148 * 8 blocks of 256)
    import ctypes
    from torchsplinekan_b200.build import SELFTEST_PATH
    st_lib = ctypes.CDLL(SELFTEST_PATH)
    st_lib.kanb200_selftest_fma_loop.restype = ctypes.c_int
    st_lib.kanb200_selftest_fma_loop.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    fma_peak = {}
    for code, name, dt, iters in ((0, "fp32", torch.float32, 1 << 16), (1, "fp64", torch.float64, 1 << 15)):
        blocks = 148 * 8
        buf = torch.empty(blocks * 256, dtype=dt, device=dev)
        run = lambda: st_lib.kanb200_selftest_fma_loop(code, blocks, iters, ctypes.c_void_p(buf.data_ptr()),
                                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        ms = timeit(run, reps=5)
        fma_peak[name] = 2.0 * blocks * 256 * iters * 16 / ms / 1e9          # TFLOP/s
        print(json.dumps({"kernel": f"fma_loop<{name}>", "ms": ms, "tflops": fma_peak[name],
                          "note": "measured FMA-pipe peak (register-only loop)"}), flush=True)

    # FP64 matrix-instruction peak (mma.sync f64; 8 independent accumulator tiles per warp)
    st_lib.kanb200_selftest_dmma_loop.restype = ctypes.c_int
    st_lib.kanb200_selftest_dmma_loop.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    for shape, name, per in ((0, "m8n8k4", 256), (1, "m16n8k8", 1024)):
        blocks, iters = 148 * 8, 1 << 13
        buf = torch.empty(blocks * 256, dtype=torch.float64, device=dev)
        run = lambda: st_lib.kanb200_selftest_dmma_loop(shape, blocks, iters, ctypes.c_void_p(buf.data_ptr()),
                                                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        ms = timeit(run, reps=5)
        fma_peak["dmma_" + name] = 2.0 * blocks * 8 * iters * 8 * per / ms / 1e9
        print(json.dumps({"kernel": f"dmma_loop<{name}>", "ms": ms, "tflops": fma_peak["dmma_" + name],
                          "note": "measured FP64 matrix-instruction peak (register-only loop)"}), flush=True)

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
    emit("edge_param_kernel<forward>", ms, flops=fl, fma_peak_tflops=fma_peak["fp32"])
    ms = timeit(lambda: nat.edge_abs_mean_backward(ga, s, H, bw, W, False, False, True, True))
    emit("edge_param_kernel<grad> + sum_slabs", ms, flops=2 * fl, fma_peak_tflops=fma_peak["fp32"])
    ms = timeit(lambda: nat.edge_abs_mean_backward(ga, s, H, bw, W, True, True, False, False))
    emit("edge_input_kernel", ms, flops=2 * fl, fma_peak_tflops=fma_peak["fp32"])
    del H

    # the same statistic straight from x (basis never stored), on the tensor cores and on the FMA pipes
    xe = torch.rand(Ne, Ie, device=dev, generator=g) * 2 - 1
    ge = ((torch.arange(G + 2 * k + 1, device=dev, dtype=torch.float32) - k) * (2.0 / G) - 1.0)[None] \
        .expand(Ie, -1).contiguous()
    ms = timeit(lambda: nat.edge_abs_mean_x(xe, None, ge, bw, W, k, nat.MODE_TC_BF16X3))
    emit("tc_edge_fwd_kernel (from x, tensor cores)", ms, flops=fl, note="2 N O I (R+1) flops counted once; 3 bf16 MMAs per product",
         tflops_counted_once=fl / ms / 1e9)
    ms = timeit(lambda: nat.edge_abs_mean_x(xe, None, ge, bw, W, k, nat.MODE_SIMT))
    emit("edge_param_kernel<forward, from x>", ms, flops=fl, fma_peak_tflops=fma_peak["fp32"])
    simt = nat.MODE_SIMT
    ms = timeit(lambda: nat.edge_abs_mean_x_backward(ga, xe, None, ge, bw, W, k, False, False, True, True, mode=simt))
    emit("edge_param_kernel<grad, from x> + sum_slabs", ms, flops=2 * fl, fma_peak_tflops=fma_peak["fp32"])
    ms = timeit(lambda: nat.edge_abs_mean_x_backward(ga, xe, None, ge, bw, W, k, True, False, False, False, mode=simt))
    emit("edge_input_kernel<from x>", ms, flops=2 * fl, fma_peak_tflops=fma_peak["fp32"])
    tc = nat.MODE_TC_BF16X3
    ms = timeit(lambda: nat.edge_abs_mean_x_backward(ga, xe, None, ge, bw, W, k, False, False, True, True, mode=tc))
    emit("tc_edge_bwd_kernel (parameter gradients, tensor cores)", ms, flops=2 * fl,
         note="phi + sign(phi)^T A: 4 N O I (R+1) flops counted once", tflops_counted_once=2 * fl / ms / 1e9)
    ms = timeit(lambda: nat.edge_abs_mean_x_backward(ga, xe, None, ge, bw, W, k, True, False, True, True, mode=tc))
    emit("tc_edge_bwd_kernel (parameter + input gradients, tensor cores)", ms, flops=3 * fl,
         note="6 N O I (R+1) flops counted once", tflops_counted_once=3 * fl / ms / 1e9)
    del s, W, xe

    # MMA issue cost: cycles per tcgen05.mma (K = 16) for one issuing thread, by accumulator width
    st_lib.kanb200_selftest_umma_rate.restype = ctypes.c_int
    st_lib.kanb200_selftest_umma_rate.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 3
    cyc = torch.zeros(4, dtype=torch.int64, device=dev)
    stat = torch.zeros(1, dtype=torch.int32, device=dev)
    for n_cols in (16, 32, 128, 256):
        for threads in (1, 2):
            for _ in range(2):
                st_lib.kanb200_selftest_umma_rate(n_cols, 512, threads, 1, ctypes.c_void_p(cyc.data_ptr()),
                                                  ctypes.c_void_p(stat.data_ptr()), None)
                torch.cuda.synchronize()
            print(json.dumps({"kernel": f"umma_rate<N={n_cols}, issuing threads={threads}>",
                              "cycles_per_mma_per_thread": cyc[1].item() / 512.0,
                              "note": "M = 128, K = 16, bf16; 512 instructions per thread, until completion"}),
                  flush=True)

    # float64 layers of the PINN-style network on the FP64 matrix instruction (131072 rows, G = 8)
    Nd, Gd = 131072, 8
    for Id, Od in ((2, 64), (64, 64), (64, 1)):
        xd = torch.rand(Nd, Id, device=dev, dtype=torch.float64, generator=g) * 2 - 1
        gd = ((torch.arange(Gd + 2 * k + 1, device=dev, dtype=torch.float64) - k) * (2.0 / Gd) - 1.0)[None] \
            .expand(Id, -1).contiguous()
        bwd_ = torch.randn(Od, Id, device=dev, dtype=torch.float64, generator=g)
        swd = torch.randn(Od, Id, Gd + k, device=dev, dtype=torch.float64, generator=g)
        scd = torch.randn(Od, Id, device=dev, dtype=torch.float64, generator=g)
        D = torch.randn(Nd, Od, device=dev, dtype=torch.float64, generator=g)
        dense = 2.0 * Nd * Od * Id * (Gd + k + 1)
        pk = fma_peak["dmma_m8n8k4"]
        ms = timeit(lambda: nat.forward(xd, gd, bwd_, swd, scd, k, nat.MODE_SIMT))
        emit(f"dm_forward_kernel<double> {Id}->{Od}", ms, flops=dense, fma_peak_tflops=pk,
             note="dense flops 2 N O I (R+1) against the measured FP64 matrix-instruction peak")
        ms = timeit(lambda: nat.backward(D, xd, gd, bwd_, swd, scd, k, False, True, True, True, nat.MODE_SIMT))
        emit(f"dm_bwd_param_kernel<double> {Id}->{Od}", ms, flops=dense, fma_peak_tflops=pk)
        ms = timeit(lambda: nat.backward(D, xd, gd, bwd_, swd, scd, k, True, False, False, False, nat.MODE_SIMT))
        emit(f"dm_bwd_input_kernel<double> {Id}->{Od}", ms, flops=dense, fma_peak_tflops=pk)


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
        name, rows = "c4 KAN[2,64,64,1] G=8 N=131072 fp64 PINN loss (FP64 matrix-instruction kernels)", 131072
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
    ms_synced = statistics.median(times)
    # the same steps back to back, as a training loop issues them (no host synchronisation between steps):
    # for the small configurations the host's launch work of step t+1 then overlaps the kernels of step t
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        run()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    print(json.dumps({"config": name, "ms_per_step": ms, "ms_per_step_synchronised": ms_synced,
                      "samples_per_s": rows / ms * 1e3, "steps": args.steps,
                      "backends": [getattr(l, "last_backend", None) for l in getattr(net, "layers", [net])]}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "reference-cuda"])
    ap.add_argument("--cpu-chunks", type=int, default=8,
                    help="chunks of 8192 rows per step of the CPU reference arm (8 = the whole 65536-row batch)")
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
    elif args.impl == "reference-cuda":
        run_reference_cuda_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
