"""
Batch-sharded data parallelism for KAN layers: one process per GPU, rows of the
batch split in contiguous blocks, weights and knots replicated, and ONE
collective per layer and step -- an all-reduce (sum) of that layer's parameter
gradients, started as soon as the layer's backward has produced them so that it
overlaps the backward of the layers below.  The reference has no multi-device
code; this module is what a data-parallel user of it needs on top.

Per layer the gradients live in one flat bucket ``[d spline_weight | d spline_scaler |
d base_weight]`` and ``param.grad`` are views into it, so nothing is copied
before or after the collective.

Two transports: ``"nccl"`` (``torch.distributed.all_reduce``) and ``"nvlink"``, where the buckets
live in symmetric memory (``torch.distributed._symmetric_memory``: every rank of the node maps
every rank's allocation, plus a multicast mapping through NVSwitch where the fabric offers one)
and the reduction is this library's own kernel (``kanb200_allreduce_sum_f32``: in-switch
``multimem`` reduction, or peer loads/stores).
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def shard_rows(n_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """``[start, end)`` of the contiguous row block owned by ``rank``; blocks differ by at most one row."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    base, extra = divmod(n_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class _ScaleThenAllReduce(torch.autograd.Function):
    """``out = all_reduce_sum(weight * t)`` (weight: this rank's own scalar).  Its adjoint is
    :class:`_AllReduceThenScale` and vice versa, so derivatives of any order go through the
    collective."""

    @staticmethod
    def forward(ctx, t, weight, group):
        ctx.group = group
        ctx.save_for_backward(weight)
        out = (t * weight).contiguous()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        (weight,) = ctx.saved_tensors
        return _AllReduceThenScale.apply(g, weight, ctx.group), None, None


class _AllReduceThenScale(torch.autograd.Function):
    """``out = weight * all_reduce_sum(t)``: the adjoint of :class:`_ScaleThenAllReduce`."""

    @staticmethod
    def forward(ctx, t, weight, group):
        ctx.group = group
        ctx.save_for_backward(weight)
        out = t.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out * weight

    @staticmethod
    def backward(ctx, g):
        (weight,) = ctx.saved_tensors
        return _ScaleThenAllReduce.apply(g, weight, ctx.group), None, None


def global_edge_means(a_local: torch.Tensor, n_local_rows: int,
                      group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Per-edge mean |phi| of the GLOBAL batch from each rank's statistic of its own rows:
    ``a[o, i] = sum_r (N_r / N) a_r[o, i]`` (one all-reduce of ``[O, I]`` values; the row counts
    travel in a second, one-element all-reduce, so ragged shards are weighted correctly).

    With gradient all-reduce alone every rank evaluates the regulariser on its shard, and because
    the entropy term is not linear in ``a`` the sum of those penalties is not the penalty of the
    whole batch.  Feeding the result of this function to the penalty instead makes every rank
    evaluate the whole-batch penalty; its backward all-reduces the incoming gradient and scales it by
    ``N_r / N``, so summing (or averaging) the ranks' parameter gradients afterwards gives exactly
    the gradient of (the sum, or the average, over ranks of) the per-rank losses.  A rank that adds
    the penalty to a loss whose gradients are SUMMED over ``P`` ranks scales it by ``1 / P``."""
    count = torch.tensor([float(n_local_rows)], dtype=torch.float64, device=a_local.device)
    total = count.clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
    weight = (count / total).to(a_local.dtype)              # stays on the device: no host synchronisation
    return _ScaleThenAllReduce.apply(a_local, weight, group)


def _layer_params(layer: nn.Module) -> List[nn.Parameter]:
    seen, out = set(), []
    for p in layer.parameters():
        if p.requires_grad and id(p) not in seen:
            seen.add(id(p))
            out.append(p)
    return out


class GradientBucket:
    """Flat per-layer gradient buckets with an overlapped all-reduce.

    ``layers``: modules in forward order (each gets one bucket).  Call
    :meth:`finish` after ``loss.backward()`` and before the optimiser step.
    ``average=True`` divides by the world size (for mean-type losses); sum-type
    losses keep the plain sum.

    ``transport``: ``"nccl"``, ``"nvlink"`` (raises when symmetric memory cannot be set up) or
    ``"auto"`` (``"nvlink"`` from 8 ranks on, for float32 CUDA parameters of one device when the set-up
    succeeds, else ``"nccl"``; the environment variable ``KAN_B200_ALLREDUCE`` = ``nccl`` / ``nvlink`` /
    ``p2p`` overrides it, ``p2p`` meaning the NVLink kernel without the multicast mapping).
    Construction is collective over the group when the NVLink transport is tried.

    ``direct=True``: ``KANLinear`` layers on the tensor-core path write their parameter gradients
    straight into the bucket (no autograd accumulation, no copy) and the all-reduce starts from the
    backward itself.  With ``chunks`` > 1 the gradients are produced in that many ranges of output
    rows and the all-reduce of a range runs while the next is computed (measured on B200 for a
    1024x1024 layer: every extra range costs about 0.04 ms of launch and tail time, more than the
    0.03 ms of all-reduce it hides at 8 ranks; it pays only for larger layers).  Only
    valid when these parameters receive gradients from the layers' plain ``forward`` alone and once
    per step (no regulariser term on them, no weight sharing, no gradient accumulation over
    micro-batches): the gradients of a step overwrite the bucket.
    """

    def __init__(self, layers: Iterable[nn.Module], process_group: Optional[dist.ProcessGroup] = None,
                 average: bool = False, transport: str = "auto", direct: bool = False, chunks: int = 1) -> None:
        if transport not in ("auto", "nccl", "nvlink"):
            raise ValueError(f"transport must be 'auto', 'nccl' or 'nvlink', got {transport!r}")
        self.group = process_group
        self.average = average
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self._buckets: List[Tuple[torch.Tensor, List[nn.Parameter]]] = []
        self._pending: List[int] = []
        self._works: list = []
        self._comm_stream = None
        self._hooks = []
        self.transport = "nccl"
        self.transport_note = ""
        self._symm = None
        layers = [layer for layer in layers if _layer_params(layer)]
        per_layer = [_layer_params(layer) for layer in layers]
        self._setup_symmetric(per_layer, transport)
        self._sinks: list = []
        self._direct_done: List[bool] = []
        for li, params in enumerate(per_layer):
            ref = params[0]
            if self._symm is not None:
                flat = self._symm.flat(li)
            else:
                flat = torch.zeros(sum(p.numel() for p in params), dtype=ref.dtype, device=ref.device)
            offset = 0
            for p in params:
                p.grad = flat[offset:offset + p.numel()].view_as(p)
                offset += p.numel()
            index = len(self._buckets)
            self._buckets.append((flat, params))
            self._pending.append(len(params))
            self._direct_done.append(False)
            for p in params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(index)))
            if ref.is_cuda and self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=ref.device)
            if direct:
                sink = _LayerSink.create(self, index, layers[li], max(1, int(chunks)) if self.world > 1 else 1)
                if sink is not None:
                    self._sinks.append(sink)

    def _setup_symmetric(self, per_layer: List[List[nn.Parameter]], transport: str) -> None:
        env = os.environ.get("KAN_B200_ALLREDUCE", "").lower()
        if env in ("nccl", "nvlink", "p2p"):
            transport = "nccl" if env == "nccl" else "nvlink"
        if transport == "nccl" or self.world == 1 or not per_layer:
            return
        if transport == "auto" and self.world < 8:
            # measured on B200 with the 42 MB bucket of a 1024x1024 layer: 2 ranks, NCCL 0.10 ms
            # against 0.13 ms for the in-switch kernel (a rank's own slice loops back through its
            # link); 4 ranks, the whole step is 2 % faster with NCCL; 8 ranks, 0.12 against 0.19 ms
            # and the step is 7 % faster with the in-switch kernel
            self.transport_note = "NCCL is the faster transport below 8 ranks"
            return
        params = [p for layer in per_layer for p in layer]
        same = all(p.is_cuda and p.dtype == torch.float32 and p.device == params[0].device for p in params)
        try:
            if not same:
                raise RuntimeError("the NVLink transport needs float32 parameters on one CUDA device")
            if self.world > 16:
                raise RuntimeError("the NVLink transport serves up to 16 ranks of one node")
            self._symm = _SymmetricBuckets([sum(p.numel() for p in layer) for layer in per_layer],
                                           params[0].device, self.group, use_multicast=(env != "p2p"))
            failure = None
        except Exception as exc:                       # noqa: BLE001  (any set-up failure -> NCCL)
            self._symm = None
            failure = exc
        # every rank must end up with the same transport (and the same kind of kernel)
        flags = torch.tensor([1 if self._symm is not None else 0,
                              1 if self._symm is not None and self._symm.multicast_ptr else 0],
                             dtype=torch.int32, device=params[0].device if all(p.is_cuda for p in params) else "cpu")
        dist.all_reduce(flags, op=dist.ReduceOp.MIN, group=self.group)
        all_ok, all_mc = (int(v) for v in flags.tolist())
        if not all_ok:
            self._symm = None
            if transport == "nvlink":
                raise RuntimeError(f"NVLink transport unavailable on at least one rank (here: {failure!r})")
            self.transport_note = f"NVLink transport unavailable ({failure!r}); using NCCL"
            return
        if not all_mc:
            self._symm.multicast_ptr = 0
        self.transport = "nvlink-multimem" if self._symm.multicast_ptr else "nvlink-p2p"

    @property
    def buckets(self) -> List[torch.Tensor]:
        return [flat for flat, _ in self._buckets]

    def bucket_bytes(self) -> int:
        return sum(flat.numel() * flat.element_size() for flat, _ in self._buckets)

    def _make_hook(self, index: int):
        def hook(param: nn.Parameter) -> None:
            if self._direct_done[index]:
                return        # the backward wrote this layer's gradients into the bucket and reduced them
            flat, params = self._buckets[index]
            # autograd may have replaced the view with a fresh tensor: fold it back.
            lo = 0
            for p in params:
                if p is param:
                    view = flat[lo:lo + p.numel()].view_as(p)
                    if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
                        view.copy_(p.grad)
                        p.grad = view
                    break
                lo += p.numel()
            self._pending[index] -= 1
            if self._pending[index] == 0:
                self._launch(index)
        return hook

    def _launch(self, index: int) -> None:
        flat, _ = self._buckets[index]
        if self.world == 1:
            return
        if flat.is_cuda:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(flat.device))
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                if self._symm is not None:
                    self._symm.all_reduce(index, 1.0 / self.world if self.average else 1.0)
                else:
                    self._works.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group,
                                                       async_op=True))
        else:
            self._works.append(dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self) -> None:
        """Waits for the collectives (the current stream waits for the communication stream)."""
        for i, left in enumerate(self._pending):
            if left > 0 and left < len(self._buckets[i][1]) and not self._direct_done[i]:
                self._launch(i)                   # partially used layer: reduce what is there
        for w in self._works:
            w.wait()
        self._works.clear()
        if self._comm_stream is not None:
            torch.cuda.current_stream(self._comm_stream.device).wait_stream(self._comm_stream)
        if self.average and self.world > 1 and self._symm is None:
            for flat, _ in self._buckets:
                flat.div_(self.world)
        self._pending = [len(params) for _, params in self._buckets]
        self._direct_done = [False] * len(self._buckets)

    def zero_grad(self) -> None:
        """Zeros the buckets in place (keeps ``param.grad`` as views)."""
        for flat, params in self._buckets:
            flat.zero_()
            lo = 0
            for p in params:
                if p.grad is None or p.grad.data_ptr() != flat[lo:lo + 1].data_ptr():
                    p.grad = flat[lo:lo + p.numel()].view_as(p)
                lo += p.numel()

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        for sink in self._sinks:
            sink.remove()
        self._sinks.clear()

    def _reduce_ranges(self, index: int, ranges: List[Tuple[int, int]]) -> None:
        """All-reduce of ``(float offset, float count)`` ranges of bucket ``index``, behind the work
        queued so far on the current stream."""
        flat, _ = self._buckets[index]
        if self.world == 1:
            return
        merged: List[Tuple[int, int]] = []
        for lo, n in sorted(ranges):                       # adjacent ranges become one collective
            if merged and merged[-1][0] + merged[-1][1] == lo:
                merged[-1] = (merged[-1][0], merged[-1][1] + n)
            else:
                merged.append((lo, n))
        ranges = merged
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(flat.device))
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ready)
            if self._symm is not None:
                self._symm.all_reduce_ranges(index, ranges, 1.0 / self.world if self.average else 1.0)
            else:
                for lo, n in ranges:
                    self._works.append(dist.all_reduce(flat[lo:lo + n], op=dist.ReduceOp.SUM, group=self.group,
                                                       async_op=True))

    def check(self) -> None:
        """Synchronises and raises if an NVLink all-reduce kernel gave up waiting for another rank."""
        if self._symm is not None:
            self._symm.check()


class _LayerSink:
    """Receives the parameter gradients of one KANLinear-like layer directly from its backward (see
    ``_C.register_grad_sink``) and starts the all-reduce of each finished range of output rows."""

    def __init__(self, bucket: "GradientBucket", index: int, layer: nn.Module, chunks: int,
                 offsets: dict) -> None:
        self.bucket, self.index, self.layer, self.chunks, self.offsets = bucket, index, layer, chunks, offsets
        from . import _C
        self._C = _C
        self.key = layer.spline_weight
        _C.register_grad_sink(self.key, self)

    @staticmethod
    def create(bucket: "GradientBucket", index: int, layer: nn.Module, chunks: int) -> Optional["_LayerSink"]:
        sw = getattr(layer, "spline_weight", None)
        bw = getattr(layer, "base_weight", None)
        if not isinstance(sw, nn.Parameter) or not isinstance(bw, nn.Parameter) or not sw.is_cuda:
            return None
        if sw.dtype != torch.float32 or sw.dim() != 3:
            return None
        flat, params = bucket._buckets[index]
        offsets, lo = {}, 0
        for p in params:
            offsets[id(p)] = lo
            lo += p.numel()
        expected = {id(sw), id(bw)}
        sc = getattr(layer, "spline_scaler", None)
        if isinstance(sc, nn.Parameter):
            expected.add(id(sc))
        if set(offsets) != expected:
            return None                                   # the layer has other parameters: hooks handle it
        O, I, R = sw.shape
        # the all-reduce kernel moves 16-byte pieces: every range of rows of every parameter must
        # start and end on one
        if (O * I) % 4 != 0 or any((off % 4) for off in offsets.values()):
            return None
        if I % 4 != 0:
            chunks = 1
        return _LayerSink(bucket, index, layer, chunks, offsets)

    def remove(self) -> None:
        self._C.unregister_grad_sink(self.key)

    def destinations(self, base_weight, spline_weight, spline_scaler):
        """Bucket views for (d base_weight, d spline_weight, d spline_scaler), or None when the call
        does not belong to this layer's parameters."""
        layer = self.layer
        if spline_weight.data_ptr() != layer.spline_weight.data_ptr():
            return None
        if (base_weight is None) or base_weight.data_ptr() != layer.base_weight.data_ptr():
            return None
        sc = getattr(layer, "spline_scaler", None)
        has_sc = isinstance(sc, nn.Parameter)
        if has_sc != (spline_scaler is not None):
            return None
        flat, _ = self.bucket._buckets[self.index]

        def view(p):
            lo = self.offsets[id(p)]
            v = flat[lo:lo + p.numel()].view_as(p)
            if p.grad is None or p.grad.data_ptr() != v.data_ptr():
                p.grad = v
            return v
        return view(layer.base_weight), view(layer.spline_weight), (view(sc) if has_sc else None)

    def row_ranges(self, O: int) -> List[Tuple[int, int]]:
        rows = -(-O // self.chunks)
        rows = -(-rows // 256) * 256                      # whole 256-output tiles of the kernels
        return [(o0, min(O, o0 + rows)) for o0 in range(0, O, rows)]

    def rows_done(self, o0: int, o1: int) -> None:
        layer = self.layer
        O, I, R = layer.spline_weight.shape
        ranges = [(self.offsets[id(layer.spline_weight)] + o0 * I * R, (o1 - o0) * I * R),
                  (self.offsets[id(layer.base_weight)] + o0 * I, (o1 - o0) * I)]
        sc = getattr(layer, "spline_scaler", None)
        if isinstance(sc, nn.Parameter):
            ranges.append((self.offsets[id(sc)] + o0 * I, (o1 - o0) * I))
        self.bucket._reduce_ranges(self.index, ranges)
        if o1 >= O:
            self.bucket._direct_done[self.index] = True


class _SymmetricBuckets:
    """One symmetric allocation ``[bucket 0 | bucket 1 | ... | signal pad]`` shared by the ranks of
    a node, and the launcher of the library's all-reduce kernel on its buckets."""

    # The in-switch reduction is bound by the links, not by the number of requests in flight: a few
    # blocks reach its rate and leave the SMs to the backward kernels of the layers below.  Peer
    # loads need many more requests in flight.
    BLOCKS_MULTIMEM = 8
    BLOCKS_P2P = 96
    MAX_BLOCKS = 128

    def __init__(self, sizes: List[int], device: torch.device, group, use_multicast: bool = True) -> None:
        import torch.distributed._symmetric_memory as symm
        from . import _native
        self._native = _native
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.offsets, total = [], 0
        self.sizes = [(n + 3) // 4 * 4 for n in sizes]          # the kernel moves 16-byte pieces
        self.used = list(sizes)
        for n in self.sizes:
            self.offsets.append(total)
            total += (n + 63) // 64 * 64                           # 256-byte aligned buckets
        self.pad_offset = total * 4
        pad_floats = _native.allreduce_pad_bytes(self.world, self.MAX_BLOCKS) // 4
        pg = group if group is not None else dist.group.WORLD
        self.buffer = symm.empty(total + pad_floats, dtype=torch.float32, device=device)
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm.rendezvous(self.buffer, pg.group_name)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        mc = int(self.handle.multicast_ptr) if use_multicast else 0
        self.multicast_ptr = mc
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        dist.barrier(group)                                        # every pad is zero before first use

    def flat(self, index: int) -> torch.Tensor:
        lo = self.offsets[index]
        return self.buffer[lo:lo + self.used[index]]

    def all_reduce(self, index: int, scale: float) -> None:
        self._native.allreduce_sum(self.peer_ptrs, self.multicast_ptr, self.offsets[index] * 4, self.pad_offset,
                                   self.sizes[index], self.rank, self.world, self.status,
                                   blocks=self.BLOCKS_MULTIMEM if self.multicast_ptr else self.BLOCKS_P2P,
                                   scale=scale)

    def all_reduce_ranges(self, index: int, ranges: List[Tuple[int, int]], scale: float) -> None:
        base = self.offsets[index] * 4
        mm = bool(self.multicast_ptr)
        # few small blocks: they share the SMs with the tensor-core kernel of the next range
        self._native.allreduce_sum_ranges(self.peer_ptrs, self.multicast_ptr,
                                          [(base + lo * 4, n) for lo, n in ranges], self.pad_offset,
                                          self.rank, self.world, self.status,
                                          blocks=self.BLOCKS_MULTIMEM if mm else 48, threads=128, scale=scale)

    def check(self) -> None:
        if int(self.status.item()) != 0:
            raise RuntimeError("NVLink all-reduce: a bounded wait on another rank ran out "
                               "(a rank is missing or far behind); the signal pad must be zeroed before reuse")


class HostBatchPrefetcher:
    """Double-buffered host-to-device staging of input batches.

    ``submit(host_batch)`` starts the copy of a pinned host batch into one of two device buffers
    on a side stream; ``next()`` returns the oldest submitted batch once the compute stream has
    been made to wait for its copy.  Submitting batch t+1 before running step t hides the copy
    behind the step (the PCIe copy engine and the SMs work at the same time)::

        pre = HostBatchPrefetcher(x_host.shape, x_host.dtype, device)
        pre.submit(batches[0])
        for t in range(steps):
            if t + 1 < steps:
                pre.submit(batches[t + 1])
            x = pre.next()
            loss = step(x)

    A staging buffer is overwritten only after everything that was queued on the compute stream
    before the ``submit`` that reuses it has finished: ``submit`` records an event there and the copy
    stream waits for it.  The last reader of the buffer (the step two batches back) was queued before
    that point, however long it runs.
    """

    def __init__(self, shape, dtype: torch.dtype, device: torch.device) -> None:
        if torch.device(device).type != "cuda":
            raise ValueError("HostBatchPrefetcher stages batches on a CUDA device")
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device)
        self._bufs = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(2)]
        self._ready = [torch.cuda.Event(), torch.cuda.Event()]
        self._handed_out = [False, False]
        self._submitted = 0
        self._taken = 0

    def submit(self, host_batch: torch.Tensor) -> None:
        if self._submitted - self._taken >= 2:
            raise RuntimeError("both staging buffers are in flight: call next() before submitting again")
        if host_batch.shape != self._bufs[0].shape or host_batch.dtype != self._bufs[0].dtype:
            raise ValueError(f"batch of shape {tuple(host_batch.shape)} / {host_batch.dtype} does not match the "
                             f"staging buffers {tuple(self._bufs[0].shape)} / {self._bufs[0].dtype}")
        i = self._submitted % 2
        if self._handed_out[i]:
            # the buffer's previous batch was given to the caller: its readers are on the compute
            # stream, queued before this point
            consumed = torch.cuda.Event()
            consumed.record(torch.cuda.current_stream(self.device))
            self.stream.wait_event(consumed)
        with torch.cuda.stream(self.stream):
            self._bufs[i].copy_(host_batch, non_blocking=True)
            self._ready[i].record(self.stream)
        self._submitted += 1

    def next(self) -> torch.Tensor:
        if self._taken >= self._submitted:
            raise RuntimeError("next() without a submitted batch")
        i = self._taken % 2
        torch.cuda.current_stream(self.device).wait_event(self._ready[i])
        self._handed_out[i] = True
        self._taken += 1
        return self._bufs[i]
