"""ctypes binding of ``lib/libkan_b200.so`` (the C ABI in ``include/kan_b200.h``).

PyTorch is used here only for device memory, streams and dtype bookkeeping:
every function takes CUDA tensors, passes their raw pointers and the current
stream to the library and returns freshly allocated outputs.  There is no CPU
implementation behind these calls -- a missing library or a CPU tensor raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional, Sequence, Tuple

import torch

from .build import LIB_PATH

F32, F64 = 0, 1
MODE_AUTO, MODE_SIMT, MODE_TC_BF16X3, MODE_TC_BF16X1 = 0, 1, 2, 3
MODES = {"auto": MODE_AUTO, "simt": MODE_SIMT, "bf16x3": MODE_TC_BF16X3, "bf16x1": MODE_TC_BF16X1}
OP_FORWARD, OP_BACKWARD, OP_EDGE_FWD, OP_EDGE_BWD, OP_BASIS, OP_EDGE_X_FWD, OP_EDGE_X_BWD = 0, 1, 2, 3, 4, 5, 6
EINVAL, EUNSUPPORTED, EWORKSPACE, ECUDA, EDEVICE = -1, -2, -3, -4, -5
MAX_DEG0_BASIS = 71
MAX_IN_FEATURES = 65535

_c_void_p, _c_int, _c_i64, _c_size = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t

# name -> (restype, argtypes); must list every symbol of include/kan_b200.h
SIGNATURES = {
    "kanb200_last_error": (ctypes.c_char_p, []),
    "kanb200_version": (_c_int, []),
    "kanb200_set_basis_impl": (_c_int, [_c_int]),
    "kanb200_get_basis_impl": (_c_int, []),
    "kanb200_set_accumulation_chunks": (_c_int, [_c_int, _c_int, _c_int]),
    "kanb200_check_shapes": (_c_int, [_c_i64, _c_i64, _c_i64, _c_int, _c_int, _c_int]),
    "kanb200_resolve_mode": (_c_int, [_c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int]),
    "kanb200_resolve_mode_for": (_c_int, [_c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int]),
    "kanb200_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int, _c_i64, _c_i64, _c_i64, _c_int, _c_int,
                                          _c_int, _c_int]),
    "kanb200_basis": (_c_int, [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_int, _c_int, _c_void_p]),
    "kanb200_basis_grad": (_c_int, [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_int,
                                    _c_int, _c_void_p]),
    "kanb200_basis_ws": (_c_int, [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_int, _c_int, _c_void_p,
                                  _c_size, _c_void_p]),
    "kanb200_basis_grad_ws": (_c_int, [_c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_i64, _c_i64, _c_int,
                                       _c_int, _c_void_p, _c_size, _c_void_p]),
    "kanb200_forward": (_c_int, [_c_int, _c_int] + [_c_void_p] * 6 + [_c_i64, _c_i64, _c_i64, _c_int, _c_int,
                                                                     _c_void_p, _c_size, _c_void_p]),
    "kanb200_backward": (_c_int, [_c_int, _c_int] + [_c_void_p] * 10 + [_c_i64, _c_i64, _c_i64, _c_int, _c_int,
                                                                       _c_void_p, _c_size, _c_void_p]),
    "kanb200_edge_abs_mean": (_c_int, [_c_int] + [_c_void_p] * 5 + [_c_i64, _c_i64, _c_i64, _c_int,
                                                                   _c_void_p, _c_size, _c_void_p]),
    "kanb200_edge_abs_mean_x": (_c_int, [_c_int, _c_int] + [_c_void_p] * 6 + [_c_i64, _c_i64, _c_i64, _c_int, _c_int,
                                                                             _c_void_p, _c_size, _c_void_p]),
    "kanb200_set_forward_variant": (_c_int, [_c_int]),
    "kanb200_set_edge_sign_recheck": (_c_int, [_c_int]),
    "kanb200_get_edge_sign_recheck": (_c_int, []),
    "kanb200_prepared_bytes": (_c_size, [_c_int, _c_i64, _c_i64, _c_int, _c_int, _c_int]),
    "kanb200_prepare_forward": (_c_int, [_c_int] + [_c_void_p] * 4 + [_c_i64, _c_i64, _c_int, _c_int, _c_void_p, _c_size,
                                         _c_void_p]),
    "kanb200_forward_prepared": (_c_int, [_c_int, _c_int, _c_void_p, _c_void_p, _c_size, _c_int, _c_void_p, _c_i64, _c_i64,
                                          _c_i64, _c_int, _c_int, _c_void_p, _c_size, _c_void_p]),
    "kanb200_edge_penalty_workspace_bytes": (_c_size, []),
    "kanb200_edge_penalty": (_c_int, [_c_int, _c_void_p, _c_i64, ctypes.c_double, ctypes.c_double, _c_void_p, _c_void_p,
                                      _c_void_p, _c_size, _c_void_p]),
    "kanb200_edge_abs_mean_x_backward": (_c_int, [_c_int, _c_int] + [_c_void_p] * 10 + [_c_i64, _c_i64, _c_i64, _c_int, _c_int,
                                                                               _c_void_p, _c_size, _c_void_p]),
    "kanb200_edge_abs_mean_noalloc": (_c_int, [_c_int] + [_c_void_p] * 5 + [_c_i64, _c_i64, _c_i64, _c_int, _c_void_p]),
    "kanb200_edge_abs_mean_backward": (_c_int, [_c_int] + [_c_void_p] * 9 + [_c_i64, _c_i64, _c_i64, _c_int,
                                                                            _c_void_p, _c_size, _c_void_p]),
    "kanb200_refit_transfer": (_c_int, [_c_int] + [_c_void_p] * 6 + [_c_i64, _c_i64, _c_int, _c_int, _c_void_p]),
    "kanb200_check_status": (_c_int, [_c_void_p, _c_void_p]),
    "kanb200_backward_param_rows": (_c_int, [_c_int] + [_c_void_p] * 9 + [_c_i64, _c_i64, _c_i64, _c_int, _c_int,
                                                                          _c_i64, _c_i64, _c_void_p, _c_size,
                                                                          _c_void_p]),
    "kanb200_allreduce_pad_bytes": (_c_size, [_c_int, _c_int]),
    "kanb200_allreduce_set_wait_limit_ms": (_c_int, [_c_int]),
    "kanb200_allreduce_sum_f32_ranges": (_c_int, [ctypes.POINTER(_c_void_p), _c_void_p, ctypes.POINTER(_c_size),
                                                  ctypes.POINTER(_c_size), _c_int, _c_size, _c_int, _c_int, _c_int,
                                                  _c_int, _c_int, ctypes.c_float, _c_void_p, _c_void_p]),
    "kanb200_allreduce_sum_f32": (_c_int, [ctypes.POINTER(_c_void_p), _c_void_p, _c_size, _c_size, _c_size,
                                           _c_int, _c_int, _c_int, _c_int, ctypes.c_float, _c_void_p, _c_void_p]),
}

_lib = None
_lock = threading.Lock()


def lib() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python torchsplinekan_b200/build.py` "
                        "(needs nvcc).  This package has no fallback implementation.")
                handle = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    if not hasattr(handle, name):
                        raise RuntimeError(f"{LIB_PATH} is older than this package (no symbol {name}): "
                                           "rebuild it with `python torchsplinekan_b200/build.py`")
                    fn = getattr(handle, name)
                    fn.restype, fn.argtypes = res, args
                _lib = handle
                variant = os.environ.get("KAN_B200_FORWARD_VARIANT")     # "tmem" | "smem": see kanb200_set_forward_variant
                if variant in ("tmem", "smem"):
                    handle.kanb200_set_forward_variant(1 if variant == "tmem" else 0)
    return _lib


def last_error() -> str:
    return lib().kanb200_last_error().decode("utf-8", "replace")


def _check(rc: int) -> None:
    if rc == 0:
        return
    msg = last_error()
    if rc == EINVAL:
        raise RuntimeError(msg)
    raise RuntimeError(f"kan_b200 error {rc}: {msg}")


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.float64:
        return F64
    raise RuntimeError(f"only FP32 and FP64 inputs are supported, got {dtype}")


def _p(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else ctypes.c_void_p(t.data_ptr())


def _stream(dev: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None or t.numel() == 0:
            continue
        if not t.is_cuda:
            raise RuntimeError("kan_b200: expected CUDA tensors (there is no CPU path in this library)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("kan_b200: all tensors must be on the same device")
    if dev is None:
        raise RuntimeError("kan_b200: no CUDA tensor given")
    return dev


_ws_cache = {}

# When set to a list, forward()/backward() append (name, start_event, end_event) recorded on the
# launching stream around the library call; the benchmark uses it for per-kernel durations.
EVENT_LOG = None


class _Timed:
    def __init__(self, name: str, dev: torch.device):
        self.name, self.dev = name, dev

    def __enter__(self):
        if EVENT_LOG is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.dev))
        return self

    def __exit__(self, *exc):
        if EVENT_LOG is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(torch.cuda.current_stream(self.dev))
            EVENT_LOG.append((self.name, self.start, end))
        return False


def workspace(dev: torch.device, nbytes: int, tag: str = "") -> Optional[torch.Tensor]:
    """Per (device, stream, tag) scratch buffer, grown on demand and reused."""
    if nbytes <= 0:
        return None
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream, tag)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = None
        _ws_cache.pop(key, None)
        buf = torch.empty(int(nbytes * 1.0) + 256, dtype=torch.uint8, device=dev)
        buf[:256].zero_()
        _ws_cache[key] = buf
    return buf


def release_workspaces() -> None:
    _ws_cache.clear()


def resolve_mode(mode: int, dtype: torch.dtype, N: int, I: int, O: int, G: int, k: int, op: int = None) -> int:
    """Kernel family of a call (``op``: OP_FORWARD or OP_BACKWARD, the default)."""
    m = lib().kanb200_resolve_mode_for(OP_BACKWARD if op is None else op, mode, _code(dtype), N, I, O, G, k)
    if m < 0:
        _check(m)
    return m


_ws_size_cache = {}


def workspace_bytes(op, mode, dtype, N, I, O, G, k, need_x=True, need_param=True) -> int:
    key = (op, mode, dtype, N, I, O, G, k, bool(need_x), bool(need_param))
    size = _ws_size_cache.get(key)
    if size is None:
        size = int(lib().kanb200_workspace_bytes(op, mode, _code(dtype), N, I, O, G, k, int(need_x), int(need_param)))
        if len(_ws_size_cache) > 4096:
            _ws_size_cache.clear()
        _ws_size_cache[key] = size
    return size


class _OnDevice:
    """Makes ``dev`` current for the duration of a library call; free when it already is."""

    def __init__(self, dev: torch.device):
        self.ctx = None if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


def basis(x: torch.Tensor, grid: torch.Tensor, k: int) -> torch.Tensor:
    dev = _need_cuda(x, grid)
    N, I = x.shape
    G = grid.shape[1] - 2 * k - 1
    H = torch.empty((N, I, G + k), dtype=x.dtype, device=dev)
    with _OnDevice(dev):
        ws = workspace(dev, workspace_bytes(OP_BASIS, MODE_AUTO, x.dtype, N, I, 1, G, k), "basis")
        _check(lib().kanb200_basis_ws(_code(x.dtype), _p(x), _p(grid), _p(H), N, I, G, k,
                                      _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return H


def basis_grad(x: torch.Tensor, grid: torch.Tensor, k: int, gH: torch.Tensor) -> torch.Tensor:
    dev = _need_cuda(x, grid, gH)
    N, I = x.shape
    G = grid.shape[1] - 2 * k - 1
    gx = torch.empty((N, I), dtype=x.dtype, device=dev)
    with _OnDevice(dev):
        ws = workspace(dev, workspace_bytes(OP_BASIS, MODE_AUTO, x.dtype, N, I, 1, G, k), "basis")
        _check(lib().kanb200_basis_grad_ws(_code(x.dtype), _p(x), _p(grid), _p(gH), _p(gx), N, I, G, k,
                                           _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return gx


def forward(x, grid, base_weight, spline_weight, spline_scaler, k: int, mode: int = MODE_AUTO,
            ws: Optional[torch.Tensor] = None) -> torch.Tensor:
    dev = _need_cuda(x, grid, spline_weight)
    N, I = x.shape
    O = spline_weight.shape[0]
    G = grid.shape[1] - 2 * k - 1
    y = torch.empty((N, O), dtype=x.dtype, device=dev)
    with _OnDevice(dev):
        if ws is None:
            ws = workspace(dev, workspace_bytes(OP_FORWARD, mode, x.dtype, N, I, O, G, k), "fwd")
        with _Timed("forward", dev):
            _check(lib().kanb200_forward(_code(x.dtype), mode, _p(x), _p(grid), _p(base_weight),
                                         _p(spline_weight), _p(spline_scaler), _p(y), N, I, O, G, k, _p(ws),
                                         0 if ws is None else ws.numel(), _stream(dev)))
    return y


def prepare_forward(grid, base_weight, spline_weight, spline_scaler, k: int) -> Optional[torch.Tensor]:
    """Table + weight image of a layer with fixed parameters (bytes on the device), or None when the
    configuration has no prepared form (float64, k > 3)."""
    dev = _need_cuda(grid, spline_weight)
    O, I, _ = spline_weight.shape
    G = grid.shape[1] - 2 * k - 1
    has_base = base_weight is not None and base_weight.numel() > 0
    nb = lib().kanb200_prepared_bytes(_code(spline_weight.dtype), I, O, G, k, int(has_base))
    if nb == 0:
        return None
    buf = torch.empty(nb, dtype=torch.uint8, device=dev)
    with _OnDevice(dev):
        _check(lib().kanb200_prepare_forward(_code(spline_weight.dtype), _p(grid), _p(base_weight if has_base else None),
                                             _p(spline_weight), _p(spline_scaler), I, O, G, k, _p(buf), nb,
                                             _stream(dev)))
    return buf


def forward_prepared(x, prepared: torch.Tensor, O: int, G: int, k: int, has_base: bool,
                     mode: int = MODE_AUTO) -> torch.Tensor:
    """``y = layer(x)`` from x and the buffer of :func:`prepare_forward`: the contraction alone."""
    dev = _need_cuda(x, prepared)
    N, I = x.shape
    y = torch.empty((N, O), dtype=x.dtype, device=dev)
    with _OnDevice(dev):
        ws = workspace(dev, max(256, workspace_bytes(OP_FORWARD, MODE_TC_BF16X3, x.dtype, N, I, O, G, k)), "fwd")
        _check(lib().kanb200_forward_prepared(_code(x.dtype), mode, _p(x), _p(prepared), prepared.numel(), int(has_base),
                                              _p(y), N, I, O, G, k, _p(ws), ws.numel(), _stream(dev)))
    return y


def backward(grad_out, x, grid, base_weight, spline_weight, spline_scaler, k: int,
             need_x: bool, need_base: bool, need_spline: bool, need_scaler: bool, mode: int = MODE_AUTO,
             ws: Optional[torch.Tensor] = None
             ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor], Optional[torch.Tensor]]:
    dev = _need_cuda(x, grid, spline_weight, grad_out)
    N, I = x.shape
    O = spline_weight.shape[0]
    G = grid.shape[1] - 2 * k - 1
    has_base = base_weight is not None and base_weight.numel() > 0
    has_scaler = spline_scaler is not None and spline_scaler.numel() > 0
    need_base = need_base and has_base
    need_scaler = need_scaler and has_scaler
    gx = torch.empty_like(x) if need_x else None
    gb = torch.empty_like(base_weight) if need_base else None
    gs = torch.empty_like(spline_weight) if need_spline else None
    gc = torch.empty_like(spline_scaler) if need_scaler else None
    with _OnDevice(dev):
        if ws is None:
            nb = workspace_bytes(OP_BACKWARD, mode, x.dtype, N, I, O, G, k, need_x,
                                 need_base or need_spline or need_scaler)
            ws = workspace(dev, nb, "bwd")
        with _Timed("backward", dev):
            _check(lib().kanb200_backward(_code(x.dtype), mode, _p(grad_out), _p(x), _p(grid), _p(base_weight),
                                          _p(spline_weight), _p(spline_scaler), _p(gx), _p(gb), _p(gs), _p(gc),
                                          N, I, O, G, k, _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return gx, gb, gs, gc


def backward_param_rows(grad_out, x, grid, base_weight, spline_weight, spline_scaler, k: int,
                        o_begin: int, o_end: int, gb: Optional[torch.Tensor], gs: Optional[torch.Tensor],
                        gc: Optional[torch.Tensor], mode: int) -> None:
    """Parameter gradients of the output rows ``[o_begin, o_end)`` written into the given full-size
    tensors ``gb [O, I]``, ``gs [O, I, R]``, ``gc [O, I]`` (None = not needed); tensor-core modes."""
    dev = _need_cuda(x, grid, spline_weight, grad_out)
    N, I = x.shape
    O = spline_weight.shape[0]
    G = grid.shape[1] - 2 * k - 1
    for t in (gb, gs, gc):
        if t is not None and not t.is_contiguous():
            raise RuntimeError("backward_param_rows: gradient destinations must be contiguous")
    with _OnDevice(dev):
        nb = workspace_bytes(OP_BACKWARD, mode, x.dtype, N, I, o_end - o_begin, G, k, False, True)
        ws = workspace(dev, nb, "bwd")
        with _Timed("backward", dev):
            _check(lib().kanb200_backward_param_rows(mode, _p(grad_out), _p(x), _p(grid), _p(base_weight),
                                                     _p(spline_weight), _p(spline_scaler), _p(gb), _p(gs), _p(gc),
                                                     N, I, O, G, k, int(o_begin), int(o_end),
                                                     _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))


def edge_abs_mean(s, H, bw, W) -> torch.Tensor:
    dev = _need_cuda(H, W)
    N, I, R = H.shape
    O = W.shape[0]
    a = torch.empty((O, I), dtype=H.dtype, device=dev)
    with _OnDevice(dev):
        nb = workspace_bytes(OP_EDGE_FWD, MODE_SIMT, H.dtype, N, I, O, max(R - 1, 1), 1)
        ws = workspace(dev, nb, "edge")
        _check(lib().kanb200_edge_abs_mean(_code(H.dtype), _p(s), _p(H), _p(bw), _p(W), _p(a), N, I, O, R,
                                           _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return a


def edge_abs_mean_x(x, s, grid, bw, W, k: int, mode: int = MODE_AUTO) -> torch.Tensor:
    """``a [O, I]`` straight from the layer input ``x`` (``s``: base values or None = SiLU of x)."""
    dev = _need_cuda(x, grid, W)
    N, I = x.shape
    O = W.shape[0]
    G = grid.shape[1] - 2 * k - 1
    a = torch.empty((O, I), dtype=x.dtype, device=dev)
    with _OnDevice(dev):
        ws = workspace(dev, workspace_bytes(OP_EDGE_X_FWD, mode, x.dtype, N, I, O, G, k), "edge_x")
        _check(lib().kanb200_edge_abs_mean_x(_code(x.dtype), mode, _p(x), _p(s), _p(grid), _p(bw), _p(W), _p(a),
                                             N, I, O, G, k, _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return a


def edge_penalty(a: torch.Tensor, mu1: float, mu2: float, need_grad: bool = True, scratch: bool = True):
    """``(mu1 sum(a) + mu2 entropy(a / sum(a)), d/da)`` (gradient None when not needed); ``scratch=False``
    withholds the workspace, i.e. forces the single-block form."""
    dev = _need_cuda(a)
    a = a.contiguous()
    value = torch.empty((), dtype=a.dtype, device=dev)
    grad = torch.empty_like(a) if need_grad else None
    nb = int(lib().kanb200_edge_penalty_workspace_bytes()) if scratch else 0
    ws = torch.empty(nb, dtype=torch.uint8, device=dev) if nb else None
    with _OnDevice(dev):
        _check(lib().kanb200_edge_penalty(_code(a.dtype), _p(a), a.numel(), float(mu1), float(mu2), _p(value),
                                          _p(grad), _p(ws), nb, _stream(dev)))
    return value, grad


def edge_abs_mean_x_backward(ga, x, s, grid, bw, W, k: int, need_x=True, need_s=True, need_bw=True, need_W=True,
                             mode: int = MODE_AUTO):
    """``(gx, ds, dbw, dW)`` of :func:`edge_abs_mean_x` (None where not needed / not applicable)."""
    dev = _need_cuda(x, grid, W, ga)
    N, I = x.shape
    O, _, R = W.shape
    G = grid.shape[1] - 2 * k - 1
    has_base = bw is not None and bw.numel() > 0
    gx = torch.empty_like(x) if need_x else None
    ds = torch.empty_like(x) if (need_s and has_base and s is not None) else None
    dbw = torch.empty((O, I), dtype=x.dtype, device=dev) if (need_bw and has_base) else None
    dW = torch.empty_like(W) if need_W else None
    with _OnDevice(dev):
        ws = workspace(dev, workspace_bytes(OP_EDGE_X_BWD, mode, x.dtype, N, I, O, G, k), "edge_x")
        _check(lib().kanb200_edge_abs_mean_x_backward(_code(x.dtype), mode, _p(ga), _p(x), _p(s), _p(grid), _p(bw), _p(W),
                                                      _p(gx), _p(ds), _p(dbw), _p(dW), N, I, O, G, k,
                                                      _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return gx, ds, dbw, dW


def set_edge_sign_recheck(on: bool) -> None:
    """Whether the tensor-core backward of the edge statistic evaluates near-zero phi again in float32
    before taking their sign (default on; off is about a third faster, signs at split-bf16 accuracy)."""
    _check(lib().kanb200_set_edge_sign_recheck(1 if on else 0))


def get_edge_sign_recheck() -> bool:
    return bool(lib().kanb200_get_edge_sign_recheck())


def edge_abs_mean_backward(ga, s, H, bw, W, need_s, need_H, need_bw, need_W):
    dev = _need_cuda(H, W, ga)
    N, I, R = H.shape
    O = W.shape[0]
    has_base = bw is not None and bw.numel() > 0
    ds = torch.empty((N, I), dtype=H.dtype, device=dev) if (need_s and has_base) else None
    dH = torch.empty_like(H) if need_H else None
    dbw = torch.empty((O, I), dtype=H.dtype, device=dev) if (need_bw and has_base) else None
    dW = torch.empty_like(W) if need_W else None
    with _OnDevice(dev):
        nb = workspace_bytes(OP_EDGE_BWD, MODE_SIMT, H.dtype, N, I, O, max(R - 1, 1), 1)
        ws = workspace(dev, nb, "edge")
        _check(lib().kanb200_edge_abs_mean_backward(_code(H.dtype), _p(ga), _p(s), _p(H), _p(bw), _p(W),
                                                    _p(ds), _p(dH), _p(dbw), _p(dW), N, I, O, R,
                                                    _p(ws), 0 if ws is None else ws.numel(), _stream(dev)))
    return ds, dH, dbw, dW


def refit_transfer(x: torch.Tensor, grid_old: torch.Tensor, grid_new: torch.Tensor, k: int):
    """``(transfer [I, R, R] float64, info [I] int32)``: per input feature the matrix that maps old
    spline coefficients to the least-squares refit on the new knots at the samples ``x``; ``info != 0``
    marks features whose normal equations are not safely positive definite."""
    dev = _need_cuda(x, grid_old, grid_new)
    N, I = x.shape
    G = grid_old.shape[1] - 2 * k - 1
    R = G + k
    gram = torch.empty((I, R, R), dtype=torch.float64, device=dev)
    transfer = torch.empty((I, R, R), dtype=torch.float64, device=dev)
    info = torch.empty((I,), dtype=torch.int32, device=dev)
    with _OnDevice(dev):
        _check(lib().kanb200_refit_transfer(_code(x.dtype), _p(x.contiguous()), _p(grid_old.contiguous()),
                                            _p(grid_new.contiguous()), _p(gram), _p(transfer), _p(info), N, I, G, k,
                                            _stream(dev)))
    return transfer, info


def check_status(ws: Optional[torch.Tensor]) -> None:
    """Raises if a tensor-core kernel that used ``ws`` reported a timed-out wait."""
    if ws is None:
        return
    with torch.cuda.device(ws.device):
        _check(lib().kanb200_check_status(_p(ws), _stream(ws.device)))


def check_all_workspaces() -> None:
    """:func:`check_status` on every scratch buffer this module handed out."""
    for buf in list(_ws_cache.values()):
        check_status(buf)


# ---------------------------------------------------------------------------
# gradient all-reduce over symmetric memory
# ---------------------------------------------------------------------------
MAX_RANKS = 16


def allreduce_set_wait_limit_ms(ms: int) -> None:
    _check(lib().kanb200_allreduce_set_wait_limit_ms(int(ms)))


def allreduce_pad_bytes(world: int, blocks: int) -> int:
    n = int(lib().kanb200_allreduce_pad_bytes(int(world), int(blocks)))
    if n == 0:
        raise RuntimeError(f"all-reduce: world size {world} / {blocks} blocks not supported")
    return n


def allreduce_sum_ranges(peer_ptrs: Sequence[int], multicast_ptr: int, ranges: Sequence[Tuple[int, int]],
                         pad_offset: int, rank: int, world: int, status: torch.Tensor, *, local_ranks: int = 1,
                         blocks: int = 8, threads: int = 512, scale: float = 1.0) -> None:
    """All-reduce of up to 4 ``(byte offset, float count)`` ranges of the allocation in one launch."""
    if not status.is_cuda or status.dtype != torch.int32 or status.numel() < 1:
        raise RuntimeError("all-reduce status must be a CUDA int32 tensor")
    arr = (_c_void_p * len(peer_ptrs))(*[int(v) for v in peer_ptrs])
    offs = (_c_size * len(ranges))(*[int(o) for o, _ in ranges])
    cnts = (_c_size * len(ranges))(*[int(n) for _, n in ranges])
    with torch.cuda.device(status.device):
        _check(lib().kanb200_allreduce_sum_f32_ranges(arr, _c_void_p(int(multicast_ptr) or None), offs, cnts,
                                                      len(ranges), int(pad_offset), int(rank), int(world),
                                                      int(local_ranks), int(blocks), int(threads), float(scale),
                                                      _p(status), _stream(status.device)))


def allreduce_sum(peer_ptrs: Sequence[int], multicast_ptr: int, payload_offset: int, pad_offset: int,
                  n_floats: int, rank: int, world: int, status: torch.Tensor, *, local_ranks: int = 1,
                  blocks: int = 32, scale: float = 1.0) -> None:
    """Launches the all-reduce kernel of this rank on the current stream of ``status.device``.
    ``peer_ptrs[p]``: this process's mapping of rank p's allocation; ``multicast_ptr``: multicast
    mapping of the same allocations or 0; ``status``: one int32 on the device."""
    if not status.is_cuda or status.dtype != torch.int32 or status.numel() < 1:
        raise RuntimeError("all-reduce status must be a CUDA int32 tensor")
    arr = (_c_void_p * len(peer_ptrs))(*[int(v) for v in peer_ptrs])
    with torch.cuda.device(status.device):
        _check(lib().kanb200_allreduce_sum_f32(arr, _c_void_p(int(multicast_ptr) or None), int(payload_offset),
                                               int(pad_offset), int(n_floats), int(rank), int(world),
                                               int(local_ranks), int(blocks), float(scale), _p(status),
                                               _stream(status.device)))
