"""
Operator surface of the native backend -- the counterpart of the reference's
pybind module ``spline_kan._C`` (csrc/kan_ext.cpp:161-222) and of its autograd
node (csrc/kan_autograd.cpp).  Same names, argument order and error behaviour;
the work is done by the C-ABI library through :mod:`._native`.

Differences that follow from the design of the kernels:
* the forward never materialises the basis; ``kan_forward`` still returns a
  dense ``basis`` tensor (from the stand-alone basis kernel) to honour the
  schema, ``kan_apply`` does not compute or save it, and ``kan_backward``
  accepts ``basis`` but recomputes what it needs from ``x``;
* CPU tensors are rejected (there is no CPU kernel behind these operators).
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import _native
from . import dense_backend as _dense

CUDA_MAX_DEG0_BASIS = _native.MAX_DEG0_BASIS
CUDA_MAX_IN_FEATURES = _native.MAX_IN_FEATURES
HAS_FUSED_KERNELS = True

_native.lib()           # load now: a missing library must fail at import, not at first use

_mode = _native.MODES.get(os.environ.get("KAN_B200_MODE", "auto").lower(), _native.MODE_AUTO)


def set_mma_mode(name: str) -> None:
    """Arithmetic of the fp32 contraction: "auto", "simt", "bf16x3" (split operands, fp32-level
    accuracy) or "bf16x1" (single bf16 MMA, about 3e-3 relative)."""
    global _mode
    if name not in _native.MODES:
        raise ValueError(f"mode must be one of {sorted(_native.MODES)}, got {name!r}")
    _mode = _native.MODES[name]


def get_mma_mode() -> str:
    return {v: k for k, v in _native.MODES.items()}[_mode]


def set_basis_impl(impl: int) -> None:
    """0 / 1 accepted for compatibility (csrc/kan_cuda.cu:274-279); anything else raises."""
    _native._check(_native.lib().kanb200_set_basis_impl(int(impl)))


def get_basis_impl() -> int:
    return int(_native.lib().kanb200_get_basis_impl())


def _has(t: Optional[torch.Tensor]) -> bool:
    return t is not None and t.numel() > 0


def _check_inputs(x, grid, base_weight, spline_weight, spline_scaler, spline_order: int, has_scaler: bool) -> None:
    """Shape / dtype / device / limit validation before any launch (csrc/kan_ops.h:27-78)."""
    if x.dim() != 2:
        raise RuntimeError(f"x must be 2-D [B, I], got {x.dim()}-D")
    if grid.dim() != 2:
        raise RuntimeError("grid must be 2-D [I, G+2k+1]")
    if spline_weight.dim() != 3:
        raise RuntimeError("spline_weight must be 3-D [O, I, R]")
    if not 1 <= spline_order <= 3:
        raise RuntimeError(f"spline_order must be 1, 2 or 3; got {spline_order}")
    I, O, T = x.size(1), spline_weight.size(0), grid.size(1)
    G = T - 2 * spline_order - 1
    if G < 1:
        raise RuntimeError(f"grid has {T} knots, too few for spline_order {spline_order}")
    if grid.size(0) != I:
        raise RuntimeError(f"grid.size(0)={grid.size(0)} must equal in_features={I}")
    if spline_weight.size(1) != I:
        raise RuntimeError(f"spline_weight.size(1) must equal in_features={I}")
    if spline_weight.size(2) != G + spline_order:
        raise RuntimeError(f"spline_weight.size(2)={spline_weight.size(2)} but grid implies R=G+k={G + spline_order}")
    if x.dtype not in (torch.float32, torch.float64):
        raise RuntimeError(f"only FP32 and FP64 inputs are supported, got {x.dtype}")
    if grid.dtype != x.dtype or spline_weight.dtype != x.dtype:
        raise RuntimeError("x, grid and spline_weight must share a dtype")
    if grid.device != x.device or spline_weight.device != x.device:
        raise RuntimeError("x, grid and spline_weight must be on the same device")
    if _has(base_weight):
        if base_weight.dim() != 2 or tuple(base_weight.shape) != (O, I):
            raise RuntimeError(f"base_weight must have shape [O, I] = [{O}, {I}]")
        if base_weight.dtype != x.dtype or base_weight.device != x.device:
            raise RuntimeError("base_weight must match x in dtype and device")
    if has_scaler:
        if spline_scaler is None or spline_scaler.dim() != 2 or tuple(spline_scaler.shape) != (O, I):
            raise RuntimeError(f"spline_scaler must have shape [O, I] = [{O}, {I}]")
        if spline_scaler.dtype != x.dtype or spline_scaler.device != x.device:
            raise RuntimeError("spline_scaler must match x in dtype and device")
    if not x.is_cuda:
        raise RuntimeError("kan_b200: x must be a CUDA tensor (this backend has no CPU kernels)")
    if G + 2 * spline_order > CUDA_MAX_DEG0_BASIS:
        raise RuntimeError(f"CUDA kernel supports G + 2k <= {CUDA_MAX_DEG0_BASIS} (got G={G}, k={spline_order}); "
                           "use backend='reference' for larger grids")
    if I > CUDA_MAX_IN_FEATURES:
        raise RuntimeError(f"CUDA kernel supports in_features <= {CUDA_MAX_IN_FEATURES}, got {I}")


def _c(t):
    return t.contiguous() if _has(t) else None


def _forward_impl(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler):
    _check_inputs(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler)
    return _native.forward(_c(x), _c(grid), _c(base_weight), _c(spline_weight),
                           _c(spline_scaler) if has_scaler else None, int(spline_order), _mode)


def kan_forward(x, grid, base_weight, spline_weight, spline_scaler, spline_order: int, has_scaler: bool
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(output [B, O], basis [B, I, R])`` (kan_forward_cuda, csrc/kan_cuda.cu:469-532)."""
    y = _forward_impl(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler)
    return y, _native.basis(_c(x), _c(grid), int(spline_order))


def _backward_impl(grad_output, x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler,
                   need_x=True, need_base=True, need_spline=True):
    _check_inputs(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler)
    if tuple(grad_output.shape) != (x.size(0), spline_weight.size(0)):
        raise RuntimeError("grad_output must have shape [B, O]")
    gx, gb, gs, gc = _native.backward(
        _c(grad_output.to(x.dtype)), _c(x), _c(grid), _c(base_weight), _c(spline_weight),
        _c(spline_scaler) if has_scaler else None, int(spline_order),
        need_x, need_base, need_spline, need_spline and has_scaler, _mode)
    return gx, gb, gs, gc


def kan_backward(grad_output, x, grid, base_weight, spline_weight, spline_scaler, basis, spline_order: int,
                 has_scaler: bool):
    """``(grad_x, grad_base_weight|None, grad_spline_weight, grad_spline_scaler|None)``
    (kan_backward_cuda, csrc/kan_cuda.cu:632-647).  ``basis`` is accepted and ignored."""
    return _backward_impl(grad_output, x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler)


def kan_backward_composite(grad_output, x, grid, base_weight, spline_weight, spline_scaler, spline_order: int,
                           has_scaler: bool):
    """Backward built from differentiable PyTorch ops only, basis recomputed from ``x``; used while a
    backward pass is being recorded so that higher-order derivatives are exact
    (kan_backward_composite, csrc/kan_cpu.cpp:301-345)."""
    B, I = x.shape
    O, _, R = spline_weight.shape
    D = grad_output
    H = _dense.compute_basis(x, grid, spline_order)
    W = spline_weight * spline_scaler.unsqueeze(2) if has_scaler else spline_weight
    DtH = (D.t() @ H.reshape(B, I * R)).reshape(O, I, R)
    if has_scaler:
        g_spline, g_scaler = spline_scaler.unsqueeze(2) * DtH, (spline_weight * DtH).sum(2)
    else:
        g_spline, g_scaler = DtH, None
    dH = _dense.compute_basis_derivative(x, grid, spline_order)
    gx = ((D @ W.reshape(O, I * R)).reshape(B, I, R) * dH).sum(2)
    g_base = None
    if _has(base_weight):
        g_base = D.t() @ torch.nn.functional.silu(x)
        sig = torch.sigmoid(x)
        gx = gx + (D @ base_weight) * (sig * (1.0 + x * (1.0 - sig)))
    return gx, g_base, g_spline, g_scaler


# Gradient sinks: a data-parallel host may register, per layer (keyed by the storage of its
# spline_weight), an object that receives the parameter gradients directly -- the backward then
# writes them range by range of output rows into the sink's tensors (no autograd accumulation)
# and tells the sink after each range, so that the all-reduce of one range overlaps the
# computation of the next.  See data_parallel.GradientBucket(direct=True).
_grad_sinks: dict = {}
_sinks_disabled = 0


class no_grad_sinks:
    """Context in which forwards do not use a registered gradient sink: for call sites whose
    parameters also receive gradients from other terms (the fused regulariser)."""

    def __enter__(self):
        global _sinks_disabled
        _sinks_disabled += 1

    def __exit__(self, *exc):
        global _sinks_disabled
        _sinks_disabled -= 1
        return False


def register_grad_sink(spline_weight: torch.Tensor, sink) -> None:
    _grad_sinks[spline_weight.data_ptr()] = sink


def unregister_grad_sink(spline_weight: torch.Tensor) -> None:
    _grad_sinks.pop(spline_weight.data_ptr(), None)


def _sink_backward(ctx, sink, grad_output, x, grid, base_weight, spline_weight, spline_scaler, k, has_scaler):
    """Backward through a gradient sink: ``(True, grad_x | None)``, or ``(False, None)`` when this
    call cannot use it (then nothing has been written)."""
    has_base = _has(base_weight)
    wants_all = ctx.needs_input_grad[3] and (ctx.needs_input_grad[2] or not has_base) and \
        (ctx.needs_input_grad[4] or not has_scaler)
    if not wants_all or x.dtype != torch.float32 or x.size(0) < 1:
        return False, None
    G = grid.size(1) - 2 * k - 1
    mode = _native.resolve_mode(_mode, x.dtype, x.size(0), x.size(1), spline_weight.size(0), G, k)
    if mode not in (_native.MODE_TC_BF16X3, _native.MODE_TC_BF16X1):
        return False, None
    dest = sink.destinations(base_weight if has_base else None, spline_weight, spline_scaler if has_scaler else None)
    if dest is None:
        return False, None
    gb, gs, gc = dest
    _check_inputs(x, grid, base_weight, spline_weight, spline_scaler, k, has_scaler)
    D = _c(grad_output.to(x.dtype))
    xc, gridc, bwc, swc = _c(x), _c(grid), _c(base_weight), _c(spline_weight)
    scc = _c(spline_scaler) if has_scaler else None
    for o0, o1 in sink.row_ranges(spline_weight.size(0)):
        _native.backward_param_rows(D, xc, gridc, bwc, swc, scc, k, o0, o1, gb, gs, gc, mode)
        sink.rows_done(o0, o1)
    gx = None
    if ctx.needs_input_grad[0]:
        gx = _native.backward(D, xc, gridc, bwc, swc, scc, k, True, False, False, False, mode)[0]
    return True, gx


class KANFunction(torch.autograd.Function):
    """Autograd node of the native layer (KANFunction, csrc/kan_autograd.cpp:13-111).

    Saves only the inputs (no basis).  Backward: composite differentiable
    formulas while grad mode is on (``create_graph=True``), native kernels with
    un-needed gradients skipped otherwise.
    """

    @staticmethod
    def forward(ctx, x, grid, base_weight, spline_weight, spline_scaler, spline_order: int, has_scaler: bool):
        ctx.spline_order, ctx.has_scaler = int(spline_order), bool(has_scaler)
        ctx.allow_sink = _sinks_disabled == 0
        y = _forward_impl(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler)
        ctx.save_for_backward(x, grid, base_weight, spline_weight, spline_scaler)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x, grid, base_weight, spline_weight, spline_scaler = ctx.saved_tensors
        k, has_scaler = ctx.spline_order, ctx.has_scaler
        has_base = _has(base_weight)
        if torch.is_grad_enabled():
            gx, gb, gs, gc = kan_backward_composite(grad_output, x, grid, base_weight, spline_weight,
                                                    spline_scaler, k, has_scaler)
        else:
            sink = _grad_sinks.get(spline_weight.data_ptr()) if (_grad_sinks and ctx.allow_sink) else None
            if sink is not None:
                handled, gx = _sink_backward(ctx, sink, grad_output, x, grid, base_weight, spline_weight,
                                             spline_scaler, k, has_scaler)
                if handled:
                    return (gx, None, None, None, None, None, None)
            need_x = ctx.needs_input_grad[0]
            need_base = ctx.needs_input_grad[2] and has_base
            need_spline = ctx.needs_input_grad[3] or (has_scaler and ctx.needs_input_grad[4])
            gx, gb, gs, gc = _backward_impl(grad_output, x, grid, base_weight, spline_weight, spline_scaler, k,
                                            has_scaler, need_x, need_base, need_spline)
        return (gx, None, gb if has_base else None, gs, gc if has_scaler else None, None, None)


def kan_apply(x, grid, base_weight, spline_weight, spline_scaler, spline_order: int, has_scaler: bool) -> torch.Tensor:
    """Autograd-aware forward; the call ``KANLinear`` uses (kan_apply, csrc/kan_autograd.cpp:117-135)."""
    return KANFunction.apply(x, grid, base_weight, spline_weight, spline_scaler, int(spline_order), bool(has_scaler))


def _check_basis_args(x, grid, k: int) -> None:
    if not (x.is_cuda and grid.is_cuda):
        raise RuntimeError("kan_basis: x and grid must be CUDA tensors")
    if x.dim() != 2 or grid.dim() != 2 or grid.size(0) != x.size(1):
        raise RuntimeError("kan_basis: x must be [B, I] and grid [I, G+2k+1]")
    if not 1 <= k <= 3:
        raise RuntimeError("kan_basis: spline_order must be 1, 2 or 3")
    if x.dtype != grid.dtype:
        raise RuntimeError("kan_basis: dtype mismatch")
    if x.dtype not in (torch.float32, torch.float64):
        raise RuntimeError("kan_basis: only FP32/FP64 supported")
    G = grid.size(1) - 2 * k - 1
    if G < 1:
        raise RuntimeError("kan_basis: grid too short")
    if G + 2 * k > CUDA_MAX_DEG0_BASIS:
        raise RuntimeError(f"CUDA kernel supports G + 2k <= {CUDA_MAX_DEG0_BASIS} (got G={G}, k={k})")
    if x.size(1) > CUDA_MAX_IN_FEATURES:
        raise RuntimeError("kan_basis: too many input features")


def basis(x, grid, spline_order: int) -> torch.Tensor:
    """Dense basis ``H [B, I, R]`` (kan_basis_cuda, csrc/kan_cuda.cu:666-680)."""
    _check_basis_args(x, grid, spline_order)
    return _native.basis(x.contiguous(), grid.contiguous(), int(spline_order))


def basis_grad(x, grid, spline_order: int, grad_basis) -> torch.Tensor:
    """``gx[b,i] = sum_r gH[b,i,r] dB_r/dx`` (kan_basis_grad_cuda, csrc/kan_cuda.cu:682-699)."""
    _check_basis_args(x, grid, spline_order)
    G = grid.size(1) - 2 * spline_order - 1
    if grad_basis.dim() != 3 or tuple(grad_basis.shape) != (x.size(0), x.size(1), G + spline_order):
        raise RuntimeError("kan_basis_grad: gH must be [B, I, G+k]")
    return _native.basis_grad(x.contiguous(), grid.contiguous(), int(spline_order),
                              grad_basis.contiguous().to(x.dtype))


def _check_edge(s, H, bw, W, has_base: bool) -> None:
    if not (H.is_cuda and W.is_cuda):
        raise RuntimeError("edge_abs_mean: H and W must be CUDA tensors")
    if H.dim() != 3 or W.dim() != 3:
        raise RuntimeError("edge_abs_mean: H must be [N,I,R], W [O,I,R]")
    if H.size(1) != W.size(1) or H.size(2) != W.size(2):
        raise RuntimeError("edge_abs_mean: H/W shape mismatch")
    if H.size(2) > 72:
        raise RuntimeError(f"edge_abs_mean: R must be <= 72, got {H.size(2)}")
    if H.size(1) > CUDA_MAX_IN_FEATURES:
        raise RuntimeError("edge_abs_mean: too many input features")
    if H.size(0) < 1:
        raise RuntimeError("edge_abs_mean: need at least one sample")
    if H.dtype != W.dtype:
        raise RuntimeError("edge_abs_mean: dtype mismatch")
    if H.dtype not in (torch.float32, torch.float64):
        raise RuntimeError("edge_abs_mean: only FP32/FP64 supported")
    if has_base:
        if tuple(s.shape) != tuple(H.shape[:2]):
            raise RuntimeError("edge_abs_mean: s must be [N, I]")
        if tuple(bw.shape) != tuple(W.shape[:2]):
            raise RuntimeError("edge_abs_mean: base_weight must be [O, I]")
        if s.dtype != H.dtype or bw.dtype != H.dtype:
            raise RuntimeError("edge_abs_mean: dtype mismatch")


def edge_abs_mean(s, H, base_weight, W) -> torch.Tensor:
    """``a[o,i] = mean_n |s bw + <H, W>|`` without phi [N,O,I] (edge_abs_mean_cuda, csrc/kan_reg_cuda.cu:263-280)."""
    has_base = _has(base_weight)
    _check_edge(s, H, base_weight, W, has_base)
    return _native.edge_abs_mean(_c(s) if has_base else None, H.contiguous(),
                                 _c(base_weight) if has_base else None, W.contiguous())


def edge_abs_mean_backward(grad_a, s, H, base_weight, W, need_s: bool, need_H: bool, need_bw: bool, need_W: bool):
    """``(ds|None, dH|None, dbw|None, dW|None)`` (edge_abs_mean_backward_cuda, csrc/kan_reg_cuda.cu:284-312)."""
    has_base = _has(base_weight)
    _check_edge(s, H, base_weight, W, has_base)
    if tuple(grad_a.shape) != tuple(W.shape[:2]):
        raise RuntimeError("edge_abs_mean_backward: grad shape")
    return _native.edge_abs_mean_backward(grad_a.contiguous().to(W.dtype), _c(s) if has_base else None,
                                          H.contiguous(), _c(base_weight) if has_base else None, W.contiguous(),
                                          need_s, need_H, need_bw, need_W)


# ---------------------------------------------------------------------------
# torch.ops.spline_kan.{kan_forward, kan_backward}: same schemas as the
# reference (csrc/kan_ext.cpp:62-75); CUDA and Meta kernels only.
# ---------------------------------------------------------------------------
def _register_torch_ops() -> bool:
    try:
        lib_def = torch.library.Library("spline_kan", "DEF")
    except Exception:
        return False                     # another provider of the namespace is loaded
    lib_def.define("kan_forward(Tensor x, Tensor grid, Tensor base_weight, Tensor spline_weight, "
                   "Tensor spline_scaler, int spline_order, bool has_scaler) -> (Tensor output, Tensor basis)")
    lib_def.define("kan_backward(Tensor grad_output, Tensor x, Tensor grid, Tensor base_weight, "
                   "Tensor spline_weight, Tensor spline_scaler, Tensor basis, int spline_order, bool has_scaler) "
                   "-> (Tensor grad_x, Tensor grad_base_weight, Tensor grad_spline_weight, Tensor grad_spline_scaler)")

    def _bwd_cuda(grad_output, x, grid, base_weight, spline_weight, spline_scaler, basis, spline_order, has_scaler):
        gx, gb, gs, gc = kan_backward(grad_output, x, grid, base_weight, spline_weight, spline_scaler, basis,
                                      spline_order, has_scaler)
        empty = x.new_empty(0)
        return gx, gb if gb is not None else empty, gs, gc if gc is not None else empty

    def _fwd_meta(x, grid, base_weight, spline_weight, spline_scaler, spline_order, has_scaler):
        R = grid.size(1) - spline_order - 1
        return x.new_empty((x.size(0), spline_weight.size(0))), x.new_empty((x.size(0), x.size(1), R))

    def _bwd_meta(grad_output, x, grid, base_weight, spline_weight, spline_scaler, basis, spline_order, has_scaler):
        empty = x.new_empty(0)
        return (x.new_empty(x.shape),
                base_weight.new_empty(base_weight.shape) if base_weight.numel() > 0 else empty,
                spline_weight.new_empty(spline_weight.shape),
                spline_scaler.new_empty(spline_scaler.shape) if has_scaler else empty)

    lib_def.impl("kan_forward", kan_forward, "CUDA")
    lib_def.impl("kan_backward", _bwd_cuda, "CUDA")
    lib_def.impl("kan_forward", _fwd_meta, "Meta")
    lib_def.impl("kan_backward", _bwd_meta, "Meta")
    globals()["_torch_library"] = lib_def          # keep the registration alive
    return True


TORCH_OPS_REGISTERED = _register_torch_ops()
