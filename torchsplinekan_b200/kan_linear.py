"""
KANLinear: one B-spline KAN layer with a native B200 backend
(API of spline_kan/kan_linear.py: same constructor, attributes, methods,
state-dict keys and error behaviour).
"""
from __future__ import annotations

import copy
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _C
from . import fused as _fused
from .dense_backend import (ReferenceKANLayer, compute_basis, curve2coeff, edge_abs_mean_dense, fit_spline_coeffs,
                            regularization_from_edge_means)

_CUDA_EXT_LOADED: bool = True            # importing ._C raises when the library is missing
REG_IMPLS = ("auto", "dense", "fused", "checkpoint")
CUDA_MAX_DEG0_BASIS = int(_C.CUDA_MAX_DEG0_BASIS)
CUDA_MAX_IN_FEATURES = int(_C.CUDA_MAX_IN_FEATURES)


def native_config_supported(in_features: int, grid_size: int, spline_order: int) -> Tuple[bool, str]:
    """``(ok, reason)``: whether the native kernels accept a layer shape (kan_linear.py:43-55)."""
    if grid_size + 2 * spline_order > CUDA_MAX_DEG0_BASIS:
        return False, (f"grid_size + 2*spline_order = {grid_size + 2 * spline_order} exceeds the "
                       f"CUDA kernel limit of {CUDA_MAX_DEG0_BASIS}")
    if in_features > CUDA_MAX_IN_FEATURES:
        return False, f"in_features = {in_features} exceeds the CUDA kernel limit of {CUDA_MAX_IN_FEATURES}"
    return True, ""


class KANLinear(nn.Module):
    """
    B-spline KAN layer ``y = base_activation(x) @ base_weight^T + B(x) @ (spline_weight * spline_scaler)^T``.

    Parameters and defaults as in the reference (kan_linear.py:103-117).
    ``backend``: "auto" (native kernels for CUDA inputs when the shape is
    supported, else the dense PyTorch formulation), "cuda" (native only; raises
    on unsupported shapes and CPU inputs) or "reference" (always dense PyTorch).
    The native kernels fuse SiLU; any other base activation is evaluated with
    PyTorch and only the spline branch runs natively.  ``create_graph=True``
    is exact on every backend.
    """

    def __init__(self, in_features: int, out_features: int, grid_size: int = 5, spline_order: int = 3,
                 scale_noise: float = 0.1, scale_base: float = 1.0, scale_spline: float = 1.0,
                 enable_standalone_scale_spline: bool = True, base_activation=nn.SiLU, grid_eps: float = 0.02,
                 grid_range: Tuple[float, float] = (-1.0, 1.0), backend: str = "auto") -> None:
        super().__init__()
        if grid_size < 1:
            raise ValueError(f"grid_size must be >= 1, got {grid_size}")
        if spline_order not in (1, 2, 3):
            raise ValueError(f"spline_order must be 1, 2, or 3, got {spline_order}")
        if backend not in ("auto", "cuda", "reference"):
            raise ValueError(f"backend must be 'auto', 'cuda', or 'reference', got {backend!r}")
        native_ok, why_not = native_config_supported(in_features, grid_size, spline_order)
        if backend == "cuda":
            if not native_ok:
                raise ValueError(f"backend='cuda' does not support this configuration: {why_not}. "
                                 "Use backend='reference' (or 'auto', which falls back automatically).")
            self._use_cuda = True
        elif backend == "reference":
            self._use_cuda = False
        else:
            self._use_cuda = native_ok
        self.backend = backend
        self.last_backend: Optional[str] = None      # plain string: cannot keep a graph alive
        # Inference with fixed parameters (export_inference): the knot table and the weight image of
        # the native kernels are then built once and reused while the parameters stay as they are.
        self.cache_operands = False
        self._operands = None                        # (key, device buffer)

        # The dense layer owns parameters and buffers; they are aliased here so
        # that state dicts carry both key sets, as the reference's do.
        self._ref = ReferenceKANLayer(
            in_features=in_features, out_features=out_features, grid_size=grid_size, spline_order=spline_order,
            scale_noise=scale_noise, scale_base=scale_base, scale_spline=scale_spline,
            enable_standalone_scale_spline=enable_standalone_scale_spline, base_activation=base_activation,
            grid_eps=grid_eps, grid_range=grid_range)
        self.base_weight = self._ref.base_weight
        self.spline_weight = self._ref.spline_weight
        if enable_standalone_scale_spline:
            self.spline_scaler = self._ref.spline_scaler
        self.register_buffer("grid", self._ref.grid)

        self.in_features = in_features
        self.out_features = out_features
        self.grid_size = grid_size
        self.spline_order = spline_order
        self.enable_standalone_scale_spline = enable_standalone_scale_spline

    # -- backend choice ----------------------------------------------------
    @property
    def selected_backend(self) -> str:
        """Backend used for CUDA inputs: "cuda" or "reference"."""
        return "cuda" if self._use_cuda else "reference"

    def backend_for(self, x: torch.Tensor) -> str:
        """Backend :meth:`forward` will use for ``x``."""
        if not self._use_cuda:
            return "reference"
        if self.backend == "cuda" or x.is_cuda:
            return "cuda"
        return "reference"

    @property
    def _native_fuses_base(self) -> bool:
        return type(self._ref.base_activation) is nn.SiLU

    # -- forward -----------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        which = self.backend_for(x)
        self.last_backend = which
        return self._cuda_forward(x) if which == "cuda" else self._ref(x)

    def _cuda_forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("KANLinear with backend='cuda' received a CPU tensor. "
                               "Move the input and model to a CUDA device, or use backend='reference'.")
        lead = x.shape[:-1]
        xf = x.reshape(-1, self.in_features)
        absent = xf.new_empty(0)
        has_scaler = self.enable_standalone_scale_spline
        fuse_base = self._native_fuses_base
        prepared = self._prepared_operands(xf, fuse_base, has_scaler) if self.cache_operands else None
        if prepared is not None:
            out = _C.forward_prepared(xf, prepared, self.out_features, self.grid_size, self.spline_order, fuse_base)
            if not fuse_base:
                out = out + F.linear(self._ref.base_activation(xf), self.base_weight)
            return out.reshape(lead + (self.out_features,))
        out = _C.kan_apply(xf, self.grid, self.base_weight if fuse_base else absent, self.spline_weight,
                           self.spline_scaler if has_scaler else absent, self.spline_order, has_scaler)
        if not fuse_base:
            out = out + F.linear(self._ref.base_activation(xf), self.base_weight)
        return out.reshape(lead + (self.out_features,))

    def _prepared_operands(self, xf: torch.Tensor, fuse_base: bool, has_scaler: bool):
        """The buffer of ``_C.prepare_forward`` for the current parameters, or None when this call
        cannot use it: gradients are wanted, the dtype is not float32, or a call of this shape does not
        run on the tensor cores.  The buffer is rebuilt when a parameter or the knots were modified in
        place (their version counters), replaced, or moved."""
        params = [self.grid, self.spline_weight] + ([self.base_weight] if fuse_base else []) + \
                 ([self.spline_scaler] if has_scaler else [])
        if xf.dtype != torch.float32 or xf.shape[0] == 0:
            return None
        if torch.is_grad_enabled() and (xf.requires_grad or any(p.requires_grad for p in params)):
            return None
        if _C.resolve_mode(xf.shape[0], self.in_features, self.out_features, self.grid_size, self.spline_order,
                           False) not in (2, 3):                 # KANB200_MODE_TC_BF16X3 / _BF16X1
            return None
        key = tuple((p.data_ptr(), p._version, p.device) for p in params)
        if self._operands is None or self._operands[0] != key:
            absent = xf.new_empty(0)
            buf = _C.prepare_forward(self.grid, self.base_weight if fuse_base else absent, self.spline_weight,
                                     self.spline_scaler if has_scaler else absent, self.spline_order, has_scaler)
            self._operands = (key, buf if buf.numel() > 0 else None)
        return self._operands[1]

    # -- knots from data ---------------------------------------------------
    def update_grid(self, x: torch.Tensor, margin: float = 0.01) -> None:
        """Moves the knots to the distribution of ``x`` and refits ``spline_weight``
        (see :meth:`ReferenceKANLayer.update_grid`).

        For CUDA inputs on the native backend the refit stays on the device: per input feature two
        [R, R] moment matrices of the new and old basis at the samples give the matrix that maps old
        coefficients to refitted ones (``kanb200_refit_transfer``), so neither the sampled curves
        [O, B, I] nor a system per (feature, output) is ever formed; only features whose normal
        equations are not safely positive definite (too few distinct samples) take the
        minimum-norm path of the dense backend."""
        xf = x.reshape(-1, self.in_features)
        if not (xf.is_cuda and self.backend_for(xf) == "cuda"):
            self._ref.update_grid(x, margin=margin)
            with torch.no_grad():
                self.grid.copy_(self._ref.grid)
            return
        ref = self._ref
        if margin <= 0:
            raise ValueError(f"margin must be positive, got {margin}")
        if not (0.0 < ref.grid_eps < 1.0):
            raise ValueError(f"grid_eps must be in (0, 1), got {ref.grid_eps}")
        if xf.shape[0] < 2:
            raise ValueError(f"update_grid requires at least 2 samples, got {xf.shape[0]}")
        from . import _native
        with torch.no_grad():
            xs = xf.to(self.grid.dtype)
            knots = ref.grid_from_samples(xs, self.grid_size, margin)
            transfer, info = _native.refit_transfer(xs, self.grid, knots, self.spline_order)
            coeffs = torch.einsum("irs,ois->oir", transfer, self.spline_weight.double())
            weak = torch.nonzero(info != 0).flatten()
            if weak.numel() > 0:
                # minimum-norm refit of the few rank-deficient features, as the dense backend does
                cols = weak.tolist()
                curve = torch.einsum("oir,bir->obi", self.spline_weight[:, cols],
                                     compute_basis(xs[:, cols], self.grid[cols], self.spline_order))
                coeffs[:, cols] = curve2coeff(xs[:, cols], curve, knots[cols], self.spline_order).double()
            self._copy_grid_(knots)
            self.spline_weight.copy_(coeffs.to(self.spline_weight.dtype))

    # -- regularisation ----------------------------------------------------
    def regularization_loss(self, reg_act: float = 1.0, reg_entropy: float = 1.0, *,
                            x: Optional[torch.Tensor] = None, mode: str = "activation",
                            reg_impl: str = "auto", chunk_size: int = 1024, reg_group=None) -> torch.Tensor:
        """Scalar sparsity penalty (kan_linear.py:275-334).  ``mode="activation"`` needs ``x``;
        ``reg_impl`` selects how mean|phi| is evaluated and ``reg_group`` whether the statistic is
        taken over the global batch (see :meth:`forward_with_regularization`)."""
        if mode not in ("activation", "coefficient"):
            raise ValueError(f"mode must be 'activation' or 'coefficient', got {mode!r}")
        if mode == "coefficient":
            return self._ref.regularization_loss(regularize_activation=reg_act, regularize_entropy=reg_entropy,
                                                 mode="coefficient")
        if x is None:
            return self._ref.regularization_loss(reg_act, reg_entropy, x=None)     # canonical error
        xf = x.reshape(-1, self.in_features)
        impl = self._resolve_reg_impl(reg_impl, xf)
        if impl == "fused":
            a = self._across_ranks(self._edge_abs_mean_from_input(xf), xf, reg_group)
            return _fused.penalty_from_edge_means(a, reg_act, reg_entropy)
        s = self._ref.base_activation(xf)
        H = self._basis(xf, impl)
        a = self._edge_abs_mean(xf, s, H, self._ref.effective_spline_weight(), impl, chunk_size)
        return regularization_from_edge_means(self._across_ranks(a, xf, reg_group), reg_act, reg_entropy)

    @staticmethod
    def _across_ranks(a: torch.Tensor, x_flat: torch.Tensor, reg_group) -> torch.Tensor:
        """The edge statistic of the global batch when a process group is given (one all-reduce of
        ``[O, I]`` values, weighted by the ranks' row counts), else ``a`` itself."""
        if reg_group is None:
            return a
        from .data_parallel import global_edge_means
        return global_edge_means(a, x_flat.shape[0], None if reg_group is True else reg_group)

    def forward_with_regularization(self, x: torch.Tensor, reg_act: float = 1.0, reg_entropy: float = 1.0, *,
                                    mode: str = "activation", reg_impl: str = "auto", chunk_size: int = 1024,
                                    reg_group=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(self(x), self.regularization_loss(reg_act, reg_entropy, x=x))`` from one evaluation of the
        base activation and the basis (kan_linear.py:340-389).

        ``reg_impl``: "auto" ("fused" when the native kernels can run, else "dense"), "dense"
        (phi [N,O,I] in PyTorch), "fused" (native kernel, phi never stored, recomputed in backward)
        or "checkpoint" (chunked PyTorch with activation checkpointing).  All give the same value
        and gradients up to rounding and keep the full graph to ``x`` and the parameters.

        ``reg_group`` (no counterpart in the reference, which has no multi-device code): None = the
        statistic of the rows this process holds (with data parallelism every rank then penalises
        its own shard); a ``torch.distributed`` process group, or True for the default group = the
        statistic of the GLOBAL batch, from one all-reduce of ``mean|phi| [O, I]`` weighted by the
        ranks' row counts (:func:`torchsplinekan_b200.global_edge_means`), so that every rank
        evaluates the whole-batch penalty and the reduced parameter gradients are those of the
        unsharded batch.
        """
        if mode == "coefficient":
            # the parameters get gradients from both terms: a data-parallel gradient sink must not
            # take over the layer's backward
            with _C.no_grad_sinks():
                y = self(x)
            return y, self.regularization_loss(reg_act, reg_entropy, mode="coefficient")
        if mode != "activation":
            raise ValueError(f"mode must be 'activation' or 'coefficient', got {mode!r}")
        lead = x.shape[:-1]
        xf = x.reshape(-1, self.in_features)
        impl = self._resolve_reg_impl(reg_impl, xf)
        if impl == "fused":
            # One evaluation of x feeds two native operators and nothing of size [N, I, R] or
            # [N, O, I] is ever stored: y from the layer kernels (kan_apply), the edge statistic
            # from the from-x edge kernels.  The parameters receive gradients from both terms, so a
            # data-parallel gradient sink must not take over the layer's backward.
            with _C.no_grad_sinks():
                y = self._cuda_forward(xf)
            self.last_backend = "cuda"
            a = self._across_ranks(self._edge_abs_mean_from_input(xf), xf, reg_group)
            return y.reshape(lead + (self.out_features,)), _fused.penalty_from_edge_means(a, reg_act, reg_entropy)
        s = self._ref.base_activation(xf)
        H = self._basis(xf, impl)
        W = self._ref.effective_spline_weight()
        y = F.linear(s, self.base_weight) + F.linear(H.reshape(xf.shape[0], -1), W.reshape(self.out_features, -1))
        self.last_backend = "reference"
        a = self._across_ranks(self._edge_abs_mean(xf, s, H, W, impl, chunk_size), xf, reg_group)
        return y.reshape(lead + (self.out_features,)), regularization_from_edge_means(a, reg_act, reg_entropy)

    def _resolve_reg_impl(self, reg_impl: str, x_flat: torch.Tensor) -> str:
        if reg_impl not in REG_IMPLS:
            raise ValueError(f"reg_impl must be one of {REG_IMPLS}, got {reg_impl!r}")
        native_ok = _fused.HAS_FUSED_KERNELS and x_flat.is_cuda and self.backend_for(x_flat) == "cuda"
        if reg_impl == "auto":
            return "fused" if native_ok else "dense"
        if reg_impl == "fused" and not native_ok:
            raise RuntimeError("reg_impl='fused' needs the native CUDA kernels, a CUDA input and a layer "
                               "configuration supported by backend='cuda'.  Use reg_impl='dense' or "
                               "'checkpoint' instead.")
        return reg_impl

    def _edge_abs_mean_from_input(self, x_flat: torch.Tensor) -> torch.Tensor:
        """``a [O, I]`` from the native from-x edge kernels.  With SiLU the kernels evaluate the base
        value (and its derivative) themselves; any other activation is evaluated by PyTorch and its
        values are handed over, so autograd carries the gradient through it."""
        s = None if self._native_fuses_base else self._ref.base_activation(x_flat)
        return _fused.edge_abs_mean_from_input(x_flat, s, self.grid, self.spline_order, self.base_weight,
                                               self._ref.effective_spline_weight())

    def _basis(self, x_flat: torch.Tensor, impl: str) -> torch.Tensor:
        return compute_basis(x_flat, self.grid, self.spline_order)

    def _edge_abs_mean(self, x_flat, s, H, W, impl, chunk_size):
        if impl == "checkpoint":
            if chunk_size < 1:
                raise ValueError(f"chunk_size must be >= 1, got {chunk_size}")
            return _fused.edge_abs_mean_chunked(s, x_flat, self.grid, self.spline_order, self.base_weight, W,
                                                chunk_size)
        return edge_abs_mean_dense(s, H, self.base_weight, W)

    @torch.no_grad()
    def edge_l1(self, x: torch.Tensor) -> torch.Tensor:
        """Per-edge L1 norm ``mean_n |phi_{o,i}(x_n)|`` -> [O, I] (kan_linear.py:451-458)."""
        xf = x.reshape(-1, self.in_features)
        impl = self._resolve_reg_impl("auto", xf)
        if impl == "fused":
            return self._edge_abs_mean_from_input(xf)       # no basis tensor, nothing saved (no_grad)
        s = self._ref.base_activation(xf)
        return self._edge_abs_mean(xf, s, self._basis(xf, impl), self._ref.effective_spline_weight(), impl, 1024)

    # -- construction helpers ---------------------------------------------
    def make_like(self, in_features: Optional[int] = None, out_features: Optional[int] = None,
                  grid_size: Optional[int] = None,
                  enable_standalone_scale_spline: Optional[bool] = None) -> "KANLinear":
        """Freshly initialised layer with this layer's hyper-parameters, dtype and device, optionally
        with another shape (kan_linear.py:424-449)."""
        ref = self._ref
        scaler = self.enable_standalone_scale_spline if enable_standalone_scale_spline is None \
            else enable_standalone_scale_spline
        twin = KANLinear(
            self.in_features if in_features is None else in_features,
            self.out_features if out_features is None else out_features,
            grid_size=self.grid_size if grid_size is None else grid_size, spline_order=self.spline_order,
            scale_noise=ref.scale_noise, scale_base=ref.scale_base, scale_spline=ref.scale_spline,
            enable_standalone_scale_spline=scaler, base_activation=copy.deepcopy(ref.base_activation),
            grid_eps=ref.grid_eps, grid_range=ref.grid_range, backend=self.backend)
        return twin.to(device=self.grid.device, dtype=self.grid.dtype)

    @torch.no_grad()
    def _copy_grid_(self, grid: torch.Tensor) -> None:
        # .to() / .double() re-create buffers per module: keep both copies equal.
        self.grid.copy_(grid)
        self._ref.grid.copy_(grid)

    def export_inference(self, requires_grad: bool = False) -> "KANLinear":
        """Independent layer computing the same function with ``spline_scaler`` folded into the
        coefficients (``enable_standalone_scale_spline=False``); frozen and in eval mode unless
        ``requires_grad`` (kan_linear.py:471-496)."""
        out = self.make_like(enable_standalone_scale_spline=False)
        with torch.no_grad():
            out.base_weight.copy_(self.base_weight)
            out.spline_weight.copy_(self._ref.effective_spline_weight())
            out._copy_grid_(self.grid)
        out.requires_grad_(requires_grad)
        # frozen parameters: the native kernels' knot table and weight image are built at the first
        # call and reused (one launch per layer and call instead of three)
        out.cache_operands = not requires_grad
        return out.train(self.training and requires_grad)

    @torch.no_grad()
    def extend_grid(self, new_grid_size: int, x: torch.Tensor, *, margin: float = 0.01,
                    adapt_knots: bool = False, ridge: float = 1e-12, n_dense: int = 0) -> "KANLinear":
        """NEW layer with ``new_grid_size`` intervals whose coefficients are the least-squares fit of
        this layer's spline curves on ``x`` (plus ``n_dense`` uniform points); base weight, scaler
        and activation are copied.  ``adapt_knots=False`` puts uniform knots over the interior
        domain widened to the sample range, ``True`` uses the quantile/uniform mix of
        :meth:`update_grid` (kan_linear.py:502-588)."""
        if new_grid_size < 1:
            raise ValueError(f"new_grid_size must be >= 1, got {new_grid_size}")
        xf = x.reshape(-1, self.in_features).to(self.grid)
        if xf.shape[0] < 2:
            raise ValueError("extend_grid needs at least 2 samples")
        k = self.spline_order
        fine = self.make_like(grid_size=new_grid_size)
        if adapt_knots:
            knots = fine._ref.grid_from_samples(xf, new_grid_size, margin)
        else:
            lo0, hi0 = self.grid[:, k], self.grid[:, k + self.grid_size]
            xmin, xmax = xf.amin(0), xf.amax(0)
            lo = torch.maximum(torch.where(xmin < lo0, xmin - margin, lo0), self.grid[:, 0])
            hi = torch.minimum(torch.where(xmax > hi0, xmax + margin, hi0), self.grid[:, -1])
            steps = torch.arange(new_grid_size + 2 * k + 1, device=lo.device, dtype=lo.dtype) - k
            knots = lo[:, None] + steps[None] * ((hi - lo) / new_grid_size)[:, None]
        pts = xf
        if n_dense > 0:
            a, b = knots[:, k], knots[:, k + new_grid_size]
            ramp = torch.linspace(0, 1, n_dense, device=a.device, dtype=a.dtype)
            pts = torch.cat([xf, a[None] + ramp[:, None] * (b - a)[None]], 0)
        curve = torch.einsum("oir,bir->obi", self.spline_weight, compute_basis(pts, self.grid, k))
        fine.base_weight.copy_(self.base_weight)
        fine.spline_weight.copy_(fit_spline_coeffs(pts, curve, knots, k, ridge=ridge))
        if self.enable_standalone_scale_spline:
            fine.spline_scaler.copy_(self.spline_scaler)
        fine._copy_grid_(knots)
        return fine.train(self.training)
