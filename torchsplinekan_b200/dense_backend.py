"""
Dense, fully differentiable PyTorch formulation of the B-spline KAN layer.

Role in this package
--------------------
* ``backend="reference"`` of :class:`~torchsplinekan_b200.KANLinear` (the same
  option the reference project offers; spline_kan/reference_backend.py).
* The differentiable formulas the native path switches to when a backward pass
  is itself being recorded (``create_graph=True``): the CUDA kernels are
  first-order only, exactly like the reference's (csrc/kan_autograd.cpp:65-74).
* Owner of the parameters / buffers, the initialisation scheme and the
  ``update_grid`` procedure, so state dicts and seeds are interchangeable with
  the reference (reference_backend.py:268-493).

Nothing here is on the accelerated path: these functions materialise the dense
[B, I, R] basis and run on whatever device their inputs live on.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


def _safe_ratio(num: torch.Tensor, den: torch.Tensor) -> torch.Tensor:
    """num / den where den != 0, else 0 (the Cox-de Boor "0/0 = 0" rule)."""
    live = den != 0
    return torch.where(live, num / torch.where(live, den, torch.ones_like(den)), torch.zeros_like(num))


def compute_basis(x: torch.Tensor, grid: torch.Tensor, k: int) -> torch.Tensor:
    """B-spline basis values ``[B, I, G + k]`` of ``x [B, I]`` on knot rows ``grid [I, G+2k+1]``.

    Degree-0 functions are indicators of the half-open spans ``[t_r, t_{r+1})``,
    the last span being closed on the right; higher degrees follow the
    Cox-de Boor recurrence with zero-length knot differences contributing zero
    (same conventions as reference_backend.py:32-96).
    """
    if k not in (0, 1, 2, 3):
        raise ValueError(f"spline_order must be 0, 1, 2, or 3, got {k}")
    xq = x.unsqueeze(-1)
    t = grid.unsqueeze(0)
    lo, hi = t[..., :-1], t[..., 1:]
    inside = (xq >= lo) & (xq < hi)
    closing = (xq >= lo[..., -1:]) & (xq <= hi[..., -1:])
    B = torch.cat([inside[..., :-1], closing], dim=-1).to(x.dtype)
    for d in range(1, k + 1):
        m = B.shape[-1] - 1
        left = _safe_ratio(xq - t[..., :m], t[..., d:d + m] - t[..., :m])
        right = _safe_ratio(t[..., d + 1:d + 1 + m] - xq, t[..., d + 1:d + 1 + m] - t[..., 1:1 + m])
        B = left * B[..., :m] + right * B[..., 1:m + 1]
    return B


def compute_basis_derivative(x: torch.Tensor, grid: torch.Tensor, k: int) -> torch.Tensor:
    """``dB_{r,k}/dx = k (B_{r,k-1}/(t_{r+k}-t_r) - B_{r+1,k-1}/(t_{r+k+1}-t_{r+1}))``, itself differentiable.

    Same conventions as :func:`compute_basis` (reference_backend.py:99-125).
    """
    if k < 1:
        raise ValueError("compute_basis_derivative requires spline_order >= 1")
    lower = compute_basis(x, grid, k - 1)
    R = grid.shape[1] - k - 1
    t = grid.unsqueeze(0)
    a = _safe_ratio(lower[..., :R], (t[..., k:k + R] - t[..., :R]).expand_as(lower[..., :R]))
    b = _safe_ratio(lower[..., 1:R + 1], (t[..., k + 1:k + 1 + R] - t[..., 1:1 + R]).expand_as(lower[..., 1:R + 1]))
    return k * (a - b)


def edge_abs_mean_dense(s: Optional[torch.Tensor], H: torch.Tensor,
                        base_weight: Optional[torch.Tensor], eff_weight: torch.Tensor) -> torch.Tensor:
    """``a[o,i] = mean_n |s[n,i] bw[o,i] + sum_r H[n,i,r] W[o,i,r]|`` via the dense phi [N, O, I].

    Differentiable to any order (reference_backend.py:128-146).
    """
    phi = torch.einsum("oir,nir->noi", eff_weight, H)
    if base_weight is not None:
        phi = s.unsqueeze(1) * base_weight.unsqueeze(0) + phi
    return phi.abs().mean(dim=0)


def regularization_from_edge_means(a: torch.Tensor, regularize_activation: float,
                                   regularize_entropy: float) -> torch.Tensor:
    """``mu1 * A + mu2 * S`` with ``A = sum a``, ``p = a / A``, ``S = -sum p log p``.

    Clamped at the dtype's smallest normal so that an all-zero layer gives a
    zero loss with finite gradients (reference_backend.py:149-170).
    """
    tiny = torch.finfo(a.dtype).tiny
    total = a.sum()
    p = a / total.clamp(min=tiny)
    p = p.clamp(min=tiny)
    entropy = -(p * p.log()).sum()
    return regularize_activation * total + regularize_entropy * entropy


def fit_spline_coeffs(x_samples: torch.Tensor, y_samples: torch.Tensor, grid: torch.Tensor, k: int,
                      ridge: float = 1e-12) -> torch.Tensor:
    """Batched ridge-regularised least squares ``[O, B, I] -> [O, I, R]`` in float64.

    Normal equations per input feature with ``lam = ridge * trace(A^T A) / R``;
    on a failed Cholesky ``lam`` grows by 1e3 (up to four tries) before a general
    solve (reference_backend.py:173-215).
    """
    if ridge <= 0:
        raise ValueError(f"ridge must be positive, got {ridge}")
    A = compute_basis(x_samples.double(), grid.double(), k)
    Y = y_samples.double()
    R = A.shape[-1]
    gram = torch.einsum("bir,bis->irs", A, A)
    rhs = torch.einsum("bir,obi->iro", A, Y)
    scale = gram.diagonal(dim1=-2, dim2=-1).sum(-1).clamp(min=1e-300) / R
    eye = torch.eye(R, dtype=torch.float64, device=A.device)
    lam = ridge
    sol = None
    for _ in range(4):
        M = gram + (lam * scale)[:, None, None] * eye
        L, info = torch.linalg.cholesky_ex(M)
        if not bool((info != 0).any()):
            sol = torch.cholesky_solve(rhs, L)
            break
        lam *= 1e3
    if sol is None:
        sol = torch.linalg.lstsq(M, rhs).solution
    return sol.permute(2, 0, 1).to(dtype=x_samples.dtype)


def curve2coeff(x_samples: torch.Tensor, y_samples: torch.Tensor, grid: torch.Tensor, k: int) -> torch.Tensor:
    """Least-squares spline coefficients ``[O, I, R]`` reproducing ``y_samples [O, B, I]`` at ``x_samples [B, I]``.

    One system ``A_i [B, R] c = Y_i [B, O]`` per input feature, solved in float64 with LAPACK's
    minimum-norm least squares in one batched call (reference_backend.py:218-265 solves the same
    systems in a Python loop).  For samples on a GPU the systems are first reduced there:
    ``A_i = Q_i R_i`` (Householder QR), ``Z_i = Q_i^T Y_i``; ``min |A c - Y| = min |R c - Z|`` has the
    same minimisers and the same singular values, so the small ``[R, R]`` systems that go to the
    CPU give the same minimum-norm solution while ``B / R`` times fewer bytes cross the bus.
    """
    A = compute_basis(x_samples, grid, k).permute(1, 0, 2).contiguous()                   # [I, B, R]
    n_feat, n_samp, n_coef = A.shape
    n_out = y_samples.shape[0]
    if n_samp < n_coef:
        # Fewer samples than coefficients: a wide system with many exact zeros.  LAPACK's default
        # driver (pivoted QR, the one the reference calls) misjudges the rank of such matrices and
        # returns vectors that do not even satisfy the equations (checked: residual of order one on a
        # block-structured 4 x 8 system that the SVD driver solves to 1e-15), so the SVD-based
        # minimum-norm driver is used here, on the CPU, for CPU and CUDA samples alike.
        Y = y_samples.permute(2, 1, 0).contiguous().to(torch.float64)
        sol = torch.linalg.lstsq(A.to(torch.float64).cpu(), Y.cpu(), driver="gelsd").solution
        return sol.permute(2, 0, 1).contiguous().to(dtype=x_samples.dtype, device=x_samples.device)
    if not A.is_cuda:
        Y = y_samples.permute(2, 1, 0).contiguous().to(torch.float64)                      # [I, B, O]
        sol = torch.linalg.lstsq(A.to(torch.float64), Y).solution                          # [I, R, O]
        return sol.permute(2, 0, 1).contiguous().to(dtype=x_samples.dtype)
    Q, Rm = torch.linalg.qr(A.to(torch.float64))                                           # [I, B, R], [I, R, R]
    Z = torch.empty((n_feat, n_coef, n_out), dtype=torch.float64, device=A.device)
    # Q^T Y in slabs of features, so that the float64 copy of Y stays below ~512 MB
    step = max(1, int((1 << 26) // max(1, n_samp * n_out)))
    for lo in range(0, n_feat, step):
        hi = min(n_feat, lo + step)
        Yc = y_samples[:, :, lo:hi].permute(2, 1, 0).to(torch.float64)                     # [i, B, O]
        Z[lo:hi] = torch.bmm(Q[lo:hi].transpose(1, 2), Yc)
    # the rank cut-off LAPACK would have applied to the tall systems
    rcond = torch.finfo(torch.float64).eps * max(n_samp, n_coef)
    sol = torch.linalg.lstsq(Rm.cpu(), Z.cpu(), rcond=rcond).solution                      # [I, R, O]
    return sol.permute(2, 0, 1).contiguous().to(dtype=x_samples.dtype, device=x_samples.device)


class ReferenceKANLayer(nn.Module):
    """Pure-PyTorch B-spline KAN layer; owns parameters, knots and their update.

    Same constructor, attributes, initialisation and state-dict keys as the
    reference class of that name (reference_backend.py:268-352).
    """

    def __init__(self, in_features: int, out_features: int, grid_size: int = 5, spline_order: int = 3,
                 scale_noise: float = 0.1, scale_base: float = 1.0, scale_spline: float = 1.0,
                 enable_standalone_scale_spline: bool = True, base_activation: nn.Module = nn.SiLU,
                 grid_eps: float = 0.02, grid_range: Tuple[float, float] = (-1.0, 1.0)) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.grid_size = grid_size
        self.spline_order = spline_order
        self.scale_noise = scale_noise
        self.scale_base = scale_base
        self.scale_spline = scale_spline
        self.enable_standalone_scale_spline = enable_standalone_scale_spline
        self.grid_eps = grid_eps
        self.grid_range = grid_range
        self.base_activation = base_activation() if isinstance(base_activation, type) else base_activation

        self.register_buffer("grid", self._build_uniform_grid(grid_range[0], grid_range[1]))
        R = grid_size + spline_order
        self.base_weight = nn.Parameter(torch.empty(out_features, in_features))
        self.spline_weight = nn.Parameter(torch.empty(out_features, in_features, R))
        if enable_standalone_scale_spline:
            self.spline_scaler = nn.Parameter(torch.empty(out_features, in_features))
        self.reset_parameters()

    def _build_uniform_grid(self, a: float, b: float) -> torch.Tensor:
        """``t_r = a + (r - k)(b - a)/G`` for r = 0..G+2k, one row per input feature (float32)."""
        G, k = self.grid_size, self.spline_order
        steps = torch.arange(G + 2 * k + 1, dtype=torch.float32)
        knots = a + (steps - k) * (b - a) / G
        return knots.unsqueeze(0).expand(self.in_features, -1).contiguous()

    def reset_parameters(self) -> None:
        """Kaiming-uniform base weights, U(-1,1) * scale_noise / sqrt(R) spline noise, constant scaler."""
        nn.init.kaiming_uniform_(self.base_weight, a=math.sqrt(5))
        R = self.grid_size + self.spline_order
        with torch.no_grad():
            self.base_weight.mul_(self.scale_base)
            noise = (torch.rand_like(self.spline_weight) - 0.5) * 2.0
            self.spline_weight.copy_(noise * self.scale_noise / math.sqrt(R))
            if self.enable_standalone_scale_spline:
                self.spline_scaler.fill_(self.scale_spline)

    def effective_spline_weight(self) -> torch.Tensor:
        """``spline_weight * spline_scaler[..., None]`` (or ``spline_weight`` without scaler)."""
        if self.enable_standalone_scale_spline:
            return self.spline_weight * self.spline_scaler.unsqueeze(-1)
        return self.spline_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        xf = x.reshape(-1, self.in_features)
        H = compute_basis(xf, self.grid, self.spline_order)
        W = self.effective_spline_weight()
        y = F.linear(self.base_activation(xf), self.base_weight) + \
            F.linear(H.reshape(xf.shape[0], -1), W.reshape(self.out_features, -1))
        return y.reshape(lead + (self.out_features,))

    # -- knots from data ---------------------------------------------------
    @torch.no_grad()
    def grid_from_samples(self, x_flat: torch.Tensor, G: int, margin: float = 0.01) -> torch.Tensor:
        """Knot rows ``[I, G+2k+1]`` adapted to the samples.

        G+1 interior points blend sample quantiles with a uniform partition of
        the margin-widened data range (weight ``grid_eps`` on the uniform part);
        k outer knots per side continue with spacing (range / G)
        (reference_backend.py:384-439).
        """
        B = x_flat.shape[0]
        k, eps = self.spline_order, self.grid_eps
        dtype, device = x_flat.dtype, x_flat.device
        ordered = x_flat.sort(dim=0).values
        lo = ordered[0] - margin
        hi = ordered[-1] + margin
        ramp = torch.linspace(0.0, 1.0, G + 1, device=device, dtype=dtype)
        uniform = lo.unsqueeze(0) + ramp.unsqueeze(-1) * (hi - lo).unsqueeze(0)
        fractions = (torch.arange(G + 1, dtype=dtype, device=device) * ((1.0 - eps) / G) + eps / 2.0).clamp(0.0, 1.0)
        pos = fractions * (B - 1)
        below = pos.long().clamp(0, B - 1)
        above = (below + 1).clamp(0, B - 1)
        w = (pos - below.to(dtype)).unsqueeze(-1)
        quantile = (1.0 - w) * ordered[below] + w * ordered[above]
        interior = (1.0 - eps) * quantile + eps * uniform
        step = (hi - lo) / G
        down = torch.arange(k, 0, -1, device=device, dtype=dtype)
        up = torch.arange(1, k + 1, device=device, dtype=dtype)
        left = interior[0].unsqueeze(0) - down.unsqueeze(-1) * step.unsqueeze(0)
        right = interior[-1].unsqueeze(0) + up.unsqueeze(-1) * step.unsqueeze(0)
        return torch.cat([left, interior, right], dim=0).t().contiguous()

    @torch.no_grad()
    def update_grid(self, x: torch.Tensor, margin: float = 0.01) -> None:
        """Moves the knots to the sample distribution and refits ``spline_weight`` to the old
        (unscaled) spline curves at the samples; scaler and base weight are untouched.  New knots
        and coefficients are both computed before either is written
        (reference_backend.py:442-493)."""
        if margin <= 0:
            raise ValueError(f"margin must be positive, got {margin}")
        if not (0.0 < self.grid_eps < 1.0):
            raise ValueError(f"grid_eps must be in (0, 1), got {self.grid_eps}")
        xf = x.reshape(-1, self.in_features)
        if xf.shape[0] < 2:
            raise ValueError(f"update_grid requires at least 2 samples, got {xf.shape[0]}")
        k = self.spline_order
        curve = torch.einsum("oir,bir->obi", self.spline_weight, compute_basis(xf, self.grid, k))
        knots = self.grid_from_samples(xf, self.grid_size, margin)
        coeffs = curve2coeff(xf, curve, knots, k)
        self.grid.copy_(knots)
        self.spline_weight.copy_(coeffs)

    # -- regularisation ----------------------------------------------------
    def regularization_loss(self, regularize_activation: float = 1.0, regularize_entropy: float = 1.0, *,
                            x: Optional[torch.Tensor] = None, mode: str = "activation") -> torch.Tensor:
        """Scalar sparsity penalty; ``mode="activation"`` (needs ``x``) or the legacy ``"coefficient"``
        (reference_backend.py:499-552)."""
        if mode not in ("activation", "coefficient"):
            raise ValueError(f"mode must be 'activation' or 'coefficient', got {mode!r}")
        if mode == "coefficient":
            return self._regularization_coefficient(regularize_activation, regularize_entropy)
        if x is None:
            raise ValueError(
                "regularization_loss with mode='activation' requires x. "
                "Pass the layer's input samples as x=<tensor>, or use "
                "mode='coefficient' for the legacy coefficient-based loss.")
        xf = x.reshape(-1, self.in_features)
        a = edge_abs_mean_dense(self.base_activation(xf), compute_basis(xf, self.grid, self.spline_order),
                                self.base_weight, self.effective_spline_weight())
        return regularization_from_edge_means(a, regularize_activation, regularize_entropy)

    def _regularization_coefficient(self, regularize_activation: float, regularize_entropy: float) -> torch.Tensor:
        """Mean |scaled coefficient| per edge, entropy normalised per output node
        (reference_backend.py:586-617)."""
        per_edge = self.effective_spline_weight().abs().mean(dim=-1)
        share = per_edge / per_edge.sum(dim=-1, keepdim=True).clamp(min=1e-8)
        share = share.clamp(min=1e-8)
        return regularize_activation * per_edge.sum() + regularize_entropy * (-(share * share.log()).sum())
