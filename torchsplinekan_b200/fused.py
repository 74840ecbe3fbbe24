"""
Autograd wrappers around the native basis and edge-statistic kernels
(counterpart of spline_kan/fused.py).

``EdgeAbsMean`` evaluates ``a[o,i] = mean_n |s[n,i] bw[o,i] + sum_r H[n,i,r] W[o,i,r]|``
without storing phi [N, O, I]; its backward recomputes phi to obtain sign(phi).
``NativeBasis`` evaluates H natively and contracts the incoming gradient with
dB/dx in registers.  When the backward is itself being recorded
(``create_graph=True``) both switch to dense differentiable PyTorch formulas
written in terms of the saved inputs, so higher-order derivatives stay exact.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _C
from .dense_backend import compute_basis, compute_basis_derivative, edge_abs_mean_dense

HAS_FUSED_KERNELS = bool(_C.HAS_FUSED_KERNELS)


class NativeBasis(torch.autograd.Function):
    """``H = basis(x) [B, I, R]`` from the native kernel (spline_kan/fused.py:43-61)."""

    @staticmethod
    def forward(ctx, x, grid, k: int):
        ctx.k = k
        ctx.save_for_backward(x, grid)
        return _C.basis(x, grid, k)

    @staticmethod
    def backward(ctx, gH):
        x, grid = ctx.saved_tensors
        if not ctx.needs_input_grad[0]:
            return None, None, None
        if torch.is_grad_enabled():
            return (gH * compute_basis_derivative(x, grid, ctx.k)).sum(-1), None, None
        return _C.basis_grad(x.contiguous(), grid, ctx.k, gH.contiguous()), None, None


class EdgeAbsMean(torch.autograd.Function):
    """Per-edge mean |phi| without the [N, O, I] tensor (spline_kan/fused.py:64-102)."""

    @staticmethod
    def forward(ctx, s, H, bw, W):
        has_base = bw is not None
        none = H.new_empty(0)
        ctx.has_base = has_base
        ctx.save_for_backward(s if has_base else none, H, bw if has_base else none, W)
        return _C.edge_abs_mean(s if has_base else none, H, bw if has_base else none, W)

    @staticmethod
    def backward(ctx, ga):
        s, H, bw, W = ctx.saved_tensors
        has_base = ctx.has_base
        need_s, need_H, need_bw, need_W = ctx.needs_input_grad
        if torch.is_grad_enabled():
            # Partial derivatives written in the saved tensors themselves, so mixed
            # second derivatives (e.g. d(dbw)/ds) survive; sign(0) = 0 as in |.|'s subgradient.
            phi = torch.einsum("oir,nir->noi", W, H)
            if has_base:
                phi = s.unsqueeze(1) * bw.unsqueeze(0) + phi
            g = phi.sign() * ga.unsqueeze(0) / H.shape[0]
            return ((g * bw.unsqueeze(0)).sum(1) if need_s and has_base else None,
                    torch.einsum("noi,oir->nir", g, W) if need_H else None,
                    (g * s.unsqueeze(1)).sum(0) if need_bw and has_base else None,
                    torch.einsum("noi,nir->oir", g, H) if need_W else None)
        ds, dH, dbw, dW = _C.edge_abs_mean_backward(ga, s, H, bw, W, bool(need_s and has_base), bool(need_H),
                                                    bool(need_bw and has_base), bool(need_W))
        return (ds if need_s and has_base else None, dH if need_H else None,
                dbw if need_bw and has_base else None, dW if need_W else None)


class EdgeAbsMeanX(torch.autograd.Function):
    """Per-edge mean |phi| straight from the layer input: ``a = mean_n |s bw + <B(x), W>|`` with
    neither phi [N, O, I] nor the basis [N, I, R] stored, forward or backward (the reference builds
    it from NativeBasis + EdgeAbsMean, spline_kan/kan_linear.py:381-416, and keeps H for backward).

    ``s``: the layer's base values ``base_activation(x)`` as a tensor, or None when the activation
    is SiLU (the kernels then evaluate it, and its derivative, themselves).
    """

    @staticmethod
    def forward(ctx, x, s, grid, k, bw, W):
        none = x.new_empty(0)
        ctx.k, ctx.has_s, ctx.has_base = int(k), s is not None, bw is not None
        ctx.save_for_backward(x, s if s is not None else none, grid, bw if bw is not None else none, W)
        return _C.edge_abs_mean_x(x, s if s is not None else none, grid, bw if bw is not None else none, W, int(k))

    @staticmethod
    def backward(ctx, ga):
        x, s, grid, bw, W = ctx.saved_tensors
        need_x, need_s, _, _, need_bw, need_W = ctx.needs_input_grad
        has_s, has_base = ctx.has_s, ctx.has_base
        if torch.is_grad_enabled():
            # dense differentiable formulas in the saved inputs themselves (create_graph=True)
            H = compute_basis(x, grid, ctx.k)
            sv = (s if has_s else torch.nn.functional.silu(x)) if has_base else None
            phi = torch.einsum("oir,nir->noi", W, H)
            if has_base:
                phi = sv.unsqueeze(1) * bw.unsqueeze(0) + phi
            g = phi.sign() * ga.unsqueeze(0) / x.shape[0]
            gx = gs = None
            if need_x:
                gx = (torch.einsum("noi,oir->nir", g, W) * compute_basis_derivative(x, grid, ctx.k)).sum(-1)
                if has_base and not has_s:
                    sig = torch.sigmoid(x)
                    gx = gx + (g * bw.unsqueeze(0)).sum(1) * (sig * (1.0 + x * (1.0 - sig)))
            if need_s and has_s:
                gs = (g * bw.unsqueeze(0)).sum(1)
            return (gx, gs, None, None, (g * sv.unsqueeze(1)).sum(0) if need_bw and has_base else None,
                    torch.einsum("noi,nir->oir", g, H) if need_W else None)
        gx, ds, dbw, dW = _C.edge_abs_mean_x_backward(ga, x, s, grid, bw, W, ctx.k, bool(need_x),
                                                      bool(need_s and has_s), bool(need_bw and has_base), bool(need_W))
        return (gx if need_x else None, ds if (need_s and has_s) else None, None, None,
                dbw if (need_bw and has_base) else None, dW if need_W else None)


class PenaltyFromEdgeMeans(torch.autograd.Function):
    """``mu1 * A + mu2 * S`` with ``A = sum a``, ``p = a / A``, ``S = -sum p log p`` (the scalar head of the
    activation regulariser, reference_backend.py:149-170) with its gradient in closed form,
    ``d/da_j = mu1 - mu2 (log p_j + S) / A``: on a GPU one launch of the native library gives value and
    gradient (kanb200_edge_penalty) instead of the twenty-odd launches the chain rule through clamp / div /
    log / mul / sum needs; elsewhere a handful of tensor operations.  The backward is written with differentiable
    operations, so higher-order derivatives work.  Same clamps as the dense formulation: ``A`` and
    ``p`` at the dtype's smallest normal (entries clamped there get no entropy gradient)."""

    @staticmethod
    def forward(ctx, a, mu1, mu2):
        ctx.mu = (float(mu1), float(mu2))
        if a.is_cuda and a.dtype in (torch.float32, torch.float64) and a.numel() > 0:
            # value and closed-form gradient from one launch of the native library
            value, ga = _C.edge_penalty(a, float(mu1), float(mu2))
            ctx.save_for_backward(a, ga)
            return value
        tiny = torch.finfo(a.dtype).tiny
        total = a.sum()
        p = (a / total.clamp(min=tiny)).clamp(min=tiny)
        logp = p.log()
        entropy = -(p * logp).sum()
        ctx.save_for_backward(a, None)
        return mu1 * total + mu2 * entropy

    @staticmethod
    def backward(ctx, g):
        a, ga_native = ctx.saved_tensors
        mu1, mu2 = ctx.mu
        if torch.is_grad_enabled():                       # create_graph: let autograd differentiate the plain formula
            with torch.enable_grad():
                a_ = a.detach().requires_grad_(True) if not a.requires_grad else a
                tiny = torch.finfo(a.dtype).tiny
                total = a_.sum()
                p = (a_ / total.clamp(min=tiny)).clamp(min=tiny)
                val = mu1 * total + mu2 * (-(p * p.log()).sum())
                (ga,) = torch.autograd.grad(val, a_, g, create_graph=True)
            return ga, None, None
        if ga_native is not None:
            return g * ga_native, None, None
        tiny = torch.finfo(a.dtype).tiny
        total = a.sum()
        safe = total.clamp(min=tiny)
        q = a / safe
        p = q.clamp(min=tiny)
        logp = p.log()
        entropy = -(p * logp).sum()
        # entries clamped at `tiny` only feel the entropy through A: mu2 (1 - S) / A; with A itself
        # clamped (an all-zero layer) nothing but mu1 is left
        dead = mu1 + mu2 * (1.0 - entropy) / safe * (total >= tiny)
        ga = torch.where(q >= tiny, mu1 - mu2 * (logp + entropy) / safe, dead)
        return g * ga, None, None


def penalty_from_edge_means(a: torch.Tensor, mu1: float, mu2: float) -> torch.Tensor:
    return PenaltyFromEdgeMeans.apply(a, mu1, mu2)


def edge_abs_mean_from_input(x: torch.Tensor, s: Optional[torch.Tensor], grid: torch.Tensor, k: int,
                             bw: Optional[torch.Tensor], W: torch.Tensor) -> torch.Tensor:
    return EdgeAbsMeanX.apply(x, s, grid, k, bw, W)


def native_basis(x: torch.Tensor, grid: torch.Tensor, k: int) -> torch.Tensor:
    return NativeBasis.apply(x, grid, k)


def edge_abs_mean(s: Optional[torch.Tensor], H: torch.Tensor, bw: Optional[torch.Tensor],
                  W: torch.Tensor) -> torch.Tensor:
    return EdgeAbsMean.apply(s, H, bw, W)


def edge_abs_mean_chunked(s: Optional[torch.Tensor], x: torch.Tensor, grid: torch.Tensor, k: int,
                          bw: Optional[torch.Tensor], W: torch.Tensor, chunk_size: int) -> torch.Tensor:
    """Pure-PyTorch low-memory variant: per-chunk phi, recomputed in backward through activation
    checkpointing (spline_kan/fused.py:114-137).  Any device, any derivative order."""
    from torch.utils.checkpoint import checkpoint

    N = x.shape[0]

    def weighted(xc, sc, bw_, W_):
        return edge_abs_mean_dense(sc, compute_basis(xc, grid, k), bw_, W_) * xc.shape[0]

    total = None
    for start in range(0, N, chunk_size):
        xc = x[start:start + chunk_size]
        sc = s[start:start + chunk_size] if s is not None else None
        part = checkpoint(weighted, xc, sc, bw, W, use_reentrant=False)
        total = part if total is None else total + part
    return total / N
