"""
Multi-threaded CPU restatement of the reference's pure-PyTorch layer, used ONLY
as the timed CPU baseline of ``bench.py`` (and pinned by the tests).  TEST /
MEASUREMENT INFRASTRUCTURE -- nothing in the shipped package imports it.

The reference's CPU path for this layer is PyTorch itself: a dense Cox-de Boor
basis, two matrix products, and autograd for the backward
(spline_kan/reference_backend.py:32-96, 358-378).  This file restates exactly
that with torch CPU tensors so the baseline uses every host thread the way the
reference would; ``kan_oracle.py`` (numpy) stays the parity checker.
"""
from __future__ import annotations

import torch


def _ratio(num, den):
    ok = den != 0
    return torch.where(ok, num / torch.where(ok, den, torch.ones_like(den)), torch.zeros_like(num))


def compute_basis(x, grid, k):
    """Dense basis [B, I, G+k]; half-open spans, last one closed, 0/0 = 0."""
    xq, t = x.unsqueeze(-1), grid.unsqueeze(0)
    lo, hi = t[..., :-1], t[..., 1:]
    B = torch.cat([((xq >= lo) & (xq < hi))[..., :-1], (xq >= lo[..., -1:]) & (xq <= hi[..., -1:])], -1).to(x.dtype)
    for d in range(1, k + 1):
        m = B.shape[-1] - 1
        B = _ratio(xq - t[..., :m], t[..., d:d + m] - t[..., :m]) * B[..., :m] + \
            _ratio(t[..., d + 1:d + 1 + m] - xq, t[..., d + 1:d + 1 + m] - t[..., 1:1 + m]) * B[..., 1:m + 1]
    return B


def layer_forward(x, grid, base_weight, spline_weight, spline_scaler, k):
    B = x.shape[0]
    O = spline_weight.shape[0]
    W = spline_weight * spline_scaler.unsqueeze(-1) if spline_scaler is not None else spline_weight
    y = compute_basis(x, grid, k).reshape(B, -1) @ W.reshape(O, -1).t()
    if base_weight is not None:
        y = torch.nn.functional.silu(x) @ base_weight.t() + y
    return y


def layer_step_sum_sq(x, grid, base_weight, spline_weight, spline_scaler, k, need_x=False):
    """Forward and autograd backward of loss = sum(y^2); returns (y, gx|None, g_base, g_spline, g_scaler)."""
    params = [p.detach().clone().requires_grad_() if p is not None else None
              for p in (base_weight, spline_weight, spline_scaler)]
    xx = x.detach().clone().requires_grad_(need_x)
    y = layer_forward(xx, grid, params[0], params[1], params[2], k)
    y.square().sum().backward()
    g = [None if p is None else p.grad for p in params]
    return y.detach(), (xx.grad if need_x else None), g[0], g[1], g[2]
