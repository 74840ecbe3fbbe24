"""Helpers shared by the GPU parity tests (imported, not collected)."""
import math

import numpy as np
import torch

from oracle import kan_oracle as ko


def cuda_ok() -> bool:
    return torch.cuda.is_available()


def dev(t, dtype=None):
    if t is None:
        return None
    a = torch.from_numpy(np.ascontiguousarray(t))
    if dtype is not None:
        a = a.to(dtype)
    return a.cuda()


def make_layer_case(N, I, O, G, k, dtype, seed, nonuniform=False, scaler=True, base=True, xscale=1.15,
                    snap_to_knots=True):
    """Seeded layer inputs/parameters as numpy arrays (dtype-preserving)."""
    rng = np.random.default_rng(seed)
    if nonuniform:
        gaps = rng.uniform(0.1, 1.0, size=(I, G + 2 * k))
        t = np.concatenate([np.zeros((I, 1)), np.cumsum(gaps, 1)], 1)
        t = t - t[:, k:k + 1]
        t = t / t[:, k + G:k + G + 1] * 2.0 - 1.0
        grid = t.astype(dtype)
    else:
        grid = ko.uniform_grid(I, G, k, dtype=dtype)
    x = (rng.uniform(-1, 1, size=(N, I)) * xscale).astype(dtype)
    if snap_to_knots and N >= 8:
        # a share of inputs sits exactly on knots (incl. both domain ends)
        for i in range(I):
            rows = rng.choice(N, size=max(1, N // 6), replace=False)
            x[rows, i] = grid[i, rng.integers(0, grid.shape[1], size=rows.size)]
    R = G + k
    bw = (rng.uniform(-1, 1, size=(O, I)) / math.sqrt(I)).astype(dtype) if base else None
    sw = (rng.uniform(-1, 1, size=(O, I, R)) * 0.3).astype(dtype)
    sc = (rng.uniform(-1, 1, size=(O, I)) / math.sqrt(I) + 0.2).astype(dtype) if scaler else None
    return dict(x=x, grid=grid, bw=bw, sw=sw, sc=sc, k=k)


def oracle_step(case, need_x=True, dtype=np.float64):
    """Oracle forward + backward of sum(y^2) evaluated in float64."""
    c = {n: (None if v is None or isinstance(v, int) else v.astype(dtype)) for n, v in case.items() if n != "k"}
    y, _ = ko.kan_forward(c["x"], c["grid"], c["bw"], c["sw"], c["sc"], case["k"])
    D = 2.0 * y
    gx, gb, gs, gsc = ko.kan_backward(D, c["x"], c["grid"], c["bw"], c["sw"], c["sc"], case["k"])
    return y, D, gx, gb, gs, gsc
