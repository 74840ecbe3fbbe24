"""Pins the numpy oracle against outputs of the real reference (tests/golden/*.npz)."""
import numpy as np
import pytest

from conftest import load_golden, rel_err
from oracle import kan_oracle as ko


def _names(z):
    return [str(n) for n in z["names"]]


def test_basis_matches_reference():
    z = load_golden("basis.npz")
    for name in _names(z):
        k = int(name[1])
        x, grid = z[name + "/x"], z[name + "/grid"]
        H = ko.compute_basis(x, grid, k)
        dH = ko.compute_basis_derivative(x, grid, k)
        assert np.abs(H - z[name + "/H"]).max() <= 1e-14, name
        assert np.abs(dH - z[name + "/dH"]).max() <= 1e-12 * max(1.0, np.abs(z[name + "/dH"]).max()), name


def test_layer_forward_backward_matches_reference():
    z = load_golden("layer.npz")
    for name in _names(z):
        x, grid = z[name + "/x"], z[name + "/grid"]
        bw, sw = z[name + "/base_weight"], z[name + "/spline_weight"]
        sc = z[name + "/spline_scaler"] if name + "/spline_scaler" in z.files else None
        k = int(z[name + "/k"])
        y, gx, gb, gs, gsc = ko.layer_step_sum_sq(x, grid, bw, sw, sc, k, need_x=True)
        tol = 1e-12 if x.dtype == np.float64 else 2e-6
        assert rel_err(y, z[name + "/y"]) < tol, name
        assert rel_err(gx, z[name + "/gx"]) < tol, name
        assert rel_err(gb, z[name + "/g_base_weight"]) < tol, name
        assert rel_err(gs, z[name + "/g_spline_weight"]) < tol, name
        if sc is not None:
            assert rel_err(gsc, z[name + "/g_spline_scaler"]) < tol, name


def test_regulariser_matches_reference():
    z = load_golden("reg.npz")
    for name in _names(z):
        s, H, bw, W = (z[name + "/" + n] for n in ("s", "H", "bw", "W"))
        tol = 1e-12 if H.dtype == np.float64 else 2e-6
        a = ko.edge_abs_mean(s, H, bw, W, chunk=16)
        assert rel_err(a, z[name + "/a"]) < tol, name
        assert rel_err(ko.edge_abs_mean(None, H, None, W), z[name + "/a_nobase"]) < tol, name
        ds, dH, dbw, dW = ko.edge_abs_mean_backward(z[name + "/ga"], s, H, bw, W, chunk=16)
        for got, key in ((ds, "ds"), (dH, "dH"), (dbw, "dbw"), (dW, "dW")):
            assert rel_err(got, z[name + "/" + key]) < tol, (name, key)
        reg = ko.regularization_from_edge_means(z[name + "/a"], 0.7, 1.3)
        assert abs(float(reg) - float(z[name + "/reg_from_a"])) <= tol * abs(float(reg)), name
        assert rel_err(ko.regularization_grad_a(z[name + "/a"], 0.7, 1.3), z[name + "/dreg_da"]) < 10 * tol, name


def test_forward_with_regularization_matches_reference():
    """y, reg and all gradients of loss = sum(y^2) + reg, assembled from oracle pieces."""
    z = load_golden("reg.npz")
    for name in _names(z):
        x, grid = z[name + "/x"], z[name + "/grid"]
        bw, sw = z[name + "/base_weight"], z[name + "/spline_weight"]
        sc = z[name + "/spline_scaler"] if name + "/spline_scaler" in z.files else None
        k = int(z[name + "/k"])
        tol = 1e-11 if x.dtype == np.float64 else 5e-6
        y, gx, gb, gs, gsc = ko.layer_step_sum_sq(x, grid, bw, sw, sc, k, need_x=True)
        H = ko.compute_basis(x, grid, k)
        s = ko.silu(x)
        W = ko.effective_weight(sw, sc)
        a = ko.edge_abs_mean(s, H, bw, W)
        reg = ko.regularization_from_edge_means(a, 0.7, 1.3)
        ga = ko.regularization_grad_a(a, 0.7, 1.3)
        ds, dH, dbw, dW = ko.edge_abs_mean_backward(ga, s, H, bw, W)
        gx = gx + ds * ko.silu_grad(x) + (dH * ko.compute_basis_derivative(x, grid, k)).sum(-1)
        gb = gb + dbw
        if sc is not None:
            gs = gs + dW * sc[:, :, None]
            gsc = gsc + (dW * sw).sum(-1)
        else:
            gs = gs + dW
        assert rel_err(y, z[name + "/fwr_y"]) < tol, name
        assert abs(float(reg) - float(z[name + "/fwr_reg"])) <= tol * abs(float(reg)), name
        assert rel_err(gx, z[name + "/fwr_gx"]) < tol, name
        assert rel_err(gb, z[name + "/fwr_g_base_weight"]) < tol, name
        assert rel_err(gs, z[name + "/fwr_g_spline_weight"]) < tol, name
        if sc is not None:
            assert rel_err(gsc, z[name + "/fwr_g_spline_scaler"]) < tol, name


def test_config0_matches_reference():
    z = load_golden("config0.npz")
    x, target = z["x"], z["target"]
    h = x
    acts = []
    for li in range(2):
        acts.append(h)
        h, _ = ko.kan_forward(h, z[f"l{li}/grid"], z[f"l{li}/base_weight"], z[f"l{li}/spline_weight"],
                              z[f"l{li}/spline_scaler"], 3)
    assert rel_err(h, z["y"]) < 2e-6
    D = (2.0 * (h - target) / h.size).astype(np.float32)
    for li in (1, 0):
        gx, gb, gs, gsc = ko.kan_backward(D, acts[li], z[f"l{li}/grid"], z[f"l{li}/base_weight"],
                                          z[f"l{li}/spline_weight"], z[f"l{li}/spline_scaler"], 3)
        assert rel_err(gb, z[f"l{li}/g_base_weight"]) < 5e-6
        assert rel_err(gs, z[f"l{li}/g_spline_weight"]) < 5e-6
        assert rel_err(gsc, z[f"l{li}/g_spline_scaler"]) < 5e-6
        D = gx


def test_uniform_grid_matches_reference_layout():
    z = load_golden("config0.npz")
    assert np.array_equal(ko.uniform_grid(16, 5, 3), z["l0/grid"])


def test_torch_cpu_baseline_matches_reference():
    """The multi-threaded CPU baseline timed by bench.py is pinned to the same golden vectors."""
    import torch
    from oracle import kan_oracle_torch as kt
    z = load_golden("layer.npz")
    for name in _names(z):
        t = lambda a: None if a is None else torch.from_numpy(a)
        sc = z[name + "/spline_scaler"] if name + "/spline_scaler" in z.files else None
        y, gx, gb, gs, gsc = kt.layer_step_sum_sq(t(z[name + "/x"]), t(z[name + "/grid"]), t(z[name + "/base_weight"]),
                                                  t(z[name + "/spline_weight"]), t(sc), int(z[name + "/k"]), True)
        tol = 1e-12 if z[name + "/x"].dtype == np.float64 else 2e-6
        assert rel_err(y.numpy(), z[name + "/y"]) < tol, name
        assert rel_err(gx.numpy(), z[name + "/gx"]) < tol, name
        assert rel_err(gb.numpy(), z[name + "/g_base_weight"]) < tol, name
        assert rel_err(gs.numpy(), z[name + "/g_spline_weight"]) < tol, name
        if sc is not None:
            assert rel_err(gsc.numpy(), z[name + "/g_spline_scaler"]) < tol, name
