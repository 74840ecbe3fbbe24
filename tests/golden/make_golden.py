"""
Generates the golden fixtures in this directory from the REAL reference package.

Run once, in a container where the reference project is checked out, with

    python tests/golden/make_golden.py /path/to/reference

It imports ``spline_kan`` (pure-PyTorch backend, CPU) from that checkout and
stores inputs and outputs of the hot-path functions as compressed ``.npz``
files.  The test-suite only reads the ``.npz`` files; the reference is never
needed at test time.

Fixtures written
----------------
basis.npz     compute_basis / compute_basis_derivative for k in {1,2,3},
              G in {1,4,5,17}, uniform / non-uniform / repeated knots, points
              that include every knot exactly and out-of-domain values (fp64).
layer.npz     KANLinear(backend="reference") forward + backward of sum(y^2)
              (fp32 and fp64; with/without scaler; uniform and update_grid
              knots; inputs partly outside the knot range).
reg.npz       edge_abs_mean_dense, regularization_from_edge_means and
              forward_with_regularization(reg_impl="dense") values + gradients.
config0.npz   KAN([16,32,8]) on x[1024,16] ~ U(-1,1): forward and MSE backward.
"""

import sys
import os
import math

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _grid(I, G, k, kind, seed):
    g = torch.Generator().manual_seed(seed)
    n = G + 2 * k + 1
    if kind == "uniform":
        t = -1 + (torch.arange(n, dtype=torch.float64) - k) * 2 / G
        return t[None].expand(I, -1).contiguous()
    gaps = torch.rand(I, n - 1, generator=g, dtype=torch.float64) * 0.9 + 0.1
    if kind == "repeated":
        gaps[:, k + G // 2] = 0.0
    t = torch.cat([torch.zeros(I, 1, dtype=torch.float64), gaps.cumsum(1)], 1)
    return t - t[:, k:k + 1] - 1.0


def _points(grid, n, seed):
    g = torch.Generator().manual_seed(seed)
    lo, hi = grid[:, 0].min().item(), grid[:, -1].max().item()
    span = hi - lo
    x = torch.rand(n, grid.shape[0], generator=g, dtype=torch.float64) * 1.4 * span + lo - 0.2 * span
    return torch.cat([x, grid.t()], 0)


def make_basis(rb):
    out = {}
    names = []
    for k in (1, 2, 3):
        for G in (1, 4, 5, 17):
            for kind in ("uniform", "nonuniform", "repeated"):
                if kind == "repeated" and G < 2:
                    continue
                name = f"k{k}_G{G}_{kind}"
                grid = _grid(3, G, k, kind, seed=G + k)
                x = _points(grid, 48, seed=k)
                out[name + "/grid"] = grid.numpy()
                out[name + "/x"] = x.numpy()
                out[name + "/H"] = rb.compute_basis(x, grid, k).numpy()
                out[name + "/dH"] = rb.compute_basis_derivative(x, grid, k).numpy()
                names.append(name)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "basis.npz"), **out)


def _randomise(layer, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in layer.parameters():
            p.add_(0.3 * torch.randn(p.shape, generator=g, dtype=torch.float64).to(p.dtype))
        if layer.enable_standalone_scale_spline:
            torch.nn.init.kaiming_uniform_(layer.spline_scaler, a=math.sqrt(5))


def make_layer(sk):
    out = {}
    names = []
    cases = [
        # name, I, O, G, k, dtype, scaler, update_grid, N, xscale
        ("f32_g5k3", 16, 32, 5, 3, torch.float32, True, False, 96, 1.0),
        ("f64_g5k3", 16, 32, 5, 3, torch.float64, True, False, 96, 1.0),
        ("f64_g5k3_wide", 7, 5, 5, 3, torch.float64, True, False, 64, 2.6),
        ("f64_g3k2_noscaler", 9, 6, 3, 2, torch.float64, False, False, 64, 1.3),
        ("f64_g8k1", 5, 4, 8, 1, torch.float64, True, False, 64, 1.3),
        ("f64_g5k3_upd", 12, 10, 5, 3, torch.float64, True, True, 128, 1.0),
        ("f32_g5k3_upd", 12, 10, 5, 3, torch.float32, True, True, 128, 1.0),
        ("f64_g20k3_upd", 6, 8, 20, 3, torch.float64, True, True, 256, 1.0),
    ]
    for ci, (name, I, O, G, k, dt, scaler, upd, N, xs) in enumerate(cases):
        torch.manual_seed(100 + ci)
        L = sk.KANLinear(I, O, grid_size=G, spline_order=k,
                         enable_standalone_scale_spline=scaler, backend="reference").to(dt)
        _randomise(L, 200 + ci)
        g = torch.Generator().manual_seed(300 + ci)
        x = ((torch.rand(N, I, generator=g, dtype=torch.float64) * 2 - 1) * xs).to(dt)
        if upd:
            L.update_grid(x[: N // 2])
        xx = x.clone().requires_grad_()
        y = L(xx)
        y.square().sum().backward()
        out[name + "/x"] = x.numpy()
        out[name + "/grid"] = L.grid.detach().numpy()
        out[name + "/base_weight"] = L.base_weight.detach().numpy()
        out[name + "/spline_weight"] = L.spline_weight.detach().numpy()
        if scaler:
            out[name + "/spline_scaler"] = L.spline_scaler.detach().numpy()
            out[name + "/g_spline_scaler"] = L.spline_scaler.grad.numpy()
        out[name + "/k"] = np.array(k)
        out[name + "/y"] = y.detach().numpy()
        out[name + "/gx"] = xx.grad.numpy()
        out[name + "/g_base_weight"] = L.base_weight.grad.numpy()
        out[name + "/g_spline_weight"] = L.spline_weight.grad.numpy()
        names.append(name)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "layer.npz"), **out)


def make_reg(sk, rb):
    out = {}
    names = []
    cases = [
        ("f64_g5k3", 10, 7, 5, 3, torch.float64, True, 80),
        ("f32_g5k3", 10, 7, 5, 3, torch.float32, True, 80),
        ("f64_g4k2_noscaler", 6, 9, 4, 2, torch.float64, False, 50),
    ]
    for ci, (name, I, O, G, k, dt, scaler, N) in enumerate(cases):
        torch.manual_seed(400 + ci)
        L = sk.KANLinear(I, O, grid_size=G, spline_order=k,
                         enable_standalone_scale_spline=scaler, backend="reference").to(dt)
        _randomise(L, 500 + ci)
        g = torch.Generator().manual_seed(600 + ci)
        x = ((torch.rand(N, I, generator=g, dtype=torch.float64) * 2.6 - 1.3)).to(dt)
        # Raw statistic and its gradients with respect to (s, H, bw, W).
        s = torch.nn.functional.silu(x).detach().requires_grad_()
        H = rb.compute_basis(x, L.grid, k).detach().requires_grad_()
        bw = L.base_weight.detach().clone().requires_grad_()
        W = L._ref.effective_spline_weight().detach().clone().requires_grad_()
        a = rb.edge_abs_mean_dense(s, H, bw, W)
        ga = torch.rand(a.shape, generator=g, dtype=torch.float64).to(dt)
        (a * ga).sum().backward()
        out[name + "/x"] = x.numpy()
        out[name + "/k"] = np.array(k)
        out[name + "/grid"] = L.grid.detach().numpy()
        out[name + "/s"] = s.detach().numpy()
        out[name + "/H"] = H.detach().numpy()
        out[name + "/bw"] = bw.detach().numpy()
        out[name + "/W"] = W.detach().numpy()
        out[name + "/a"] = a.detach().numpy()
        out[name + "/ga"] = ga.numpy()
        out[name + "/ds"] = s.grad.numpy()
        out[name + "/dH"] = H.grad.numpy()
        out[name + "/dbw"] = bw.grad.numpy()
        out[name + "/dW"] = W.grad.numpy()
        # no-base variant of the statistic
        out[name + "/a_nobase"] = rb.edge_abs_mean_dense(None, H.detach(), None, W.detach()).numpy()
        # Scalar penalty + layer-level forward_with_regularization gradients.
        reg = rb.regularization_from_edge_means(a.detach(), 0.7, 1.3)
        out[name + "/reg_from_a"] = reg.numpy()
        a2 = a.detach().clone().requires_grad_()
        rb.regularization_from_edge_means(a2, 0.7, 1.3).backward()
        out[name + "/dreg_da"] = a2.grad.numpy()
        xx = x.clone().requires_grad_()
        for p in L.parameters():
            p.grad = None
        y, r = L.forward_with_regularization(xx, 0.7, 1.3, reg_impl="dense")
        (y.square().sum() + r).backward()
        out[name + "/base_weight"] = L.base_weight.detach().numpy()
        out[name + "/spline_weight"] = L.spline_weight.detach().numpy()
        if scaler:
            out[name + "/spline_scaler"] = L.spline_scaler.detach().numpy()
            out[name + "/fwr_g_spline_scaler"] = L.spline_scaler.grad.numpy()
        out[name + "/fwr_y"] = y.detach().numpy()
        out[name + "/fwr_reg"] = r.detach().numpy()
        out[name + "/fwr_gx"] = xx.grad.numpy()
        out[name + "/fwr_g_base_weight"] = L.base_weight.grad.numpy()
        out[name + "/fwr_g_spline_weight"] = L.spline_weight.grad.numpy()
        names.append(name)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "reg.npz"), **out)


def make_config0(sk):
    torch.manual_seed(0)
    net = sk.KAN([16, 32, 8], grid_size=5, spline_order=3, backend="reference")
    with torch.no_grad():
        for i, layer in enumerate(net.layers):
            torch.manual_seed(10 + i)
            torch.nn.init.kaiming_uniform_(layer.spline_scaler, a=math.sqrt(5))
    x = torch.rand(1024, 16, generator=torch.Generator().manual_seed(0)) * 2 - 1
    target = torch.randn(1024, 8, generator=torch.Generator().manual_seed(1))
    y = net(x)
    loss = torch.nn.functional.mse_loss(y, target)
    loss.backward()
    out = {"x": x.numpy(), "target": target.numpy(), "y": y.detach().numpy(),
           "loss": loss.detach().numpy()}
    for li, layer in enumerate(net.layers):
        for pname in ("base_weight", "spline_weight", "spline_scaler"):
            p = getattr(layer, pname)
            out[f"l{li}/{pname}"] = p.detach().numpy()
            out[f"l{li}/g_{pname}"] = p.grad.numpy()
        out[f"l{li}/grid"] = layer.grid.numpy()
    np.savez_compressed(os.path.join(HERE, "config0.npz"), **out)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KAN_REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("usage: make_golden.py /path/to/reference")
    sys.path.insert(0, ref_root)
    import spline_kan as sk
    from spline_kan import reference_backend as rb
    torch.set_num_threads(1)            # bit-stable reductions
    make_basis(rb)
    make_layer(sk)
    make_reg(sk, rb)
    make_config0(sk)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
