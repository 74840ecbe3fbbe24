"""CPU-side checks: the C-ABI library loads and exports what the header declares, validation
runs before any launch, and the PyTorch-facing API mirrors the reference (names, state-dict keys,
initialisation, dense backend numerics, update_grid)."""
import ctypes
import math
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, load_golden, rel_err

import torchsplinekan_b200 as sk
from torchsplinekan_b200 import _C, _native, dense_backend as db


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "kan_b200.h")).read()
    declared = set(re.findall(r"\b(kanb200_\w+)\s*\(", header))
    assert len(declared) >= 15
    handle = ctypes.CDLL(_native.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in kan_b200.h but not exported"
    assert declared == set(_native.SIGNATURES), "ctypes signature table out of sync with the header"
    assert _native.lib().kanb200_version() >= 100


def test_shape_validation_messages():
    lib = _native.lib()
    assert lib.kanb200_check_shapes(8, 4, 4, 5, 3, _native.F32) == 0
    assert lib.kanb200_check_shapes(8, 4, 4, 66, 3, _native.F32) == _native.EINVAL
    assert re.search(r"G \+ 2k", _native.last_error())
    assert lib.kanb200_check_shapes(8, 70000, 4, 5, 3, _native.F32) == _native.EINVAL
    assert "in_features" in _native.last_error()
    assert lib.kanb200_check_shapes(8, 4, 4, 5, 4, _native.F32) == _native.EINVAL
    assert lib.kanb200_check_shapes(8, 4, 4, 5, 3, 7) == _native.EINVAL
    assert lib.kanb200_set_basis_impl(7) == _native.EINVAL
    assert lib.kanb200_get_basis_impl() == 1


def test_mode_resolution_and_workspace_sizes():
    f32, f64 = torch.float32, torch.float64
    assert _native.resolve_mode(_native.MODE_AUTO, f32, 65536, 1024, 1024, 5, 3) == _native.MODE_TC_BF16X3
    assert _native.resolve_mode(_native.MODE_AUTO, f64, 65536, 1024, 1024, 5, 3) == _native.MODE_SIMT
    # wide grids (a feature owns ceil((G + k) / 8) chunks of 8 columns) stay on the tensor cores
    assert _native.resolve_mode(_native.MODE_AUTO, f32, 16384, 512, 512, 64, 3) == _native.MODE_TC_BF16X3
    assert _native.resolve_mode(_native.MODE_AUTO, f32, 16384, 512, 512, 8, 4) == _native.MODE_SIMT   # k > 3
    # the forward alone moves to the tensor cores earlier than the backward (kanb200_resolve_mode_for)
    assert _native.resolve_mode(_native.MODE_AUTO, f32, 1024, 256, 10, 5, 3) == _native.MODE_SIMT
    assert _native.resolve_mode(_native.MODE_AUTO, f32, 1024, 256, 10, 5, 3, _native.OP_FORWARD) == _native.MODE_TC_BF16X3
    assert _native.resolve_mode(_native.MODE_AUTO, f32, 1024, 32, 8, 5, 3, _native.OP_FORWARD) == _native.MODE_SIMT
    assert _native.resolve_mode(_native.MODE_AUTO, f64, 65536, 64, 1, 8, 3, _native.OP_FORWARD) == _native.MODE_SIMT
    # scalar heads with many rows run on the narrow-layer kernels: no forward scratch, slabs for the gradients
    assert _native.workspace_bytes(_native.OP_FORWARD, _native.MODE_AUTO, f64, 131072, 64, 1, 8, 3) == 0
    assert _native.workspace_bytes(_native.OP_BACKWARD, _native.MODE_AUTO, f64, 131072, 64, 1, 8, 3, True, True) > 256
    assert _native.workspace_bytes(_native.OP_BACKWARD, _native.MODE_AUTO, f64, 131072, 64, 1, 8, 3, True, False) == 0
    with pytest.raises(RuntimeError, match="tensor-core"):
        _native.resolve_mode(_native.MODE_TC_BF16X3, f64, 1024, 64, 64, 5, 3)
    # G = 64, k = 3: 71 knots -> 76 + 20 * 71 floats per feature; 9 chunks per feature -> 576 column
    # blocks of spline + 8 of base
    fw64 = _native.workspace_bytes(_native.OP_FORWARD, _native.MODE_TC_BF16X3, f32, 16384, 512, 512, 64, 3)
    assert fw64 == 256 + 512 * (76 + 20 * 71) * 4 + 2 * (576 + 8) * 2 * 32768
    fw = _native.workspace_bytes(_native.OP_FORWARD, _native.MODE_AUTO, f32, 65536, 1024, 1024, 5, 3)
    # header + 1 KiB polynomial table per feature + packed weights: 4 output tiles x 144 column
    # blocks x (hi + lo) x 32 KiB
    assert fw == 256 + 1024 * 1024 + 4 * 144 * 2 * 32768
    bw = _native.workspace_bytes(_native.OP_BACKWARD, _native.MODE_AUTO, f32, 65536, 1024, 1024, 5, 3, False, True)
    assert bw > 65536 * 1024 * 4          # bf16 hi/lo image of dY plus the partial slab
    # float64 from 512 rows on: the weight image of the matrix-instruction kernels, 8 * 16 * 9 doubles
    assert _native.workspace_bytes(_native.OP_FORWARD, _native.MODE_SIMT, f64, 1024, 16, 8, 5, 3) == 256 + 9216
    assert _native.workspace_bytes(_native.OP_FORWARD, _native.MODE_SIMT, f64, 511, 16, 8, 5, 3) == 0
    assert _native.workspace_bytes(_native.OP_FORWARD, _native.MODE_SIMT, f32, 1024, 16, 8, 5, 3) == 0
    assert _native.workspace_bytes(_native.OP_EDGE_BWD, _native.MODE_SIMT, f64, 1024, 16, 8, 7, 1) > 0


def test_operator_errors_carry_numbers():
    """Messages built from numbers (sizes, limits) come out of the compiled operator layer intact
    -- a module linked against a foreign C++ runtime crashes exactly there."""
    z = torch.zeros
    with pytest.raises(RuntimeError, match=r"spline_weight.size\(2\)=7 but grid implies R=G\+k=8"):
        _C.kan_forward(z(4, 3), z(3, 12), z(5, 3), z(5, 3, 7), z(5, 3), 3, True)


def test_cpu_tensors_are_rejected_not_emulated():
    L = sk.KANLinear(4, 3, backend="cuda")
    with pytest.raises(RuntimeError, match="CPU tensor"):
        L(torch.zeros(2, 4))
    with pytest.raises(RuntimeError):
        _C.basis(torch.zeros(2, 4), torch.zeros(4, 12), 3)
    x, g = torch.zeros(2, 4), torch.zeros(4, 12)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.spline_kan.kan_forward(x, g, torch.zeros(3, 4), torch.zeros(3, 4, 8), torch.zeros(3, 4), 3, True)


def test_meta_kernels_give_shapes():
    x = torch.empty(5, 4, device="meta")
    y, H = torch.ops.spline_kan.kan_forward(x, torch.empty(4, 12, device="meta"), torch.empty(3, 4, device="meta"),
                                            torch.empty(3, 4, 8, device="meta"), torch.empty(3, 4, device="meta"),
                                            3, True)
    assert y.shape == (5, 3) and H.shape == (5, 4, 8)


def test_constructor_validation_and_limits():
    with pytest.raises(ValueError, match="grid_size"):
        sk.KANLinear(4, 4, grid_size=0)
    with pytest.raises(ValueError, match="spline_order"):
        sk.KANLinear(4, 4, spline_order=4)
    with pytest.raises(ValueError, match="backend"):
        sk.KANLinear(4, 4, backend="fast")
    assert sk.KANLinear(4, 4, grid_size=65, spline_order=3, backend="cuda").selected_backend == "cuda"   # 71 fits
    with pytest.raises(ValueError, match="CUDA kernel limit"):
        sk.KANLinear(4, 4, grid_size=66, spline_order=3, backend="cuda")
    auto = sk.KANLinear(4, 4, grid_size=66, spline_order=3, backend="auto")
    assert auto.selected_backend == "reference"
    with pytest.raises(ValueError):
        sk.KAN([4])


def test_state_dict_keys_and_init_match_reference():
    torch.manual_seed(0)
    net = sk.KAN([16, 32, 8], grid_size=5, spline_order=3, backend="reference")
    keys = sorted(net.layers[0].state_dict().keys())
    assert keys == ["_ref.base_weight", "_ref.grid", "_ref.spline_scaler", "_ref.spline_weight",
                    "base_weight", "grid", "spline_scaler", "spline_weight"]
    z = load_golden("config0.npz")
    for li, layer in enumerate(net.layers):
        assert np.array_equal(layer.base_weight.detach().numpy(), z[f"l{li}/base_weight"])
        assert np.array_equal(layer.spline_weight.detach().numpy(), z[f"l{li}/spline_weight"])
        assert np.array_equal(layer.grid.numpy(), z[f"l{li}/grid"])
        assert float(layer.spline_scaler.min()) == 1.0


def test_dense_backend_matches_golden():
    z = load_golden("basis.npz")
    for name in [str(n) for n in z["names"]]:
        k = int(name[1])
        x, grid = torch.from_numpy(z[name + "/x"]), torch.from_numpy(z[name + "/grid"])
        assert np.abs(db.compute_basis(x, grid, k).numpy() - z[name + "/H"]).max() <= 1e-14
        assert np.abs(db.compute_basis_derivative(x, grid, k).numpy() - z[name + "/dH"]).max() <= \
            1e-12 * max(1.0, np.abs(z[name + "/dH"]).max())


def test_config0_training_step_on_dense_backend():
    z = load_golden("config0.npz")
    torch.manual_seed(0)
    net = sk.KAN([16, 32, 8], grid_size=5, spline_order=3, backend="reference")
    with torch.no_grad():
        for li, layer in enumerate(net.layers):
            layer.spline_scaler.copy_(torch.from_numpy(z[f"l{li}/spline_scaler"]))
    y = net(torch.from_numpy(z["x"]))
    torch.nn.functional.mse_loss(y, torch.from_numpy(z["target"])).backward()
    assert rel_err(y.detach().numpy(), z["y"]) < 2e-6
    for li, layer in enumerate(net.layers):
        for pn in ("base_weight", "spline_weight", "spline_scaler"):
            assert rel_err(getattr(layer, pn).grad.numpy(), z[f"l{li}/g_{pn}"]) < 5e-6, (li, pn)


def _rebuild_golden_layer(ci, name, I, O, G, k, dt, scaler, N, xs):
    """Re-creates the layer of tests/golden/make_golden.py::make_layer with this package."""
    torch.manual_seed(100 + ci)
    L = sk.KANLinear(I, O, grid_size=G, spline_order=k, enable_standalone_scale_spline=scaler,
                     backend="reference").to(dt)
    g = torch.Generator().manual_seed(200 + ci)
    with torch.no_grad():
        for p in L.parameters():
            p.add_(0.3 * torch.randn(p.shape, generator=g, dtype=torch.float64).to(p.dtype))
        if scaler:
            torch.nn.init.kaiming_uniform_(L.spline_scaler, a=math.sqrt(5))
    g = torch.Generator().manual_seed(300 + ci)
    x = ((torch.rand(N, I, generator=g, dtype=torch.float64) * 2 - 1) * xs).to(dt)
    return L, x


def test_update_grid_matches_reference():
    z = load_golden("layer.npz")
    for ci, name, I, O, G, k, dt, N in ((5, "f64_g5k3_upd", 12, 10, 5, 3, torch.float64, 128),
                                        (7, "f64_g20k3_upd", 6, 8, 20, 3, torch.float64, 256)):
        L, x = _rebuild_golden_layer(ci, name, I, O, G, k, dt, True, N, 1.0)
        assert np.array_equal(x.numpy(), z[name + "/x"])
        L.update_grid(x[: N // 2])
        assert np.abs(L.grid.numpy() - z[name + "/grid"]).max() < 1e-14, name
        assert torch.equal(L.grid, L._ref.grid)
        assert rel_err(L.spline_weight.detach().numpy(), z[name + "/spline_weight"]) < 1e-9, name
        assert np.array_equal(L.base_weight.detach().numpy(), z[name + "/base_weight"])
        t = L.grid
        assert bool((t[:, 1:] > t[:, :-1]).all())
    with pytest.raises(ValueError, match="margin"):
        L.update_grid(x, margin=0.0)


def test_forward_with_regularization_dense_matches_golden():
    z = load_golden("reg.npz")
    name = "f64_g5k3"
    L = sk.KANLinear(10, 7, backend="reference").double()
    with torch.no_grad():
        L.base_weight.copy_(torch.from_numpy(z[name + "/base_weight"]))
        L.spline_weight.copy_(torch.from_numpy(z[name + "/spline_weight"]))
        L.spline_scaler.copy_(torch.from_numpy(z[name + "/spline_scaler"]))
    x = torch.from_numpy(z[name + "/x"]).requires_grad_()
    for impl in ("dense", "checkpoint", "auto"):
        for p in L.parameters():
            p.grad = None
        x.grad = None
        y, r = L.forward_with_regularization(x, 0.7, 1.3, reg_impl=impl, chunk_size=17)
        (y.square().sum() + r).backward()
        assert rel_err(y.detach().numpy(), z[name + "/fwr_y"]) < 1e-12
        assert abs(float(r) - float(z[name + "/fwr_reg"])) < 1e-12 * abs(float(r))
        assert rel_err(x.grad.numpy(), z[name + "/fwr_gx"]) < 1e-11
        assert rel_err(L.spline_weight.grad.numpy(), z[name + "/fwr_g_spline_weight"]) < 1e-11
    with pytest.raises(RuntimeError, match="fused"):
        L.forward_with_regularization(x, reg_impl="fused")
    with pytest.raises(ValueError, match="reg_impl"):
        L.forward_with_regularization(x, reg_impl="nope")
    with pytest.raises(ValueError, match="chunk_size"):
        L.forward_with_regularization(x, reg_impl="checkpoint", chunk_size=0)
    assert L.last_backend == "reference"


def test_export_and_extend_grid_preserve_the_function():
    torch.manual_seed(3)
    L = sk.KANLinear(5, 4, backend="reference").double()
    with torch.no_grad():
        torch.nn.init.kaiming_uniform_(L.spline_scaler, a=math.sqrt(5))
    x = torch.rand(200, 5, dtype=torch.float64) * 2 - 1
    E = L.export_inference()
    assert not E.enable_standalone_scale_spline and "spline_scaler" not in E.state_dict()
    assert torch.allclose(E(x), L(x), atol=1e-12)
    F2 = L.extend_grid(10, x)
    assert F2.grid_size == 10 and F2.spline_weight.shape[-1] == 13
    assert torch.allclose(F2(x), L(x), atol=1e-8)


def test_shard_rows_partitions_the_batch():
    for n, w in ((65536, 8), (10, 4), (7, 8), (0, 2)):
        spans = [sk.shard_rows(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans[:-1], spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1


def test_gradient_bucket_arguments_and_row_ranges():
    """Host logic of the data-parallel helpers that needs no device."""
    import torchsplinekan_b200 as sk
    from torchsplinekan_b200.data_parallel import _LayerSink
    with pytest.raises(ValueError, match="transport"):
        sk.GradientBucket([torch.nn.Linear(2, 2)], transport="bogus")
    sink = _LayerSink.__new__(_LayerSink)
    sink.chunks = 4
    assert sink.row_ranges(1024) == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    assert sink.row_ranges(1000) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert sink.row_ranges(300) == [(0, 256), (256, 300)]            # whole 256-row tiles
    sink.chunks = 1
    assert sink.row_ranges(1000) == [(0, 1000)]
    # CPU parameters: the bucket falls back to the process group's own all-reduce, no sink is made
    lin = torch.nn.Linear(3, 2)
    b = sk.GradientBucket([lin], direct=True)
    assert b.transport == "nccl" and b._sinks == [] and b.buckets[0].numel() == 8
    lin(torch.ones(1, 3)).sum().backward()
    b.finish()
    assert lin.weight.grad.data_ptr() == b.buckets[0].data_ptr()
    with pytest.raises(ValueError, match="CUDA device"):
        sk.HostBatchPrefetcher((2, 2), torch.float32, torch.device("cpu"))


def test_data_parallel_entry_points_validate_before_any_launch():
    """Argument checks of the row-range backward and of the all-reduce return error codes without
    touching a device (no compute call is made here)."""
    lib = _native.lib()
    p = ctypes.c_void_p(4096)                 # never dereferenced: every call below is refused
    rows = lambda o0, o1, mode=_native.MODE_TC_BF16X3: lib.kanb200_backward_param_rows(
        mode, p, p, p, p, p, p, p, p, p, 512, 64, 1024, 5, 3, o0, o1, p, 1 << 20, None)
    assert rows(256, 256) == _native.EINVAL and "rows" in _native.last_error()
    assert rows(0, 2000) == _native.EINVAL
    assert rows(0, 256, _native.MODE_SIMT) == _native.EUNSUPPORTED
    assert lib.kanb200_allreduce_pad_bytes(8, 128) == 8 * 128 * 4
    assert lib.kanb200_allreduce_pad_bytes(17, 8) == 0
    bases = (ctypes.c_void_p * 2)(4096, 8192)
    status = ctypes.c_void_p(4096)
    ar = lambda n, world=2, rank=0, local=1, blocks=8, pad=1 << 20, mc=None: lib.kanb200_allreduce_sum_f32(
        bases, mc, 0, pad, n, rank, world, local, blocks, 1.0, status, None)
    assert ar(1023) == _native.EINVAL and "multiple of 4" in _native.last_error()
    assert ar(1024, pad=1024) == _native.EINVAL and "overlaps" in _native.last_error()
    assert ar(1024, world=17) == _native.EINVAL
    assert ar(1024, rank=2) == _native.EINVAL
    assert ar(1024, blocks=0) == _native.EINVAL
    assert ar(1024, local=2, mc=ctypes.c_void_p(4096)) == _native.EINVAL and "peer loads" in _native.last_error()
    offs = (ctypes.c_size_t * 5)(0, 4096, 8192, 12288, 16384)
    cnts = (ctypes.c_size_t * 5)(64, 64, 64, 64, 64)
    assert lib.kanb200_allreduce_sum_f32_ranges(bases, None, offs, cnts, 5, 1 << 20, 0, 2, 1, 8, 128, 1.0,
                                                status, None) == _native.EINVAL
    assert lib.kanb200_allreduce_sum_f32_ranges(bases, None, offs, cnts, 2, 1 << 20, 0, 2, 1, 8, 100, 1.0,
                                                status, None) == _native.EINVAL
    # scratch of the table-driven basis kernels: only float32 with G + k = 8 and enough values
    f32, f64 = torch.float32, torch.float64
    assert _native.workspace_bytes(_native.OP_BASIS, _native.MODE_AUTO, f32, 65536, 1024, 1, 5, 3) == 256 + 1024 * 1024
    assert _native.workspace_bytes(_native.OP_BASIS, _native.MODE_AUTO, f64, 65536, 1024, 1, 5, 3) == 0
    assert _native.workspace_bytes(_native.OP_BASIS, _native.MODE_AUTO, f32, 65536, 1024, 1, 8, 3) == 0
    assert _native.workspace_bytes(_native.OP_BASIS, _native.MODE_AUTO, f32, 1024, 64, 1, 5, 3) == 0


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_penalty_head_closed_form_matches_dense_formulation(dtype):
    """The scalar head of the activation regulariser with its gradient in closed form against
    autograd through the dense formulation (reference_backend.py:149-170): generic edge means,
    some exactly zero, all zero; and second derivatives through the function."""
    from torchsplinekan_b200 import fused
    from torchsplinekan_b200.dense_backend import regularization_from_edge_means
    torch.manual_seed(0)
    cases = [torch.rand(5, 7, dtype=dtype) + 0.01,
             torch.cat([torch.zeros(2, 7, dtype=dtype), torch.rand(3, 7, dtype=dtype)]),
             torch.zeros(3, 4, dtype=dtype)]
    tol = 1e-14 if dtype == torch.float64 else 1e-6
    for a0 in cases:
        a = a0.clone().requires_grad_()
        (want,) = torch.autograd.grad(regularization_from_edge_means(a, 0.7, 1.3) * 2.0, a)
        b = a0.clone().requires_grad_()
        out = fused.penalty_from_edge_means(b, 0.7, 1.3)
        (got,) = torch.autograd.grad(out * 2.0, b)
        assert float((out.detach() - regularization_from_edge_means(a0, 0.7, 1.3)).abs()) <= tol
        assert float((got - want).abs().max()) <= tol
    if dtype == torch.float64:
        a = (torch.rand(4, 3, dtype=dtype) + 0.05).requires_grad_()
        f = lambda t: fused.penalty_from_edge_means(t, 0.7, 1.3)
        assert torch.autograd.gradcheck(f, (a,)) and torch.autograd.gradgradcheck(f, (a,))
