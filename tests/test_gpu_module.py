"""GPU tests of the PyTorch-facing API (KANLinear / KAN with backend="cuda", the operator surface,
forward_with_regularization).  The parity target is the dense PyTorch backend -- the same
formulation as the reference's backend, itself pinned to the reference by tests/test_host_api.py
and the golden files -- evaluated in float64 where a float32 kernel is checked."""
import math

import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err

pytestmark = pytest.mark.gpu

sk = pytest.importorskip("torchsplinekan_b200")
from torchsplinekan_b200 import _C, _native, dense_backend as db   # noqa: E402

TOL32, TOL64 = 1e-5, 1e-12


def _err(a, b):
    return rel_err(a.detach().double().cpu().numpy(), b.detach().double().cpu().numpy())


def _pair(I, O, G=5, k=3, dtype=torch.float32, scaler=True, seed=0, act=torch.nn.SiLU, ref_dtype=None):
    """Native layer and a dense twin with identical parameters (randomised scaler)."""
    torch.manual_seed(seed)
    nat = sk.KANLinear(I, O, grid_size=G, spline_order=k, enable_standalone_scale_spline=scaler,
                       base_activation=act, backend="cuda").to("cuda", dtype)
    with torch.no_grad():
        if scaler:
            torch.nn.init.kaiming_uniform_(nat.spline_scaler, a=math.sqrt(5))
        nat.spline_weight.mul_(3.0)
    ref = sk.KANLinear(I, O, grid_size=G, spline_order=k, enable_standalone_scale_spline=scaler,
                       base_activation=act, backend="reference").to("cuda", ref_dtype or dtype)
    ref.load_state_dict({n: v.to(ref_dtype or dtype) for n, v in nat.state_dict().items()})
    return nat, ref


def _step(layer, x, loss=lambda y: y.square().sum()):
    for p in layer.parameters():
        p.grad = None
    xx = x.clone().requires_grad_()
    y = layer(xx)
    loss(y).backward()
    return [y, xx.grad] + [p.grad for p in layer.parameters()]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL32), (torch.float64, TOL64)])
@pytest.mark.parametrize("I,O,N", [(16, 32, 1024), (64, 128, 700), (8, 4, 33)])
def test_layer_matches_dense_backend(I, O, N, dtype, tol):
    nat, ref = _pair(I, O, dtype=dtype, ref_dtype=torch.float64)
    x = (torch.rand(N, I, device="cuda", dtype=dtype) * 2.4 - 1.2)
    got = _step(nat, x)
    want = _step(ref, x.double())
    assert nat.last_backend == "cuda" and ref.last_backend == "reference"
    for a, b in zip(got, want):
        assert _err(a, b) < tol


def test_leading_dims_and_cpu_and_half_inputs():
    nat, ref = _pair(6, 5)
    x = torch.rand(3, 7, 6, device="cuda") * 2 - 1
    assert nat(x).shape == (3, 7, 5)
    assert _err(nat(x), ref(x)) < TOL32
    with pytest.raises(RuntimeError, match="CPU tensor"):
        nat(x.cpu())
    with pytest.raises(RuntimeError, match="FP32 and FP64"):
        nat.half()(x.half())


def test_backward_skips_unneeded_grads():
    torch.manual_seed(1)
    L = sk.KANLinear(8, 4, backend="cuda").cuda()
    x = torch.rand(64, 8, device="cuda") * 2 - 1
    L(x).sum().backward()
    assert all(p.grad is not None for p in L.parameters())
    frozen = sk.KANLinear(8, 4, backend="cuda").cuda().requires_grad_(False)
    xx = x.clone().requires_grad_()
    frozen(xx).sum().backward()
    ref = sk.KANLinear(8, 4, backend="reference").cuda()
    ref.load_state_dict(frozen.state_dict())
    xr = x.clone().requires_grad_()
    ref(xr).sum().backward()
    assert torch.allclose(xx.grad, xr.grad, atol=1e-5)
    assert all(p.grad is None for p in frozen.parameters())


def test_gradcheck_and_gradgradcheck_native_fp64():
    torch.manual_seed(0)
    L = sk.KANLinear(3, 2, grid_size=4, backend="cuda").to("cuda", torch.float64)
    x = (torch.rand(5, 3, device="cuda", dtype=torch.float64) * 1.6 - 0.8).requires_grad_()
    assert torch.autograd.gradcheck(lambda t: L(t), (x,), eps=1e-6, atol=1e-7)
    assert torch.autograd.gradgradcheck(lambda t: L(t), (x,), eps=1e-6, atol=1e-6)


def test_second_derivative_matches_dense_backend():
    """PINN-style u_xx through create_graph=True (composite backward), float64, 1e-12."""
    torch.manual_seed(0)
    net = sk.KAN([2, 16, 16, 1], grid_size=8, spline_order=3, backend="cuda").to("cuda", torch.float64)
    ref = sk.KAN([2, 16, 16, 1], grid_size=8, spline_order=3, backend="reference").to("cuda", torch.float64)
    ref.load_state_dict(net.state_dict())
    x = torch.rand(512, 2, device="cuda", dtype=torch.float64) * 2 - 1

    def uxx_and_grads(model):
        for p in model.parameters():
            p.grad = None
        xx = x.clone().requires_grad_()
        u = model(xx)
        ux = torch.autograd.grad(u.sum(), xx, create_graph=True)[0]
        uxx = torch.autograd.grad(ux[:, 0].sum(), xx, create_graph=True)[0][:, 0]
        (uxx.square().mean() + u.square().mean()).backward()
        return [u, uxx] + [p.grad for p in model.parameters()]

    for a, b in zip(uxx_and_grads(net), uxx_and_grads(ref)):
        assert _err(a, b) < 1e-10 if a.dim() == 3 else _err(a, b) < 1e-9


def test_custom_base_activation_runs_spline_natively():
    nat, ref = _pair(5, 4, dtype=torch.float64, act=torch.nn.Tanh)
    x = torch.rand(40, 5, device="cuda", dtype=torch.float64) * 2 - 1
    for a, b in zip(_step(nat, x), _step(ref, x)):
        assert _err(a, b) < TOL64


def test_config0_golden_on_gpu():
    z = load_golden("config0.npz")
    torch.manual_seed(0)
    net = sk.KAN([16, 32, 8], grid_size=5, spline_order=3, backend="cuda")
    with torch.no_grad():
        for li, layer in enumerate(net.layers):
            layer.spline_scaler.copy_(torch.from_numpy(z[f"l{li}/spline_scaler"]))
    net = net.cuda()
    y = net(torch.from_numpy(z["x"]).cuda())
    torch.nn.functional.mse_loss(y, torch.from_numpy(z["target"]).cuda()).backward()
    assert rel_err(y.detach().cpu().numpy(), z["y"]) < TOL32
    for li, layer in enumerate(net.layers):
        for pn in ("base_weight", "spline_weight", "spline_scaler"):
            assert rel_err(getattr(layer, pn).grad.cpu().numpy(), z[f"l{li}/g_{pn}"]) < TOL32, (li, pn)


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-10), (torch.float32, 5e-5)])
def test_forward_with_regularization_fused_matches_dense(dtype, tol):
    torch.manual_seed(0)
    net = sk.KAN([12, 20, 6], grid_size=5, spline_order=3, backend="cuda").to("cuda", dtype)
    ref = sk.KAN([12, 20, 6], grid_size=5, spline_order=3, backend="reference").to("cuda", torch.float64)
    ref.load_state_dict({n: v.double() for n, v in net.state_dict().items()})
    x = torch.rand(300, 12, device="cuda", dtype=dtype) * 2.6 - 1.3        # partly outside the knots

    def run(model, xin, impl):
        for p in model.parameters():
            p.grad = None
        xx = xin.clone().requires_grad_()
        y, r = model.forward_with_regularization(xx, 1e-2, 1e-2, reg_impl=impl)
        (y.square().mean() + r).backward()
        return [y, r, xx.grad] + [p.grad for p in model.parameters()]

    got = run(net, x, "fused")
    want = run(ref, x.double(), "dense")
    assert net.layers[0].last_backend == "cuda"
    for a, b in zip(got, want):
        assert _err(a, b) < tol
    assert _err(net.regularization_loss(1e-2, 1e-2, x=x), want[1]) < tol


def test_fused_regulariser_memory_stays_below_phi():
    """Peak extra memory of the fused path is a fraction of phi [N,O,I] (the reference asserts the
    same bound, tests/test_fused_regularization.py:200-219 of the reference)."""
    torch.manual_seed(0)
    L = sk.KANLinear(128, 128, backend="cuda").cuda()
    x = torch.rand(4096, 128, device="cuda") * 2 - 1
    phi_bytes = 4096 * 128 * 128 * 4
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    y, r = L.forward_with_regularization(x, 1e-2, 1e-2, reg_impl="fused")
    (y.sum() + r).backward()
    torch.cuda.synchronize()
    assert torch.cuda.max_memory_allocated() - base < 0.5 * phi_bytes


def test_mnist_shaped_step_with_updated_grid():
    """Reduced copy of the 784-256-256-10 training step: update_grid knots, fused regulariser,
    cross-entropy; native (tensor-core + SIMT layers) against the dense backend in float64."""
    torch.manual_seed(0)
    net = sk.KAN([784, 256, 256, 10], backend="cuda").cuda()
    g = torch.Generator().manual_seed(0)
    x = (torch.rand(1024, 784, generator=g) * 2 - 1).cuda()
    labels = torch.randint(0, 10, (1024,), generator=torch.Generator().manual_seed(1)).cuda()
    net.update_grid(x[:512])
    ref = sk.KAN([784, 256, 256, 10], backend="reference").to("cuda", torch.float64)
    ref.load_state_dict({n: v.double() for n, v in net.state_dict().items()})
    ref32 = sk.KAN([784, 256, 256, 10], backend="reference").cuda()
    ref32.load_state_dict(net.state_dict())

    def run(model, xin, impl):
        for p in model.parameters():
            p.grad = None
        y, r = model.forward_with_regularization(xin, 1e-2, 1e-2, reg_impl=impl)
        (torch.nn.functional.cross_entropy(y, labels) + r).backward()
        return [y, r] + [p.grad for p in model.parameters()]

    got, want, want32 = run(net, x, "fused"), run(ref, x.double(), "dense"), run(ref32, x, "dense")
    names = ["y", "reg"] + [n for n, _ in net.named_parameters()]
    errs = {n: _err(a, b) for n, a, b in zip(names, got, want)}
    errs32 = {n: _err(a, b) for n, a, b in zip(names, got, want32)}
    dense_gap = {n: _err(a, b) for n, a, b in zip(names, want32, want)}
    print("fused32 vs dense64", errs)
    print("fused32 vs dense32", errs32)
    print("dense32 vs dense64", dense_gap)
    # y and the penalty itself are smooth in the rounding error.
    assert errs["y"] < 5e-5 and errs["reg"] < 5e-5, errs
    # The penalty's gradient contains sign(phi): where |phi| is at rounding level two evaluations
    # disagree on the sign, and every such flip moves the entries of one edge by up to 2 ga / N --
    # 2e-3 of the largest possible entry at 1024 rows, whatever the arithmetic (float32 against
    # float64 dense PyTorch shows the same).  Flips are discrete, so the max-norm is held to the
    # dense float32 gap with slack OR a few flips' worth, and the relative L2 norm (which single
    # entries hardly move, but a wrong kernel would) to 2e-3.
    n_rows = x.shape[0]
    for n, a, b in zip(names, got, want):
        assert errs[n] < max(5e-5, 3.0 * dense_gap[n], 5.0 / n_rows), (n, errs[n], dense_gap[n])
        assert float((a.double() - b).norm() / b.norm()) < 2e-3, n
    # plain forward/backward goes through kan_apply (tensor cores for the two wide layers)
    for p in net.parameters():
        p.grad = None
    for p in ref.parameters():
        p.grad = None
    y = net(x)
    torch.nn.functional.cross_entropy(y, labels).backward()
    y64 = ref(x.double())
    torch.nn.functional.cross_entropy(y64, labels).backward()
    # three layers deep the per-layer error (< 1e-5, checked layer by layer elsewhere) compounds
    assert _err(y, y64) < 5e-5
    for (n, p), q in zip(net.named_parameters(), ref.parameters()):
        assert _err(p.grad, q.grad) < 1e-4, n


@pytest.mark.parametrize("mode", ["auto", "simt"])
def test_wide_grid_layer(mode):
    """G = 64 after a grid update on bimodal data (clustered knots): tensor-core path (auto at this
    size) and gather path."""
    nat, ref = _pair(64, 48, G=64, k=3, ref_dtype=torch.float64)
    g = torch.Generator().manual_seed(0)
    x = torch.where(torch.rand(2048, 64, generator=g) < 0.5, -0.5, 0.5) + 0.15 * torch.randn(2048, 64, generator=g)
    x = x.clamp_(-1, 1).cuda()
    ref.update_grid(x.double())
    nat.load_state_dict({n: v.float() for n, v in ref.state_dict().items()})
    _C.set_mma_mode(mode)
    try:
        got = _step(nat, x)
    finally:
        _C.set_mma_mode("auto")
    for a, b in zip(got, _step(ref, x.double())):
        assert _err(a, b) < TOL32


def test_torch_ops_surface():
    nat, _ = _pair(6, 5)
    x = torch.rand(50, 6, device="cuda") * 2 - 1
    y, H = torch.ops.spline_kan.kan_forward(x, nat.grid, nat.base_weight, nat.spline_weight, nat.spline_scaler, 3, True)
    assert H.shape == (50, 6, 8) and _err(y, nat(x)) < 1e-6
    assert _err(H, db.compute_basis(x, nat.grid, 3)) < 1e-6
    D = torch.randn_like(y)
    gx, gb, gs, gc = torch.ops.spline_kan.kan_backward(D, x, nat.grid, nat.base_weight, nat.spline_weight,
                                                       nat.spline_scaler, H, 3, True)
    xx = x.clone().requires_grad_()
    (nat(xx) * D).sum().backward()
    assert _err(gx, xx.grad) < 1e-6 and _err(gs, nat.spline_weight.grad) < 1e-6
    with pytest.raises(RuntimeError, match=r"spline_weight.size\(2\)"):
        _C.kan_forward(x, nat.grid, nat.base_weight, nat.spline_weight[:, :, :7].contiguous(), nat.spline_scaler, 3, True)
    with pytest.raises(RuntimeError, match=r"G \+ 2k"):
        _C.kan_forward(x, torch.zeros(6, 73, device="cuda"), nat.base_weight,
                       torch.zeros(5, 6, 69, device="cuda"), nat.spline_scaler, 3, True)
    with pytest.raises(RuntimeError):
        _C.set_basis_impl(7)
    assert _C.get_basis_impl() == 1


def test_virtual_shards_sum_to_full_batch_gradient():
    """Eight row shards processed one after the other give the unsharded gradients, within the
    tolerance of the arithmetic (the full batch runs on the tensor cores, the small shards on the
    gather kernels)."""
    nat, _ = _pair(64, 96)
    x = torch.rand(4096, 64, device="cuda") * 2 - 1
    full = _step(nat, x)[2:]
    acc = [torch.zeros_like(g) for g in full]
    for r in range(8):
        a, b = sk.shard_rows(4096, 8, r)
        for s, g in zip(acc, _step(nat, x[a:b])[2:]):
            s += g
    for s, g in zip(acc, full):
        assert _err(s, g) < TOL32


def test_full_size_layer_properties():
    """1024 -> 1024 at 65536 rows: tensor-core path against the float64 SIMT kernels on a row
    subset, plus size-independent properties (row independence, linearity in dY)."""
    torch.manual_seed(0)
    L = sk.KANLinear(1024, 1024, backend="cuda").cuda()
    with torch.no_grad():
        torch.nn.init.kaiming_uniform_(L.spline_scaler, a=math.sqrt(5))
    x = torch.randn(65536, 1024, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0)).clamp_(-1, 1)
    args = (L.grid, L.base_weight.detach(), L.spline_weight.detach(), L.spline_scaler.detach())
    y = _native.forward(x, *args, 3, _native.MODE_AUTO)
    sub = slice(30000, 30000 + 2048)
    a64 = [t.double() for t in args]
    y64 = _native.forward(x[sub].double().contiguous(), *a64, 3, _native.MODE_SIMT)
    assert _err(y[sub], y64) < TOL32
    # rows are independent: the same rows evaluated alone give the same values
    y_alone = _native.forward(x[sub].contiguous(), *args, 3, _native.MODE_AUTO)
    assert torch.equal(y_alone, y[sub])
    # parameter gradients: full batch vs float64 on a subset cannot be compared directly, so check
    # additivity over row blocks and linearity in dY instead
    D = torch.randn_like(y)
    g_full = _native.backward(D, x, *args, 3, False, True, True, True)
    lo = _native.backward(D[:32768].contiguous(), x[:32768].contiguous(), *args, 3, False, True, True, True)
    hi = _native.backward(D[32768:].contiguous(), x[32768:].contiguous(), *args, 3, False, True, True, True)
    for f, a, b in zip(g_full[1:], lo[1:], hi[1:]):
        assert _err(a + b, f) < 2e-6
    g2 = _native.backward(2 * D, x, *args, 3, False, True, True, True)
    for f, a in zip(g_full[1:], g2[1:]):
        assert _err(a, 2 * f) < 1e-6
    # and against float64 for a block small enough for the SIMT kernels
    g64 = _native.backward(D[sub].double().contiguous(), x[sub].double().contiguous(), *a64, 3, False, True, True, True)
    g32 = _native.backward(D[sub].contiguous(), x[sub].contiguous(), *args, 3, False, True, True, True)
    for a, b in zip(g32[1:], g64[1:]):
        assert _err(a, b) < TOL32
    for buf in list(_native._ws_cache.values()):
        _native.check_status(buf)
    _native.release_workspaces()


def test_host_batch_prefetcher_order_and_reuse():
    """Batches come out in submission order with the right contents while copies run ahead of the
    consumer; a third submit without a next() is refused."""
    import torchsplinekan_b200 as sk
    dev = torch.device("cuda", 0)
    batches = [torch.full((1 << 20,), float(t)).pin_memory() for t in range(6)]
    pre = sk.HostBatchPrefetcher(batches[0].shape, batches[0].dtype, dev)
    pre.submit(batches[0])
    sums = []
    for t in range(6):
        if t + 1 < 6:
            pre.submit(batches[t + 1])
        x = pre.next()
        sums.append((x.double().sum() / x.numel()))
    assert [float(s) for s in sums] == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0]
    pre.submit(batches[0])
    pre.submit(batches[1])
    with pytest.raises(RuntimeError, match="in flight"):
        pre.submit(batches[2])
    with pytest.raises(ValueError, match="does not match"):
        sk.HostBatchPrefetcher((4,), torch.float32, dev).submit(torch.zeros(5).pin_memory())


def test_training_step_in_cuda_graph():
    """The operators neither synchronise nor allocate outside the caching allocator, so a whole
    training step can be captured in a CUDA graph; replays on new inputs match eager execution."""
    torch.manual_seed(0)
    net = sk.KAN([16, 32, 8], backend="cuda").cuda()
    x_static = torch.zeros(1024, 16, device="cuda")
    tgt = torch.randn(1024, 8, device="cuda")

    def step(x):
        for p in net.parameters():
            p.grad = None
        loss = torch.nn.functional.mse_loss(net(x), tgt)
        loss.backward()
        return loss

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step(x_static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        loss_static = step(x_static)
    grads_static = [p.grad for p in net.parameters()]
    for seed in (1, 2):
        x = torch.rand(1024, 16, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed)) * 2 - 1
        x_static.copy_(x)
        graph.replay()
        got = [float(loss_static)] + [g.clone() for g in grads_static]
        want_loss = step(x)
        want = [float(want_loss)] + [p.grad.clone() for p in net.parameters()]
        assert got[0] == pytest.approx(want[0], rel=1e-6)
        for a, b in zip(got[1:], want[1:]):
            assert _err(a, b) < 1e-6


@pytest.mark.parametrize("chunks", [1, 4])
@pytest.mark.parametrize("need_x", [False, True])
def test_direct_gradient_sink_matches_autograd(chunks, need_x):
    """GradientBucket(direct=True): the backward writes the parameter gradients into the bucket
    range by range of output rows; same numbers as the ordinary autograd path."""
    import torchsplinekan_b200 as sk
    torch.manual_seed(3)
    layer = sk.KANLinear(64, 1000, backend="cuda").cuda()       # 4 ranges of 256 rows, the last ragged
    plain = sk.KANLinear(64, 1000, backend="cuda").cuda()
    plain.load_state_dict(layer.state_dict())
    x = (torch.rand(700, 64, device="cuda") * 2 - 1).requires_grad_(need_x)
    x2 = x.detach().clone().requires_grad_(need_x)
    bucket = sk.GradientBucket([layer], direct=True)
    try:
        assert len(bucket._sinks) == 1
        bucket._sinks[0].chunks = chunks
        assert len(bucket._sinks[0].row_ranges(1000)) == chunks
        for _ in range(2):                                       # a second step overwrites, not accumulates
            bucket.zero_grad()
            layer(x).square().sum().backward()
            bucket.finish()
        plain(x2).square().sum().backward()
        for (n, p), q in zip(layer.named_parameters(), plain.parameters()):
            assert p.grad.data_ptr() >= bucket.buckets[0].data_ptr()
            assert _err(p.grad, q.grad) < 1e-6, n
        if need_x:
            assert _err(x.grad, 2 * x2.grad) < 1e-6              # x.grad accumulated over the two steps
    finally:
        bucket.remove()
    # after remove() the layer is back on the ordinary path
    layer.zero_grad()
    layer(x.detach()).square().sum().backward()
    assert _err(layer.spline_weight.grad, plain.spline_weight.grad) < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-9), (torch.float32, 2e-5)])
def test_update_grid_on_gpu_matches_cpu_solve(dtype, tol):
    """update_grid on CUDA samples (systems reduced by QR on the GPU, small systems solved on the
    CPU) against the same layer updated on the CPU (tall systems solved directly)."""
    import torchsplinekan_b200 as sk
    torch.manual_seed(4)
    cpu = sk.KANLinear(24, 17, grid_size=6, backend="reference").to(dtype)
    gpu = sk.KANLinear(24, 17, grid_size=6, backend="cuda").to("cuda", dtype)
    gpu.load_state_dict(cpu.state_dict())
    g = torch.Generator().manual_seed(5)
    x = torch.where(torch.rand(3000, 24, generator=g) < 0.5, -0.5, 0.5) + 0.2 * torch.randn(3000, 24, generator=g)
    x = x.clamp_(-1, 1).to(dtype)
    x[:, 3] = 0.25                                      # a constant feature: rank-deficient system
    cpu.update_grid(x)
    gpu.update_grid(x.cuda())
    assert _err(gpu.grid.cpu(), cpu.grid) < (1e-12 if dtype == torch.float64 else 1e-6)
    probe = (torch.rand(500, 24, generator=g) * 2 - 1).to(dtype)
    assert _err(gpu(probe.cuda()).cpu(), cpu(probe)) < tol
    keep = [i for i in range(24) if i != 3]
    assert _err(gpu.spline_weight[:, keep].cpu(), cpu.spline_weight[:, keep]) < tol


@pytest.mark.parametrize("act", [torch.nn.SiLU, torch.nn.Tanh])
def test_export_inference_caches_the_operand_images(act):
    """export_inference() (kan_linear.py:471-496) returns a frozen layer whose native forward builds the
    knot table and the weight image once and reuses them: same values as the trained layer, identical
    bits from call to call, and a rebuild as soon as a parameter or the knots change in place, are
    replaced by load_state_dict, or gradients are wanted again."""
    layer, _ = _pair(64, 300, act=act)
    x = (torch.rand(2048, 64, device="cuda") * 2 - 1)
    twin = layer.export_inference()
    assert twin.cache_operands and not layer.cache_operands and twin._operands is None
    with torch.no_grad():
        want = layer(x)
    got = twin(x)
    assert twin._operands is not None and twin._operands[1] is not None     # the tensor-core path took it
    assert twin.last_backend == "cuda" and not got.requires_grad
    assert _err(got, want) < 1e-6
    buf = twin._operands[1]
    assert torch.equal(twin(x), got) and twin._operands[1] is buf           # reused, not rebuilt
    assert torch.equal(twin(x[:1000]), got[:1000])
    # in-place change of a parameter: the cache notices (version counter) and the values follow
    with torch.no_grad():
        twin.spline_weight.mul_(2.0)
        twin.base_weight.zero_()
        layer.spline_weight.mul_(2.0)
        layer.base_weight.zero_()
        want2 = layer(x)
    got2 = twin(x)
    assert twin._operands[1] is not buf and _err(got2, want2) < 1e-6
    # new knots
    twin.update_grid(x[:512])
    layer_knots = twin.grid.clone()
    got3 = twin(x)
    plain = twin.make_like()
    plain.load_state_dict(twin.state_dict())
    assert not plain.cache_operands and torch.equal(plain.grid, layer_knots)
    with torch.no_grad():
        assert torch.equal(plain(x), got3)
    # gradients wanted again: the ordinary operator runs (and differentiates)
    xg = x[:300].clone().requires_grad_(True)
    twin(xg).sum().backward()
    assert xg.grad is not None and torch.isfinite(xg.grad).all()
    # a small call stays on the gather kernels and leaves the cache alone
    key = twin._operands[0]
    twin(x[:8])
    assert twin._operands[0] == key
    # float64 twin: no prepared form, ordinary path
    t64 = layer.double().export_inference()
    y64 = t64(x.double())
    assert t64._operands is None and y64.dtype == torch.float64


def test_export_inference_network_matches():
    """KAN.export_inference: every layer of the frozen network runs from its cached operands."""
    torch.manual_seed(0)
    net = sk.KAN([64, 256, 20], backend="cuda").to("cuda")          # both layers large enough for the tensor cores
    x = torch.rand(8192, 64, device="cuda") * 2 - 1
    frozen = net.export_inference()
    with torch.no_grad():
        want = net(x)
    got = frozen(x)
    assert all(l.cache_operands and l._operands is not None for l in frozen.layers)
    assert _err(got, want) < 1e-6
    assert torch.equal(frozen(x), got)
