"""GPU parity tests: every call goes through the C ABI (ctypes) of libkan_b200.so
and is compared with the numpy oracle / the golden vectors of the reference."""
import numpy as np
import pytest
import torch

from conftest import load_golden, rel_err
from gpu_util import dev, make_layer_case, oracle_step
from oracle import kan_oracle as ko

pytestmark = pytest.mark.gpu

nat = pytest.importorskip("torchsplinekan_b200._native")

# fp32 tolerance of the north-star (relative to max|ref| per tensor); fp64: 1e-12
TOL32 = 1e-5
TOL64 = 1e-12


# ---------------------------------------------------------------------------
# tensor-core operand layouts (self-test kernel)
# ---------------------------------------------------------------------------
def _bf16_bits(a):
    """float32 array with bf16-representable values -> uint16 bit patterns."""
    return (a.astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)


def _img_kmajor(M):
    """[rows, 64] matrix -> K-major 128B-swizzled byte image (rows x 128 B), bf16."""
    return _img_kmajor_bits(_bf16_bits(M))


def _img_kmajor_bits(bits):
    rows = bits.shape[0]
    img = np.zeros(rows * 64, dtype=np.uint16)
    for r in range(rows):
        for c in range(8):
            off = (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)
            img[off // 2: off // 2 + 8] = bits[r, c * 8: c * 8 + 8]
    return img


def _img_mnmajor(M):
    """[mn, 64(k)] matrix -> MN-major image [mn group of 64][k group of 8][8 k rows][128 B]."""
    mn = M.shape[0]
    img = np.zeros(mn * 64, dtype=np.uint16)
    bits = _bf16_bits(M)
    for g in range(mn // 64):
        for kk in range(64):
            for ch in range(8):
                off = (g * 8 + (kk >> 3)) * 1024 + (kk & 7) * 128 + ((ch ^ (kk & 7)) << 4)
                img[off // 2: off // 2 + 8] = bits[g * 64 + ch * 8: g * 64 + ch * 8 + 8, kk]
    return img


def _run_selftest(layout, a_img, b_img):
    """Runs the operand-layout self-test kernel (its own small library, not part of the product ABI):
    the caller names the layout (0 = K-major, 1 = MN-major); descriptors are built inside from the
    same helpers the production kernels use."""
    import ctypes
    import os
    from torchsplinekan_b200.build import SELFTEST_PATH
    assert os.path.exists(SELFTEST_PATH), "build the self-test library with torchsplinekan_b200/build.py"
    lib = ctypes.CDLL(SELFTEST_PATH)
    fn = lib.kanb200_selftest_umma_layout
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_int] + [ctypes.c_void_p] * 5
    a = torch.from_numpy(a_img.view(np.int16)).cuda()
    b = torch.from_numpy(b_img.view(np.int16)).cuda()
    assert a.numel() == 128 * 64 and b.numel() == 256 * 64
    D = torch.zeros(128, 256, dtype=torch.float32, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = fn(layout, ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(D.data_ptr()),
            ctypes.c_void_p(st.data_ptr()), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0, "self-test kernel reported a timed-out wait"
    return D.cpu().numpy()


def _small_int_matrix(rng, rows):
    return rng.integers(-4, 5, size=(rows, 64)).astype(np.float32)


def test_umma_layout_k_major():
    rng = np.random.default_rng(0)
    A, B = _small_int_matrix(rng, 128), _small_int_matrix(rng, 256)
    D = _run_selftest(0, _img_kmajor(A), _img_kmajor(B))
    assert np.array_equal(D, A @ B.T)


def test_umma_layout_mn_major():
    rng = np.random.default_rng(1)
    A, B = _small_int_matrix(rng, 128), _small_int_matrix(rng, 256)
    D = _run_selftest(1, _img_mnmajor(A), _img_mnmajor(B))
    assert np.array_equal(D, A @ B.T)


def _run_selftest_general(a_img, b_img, params, n):
    import ctypes
    from torchsplinekan_b200.build import SELFTEST_PATH
    lib = ctypes.CDLL(SELFTEST_PATH)
    fn = lib.kanb200_selftest_umma_general
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_void_p] * 6
    a = torch.from_numpy(a_img.view(np.int16)).cuda()
    b = torch.from_numpy(b_img.view(np.int16)).cuda()
    D = torch.zeros(128, n, dtype=torch.float32, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = (ctypes.c_uint * 16)(*params, 0, 0)
    assert fn(a.data_ptr(), b.data_ptr(), ctypes.cast(p, ctypes.c_void_p), D.data_ptr(), st.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return D.cpu().numpy()


@pytest.mark.parametrize("q", [0, 1])
def test_umma_one_tile_read_by_two_products(q):
    """The operand readings the edge-statistic backward kernel relies on: ONE 128-byte-swizzled tile of
    rows [k][64 values] is the K-major operand of one product and, read MN-major with 32 columns that
    start 64 q bytes into every row, the operand of the next; and a sign tile stored as two K-major
    blocks of 64 samples is read MN-major (two groups of 64, 16 KB apart) by the third."""
    rng = np.random.default_rng(7 + q)
    # params: a_bytes, b_bytes, a_mn, b_mn, a_lbo, a_sbo, a_step, a_off, b_lbo, b_sbo, b_step, b_off, n, ksteps
    A = rng.integers(-4, 5, (128, 64)).astype(np.float32)
    B = rng.integers(-4, 5, (64, 64)).astype(np.float32)
    D = _run_selftest_general(_img_kmajor(A), _img_kmajor(B),
                              [16384, 8192, 0, 1, 16, 1024, 32, 0, 8192, 1024, 2048, 64 * q, 32, 4], 32)
    assert np.array_equal(D, A @ B[:, 32 * q:32 * q + 32])
    S = rng.integers(-1, 2, (128, 128)).astype(np.float32)
    W = rng.integers(-4, 5, (128, 64)).astype(np.float32)
    s_img = np.concatenate([_img_kmajor(S[:, :64]), _img_kmajor(S[:, 64:])])
    D = _run_selftest_general(s_img, _img_kmajor(W),
                              [32768, 16384, 1, 1, 16384, 1024, 2048, 0, 8192, 1024, 2048, 64 * q, 32, 8], 32)
    assert np.array_equal(D, S.T @ W[:, 32 * q:32 * q + 32])
    D = _run_selftest_general(s_img, _img_kmajor(B),
                              [32768, 8192, 0, 1, 16, 1024, 32, 16384, 8192, 1024, 2048, 64 * q, 32, 4], 32)
    assert np.array_equal(D, S[:, 64:] @ B[:, 32 * q:32 * q + 32])


# ---------------------------------------------------------------------------
# basis / basis gradient
# ---------------------------------------------------------------------------
def test_basis_matches_golden_fp64():
    z = load_golden("basis.npz")
    for name in [str(n) for n in z["names"]]:
        k = int(name[1])
        x, grid = dev(z[name + "/x"]), dev(z[name + "/grid"])
        H = nat.basis(x, grid, k).cpu().numpy()
        assert np.abs(H - z[name + "/H"]).max() <= 1e-13, name
        gH = np.random.default_rng(3).standard_normal(H.shape)
        gx = nat.basis_grad(x, grid, k, dev(gH)).cpu().numpy()
        ref = (gH * z[name + "/dH"]).sum(-1)
        assert np.abs(gx - ref).max() <= 1e-10 * max(1.0, np.abs(ref).max()), name


@pytest.mark.parametrize("G,k", [(5, 3), (64, 3), (17, 2), (1, 1)])
def test_basis_fp32_random(G, k):
    c = make_layer_case(777, 5, 3, G, k, np.float32, seed=G + k, nonuniform=True, xscale=1.4)
    H = nat.basis(dev(c["x"]), dev(c["grid"]), k).cpu().numpy()
    ref = ko.compute_basis(c["x"].astype(np.float64), c["grid"].astype(np.float64), k)
    assert np.abs(H - ref).max() < 5e-6
    # out-of-range inputs give exactly zero rows
    out = (c["x"] < c["grid"][:, 0]) | (c["x"] > c["grid"][:, -1])
    assert (H[out] == 0).all()


@pytest.mark.parametrize("G,k", [(5, 3), (6, 2), (7, 1)])
def test_basis_table_kernels_large_batch(G, k):
    """float32 with G + k = 8 and more than 2^21 values: the table-driven kernels (per-span
    polynomials, knots in registers); ragged feature group, inputs on knots and out of range."""
    N, I = 8200, 260
    c = make_layer_case(N, I, 3, G, k, np.float32, seed=G * 10 + k, nonuniform=True, xscale=1.3)
    assert nat.workspace_bytes(nat.OP_BASIS, nat.MODE_AUTO, torch.float32, N, I, 1, G, k) > 0
    assert nat.workspace_bytes(nat.OP_BASIS, nat.MODE_AUTO, torch.float32, 777, 5, 1, G, k) == 0
    x, grid = dev(c["x"]), dev(c["grid"])
    H = nat.basis(x, grid, k)
    rng = np.random.default_rng(1)
    gH = rng.standard_normal((N, I, 8)).astype(np.float32)
    gx = nat.basis_grad(x, grid, k, dev(gH))
    rows = np.sort(rng.choice(N, size=600, replace=False))
    rows[-1] = N - 1
    x64, g64 = c["x"][rows].astype(np.float64), c["grid"].astype(np.float64)
    ref = ko.compute_basis(x64, g64, k)
    got = H[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert np.abs(got - ref).max() < 5e-6
    out = (c["x"][rows] < c["grid"][:, 0]) | (c["x"][rows] > c["grid"][:, -1])
    assert out.any() and (got[out] == 0).all()
    dref = (ko.compute_basis_derivative(x64, g64, k) * gH[rows].astype(np.float64)).sum(-1)
    dgot = gx[torch.from_numpy(rows).cuda()].cpu().numpy()
    assert np.abs(dgot - dref).max() < 1e-5 * max(1.0, np.abs(dref).max())
    # the calls without scratch run the recurrence kernels and agree
    import ctypes
    H2 = torch.empty_like(H)
    rc = nat.lib().kanb200_basis(0, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(grid.data_ptr()),
                                 ctypes.c_void_p(H2.data_ptr()), N, I, G, k,
                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0 and float((H2 - H).abs().max()) < 5e-6


def test_basis_empty_batch():
    c = make_layer_case(4, 3, 2, 5, 3, np.float32, seed=0)
    H = nat.basis(torch.empty(0, 3, device="cuda"), dev(c["grid"]), 3)
    assert H.shape == (0, 3, 8)


# ---------------------------------------------------------------------------
# layer forward / backward
# ---------------------------------------------------------------------------
def _run_layer(case, mode, need_x=True):
    t = {n: dev(v) for n, v in case.items() if n != "k"}
    k = case["k"]
    y = nat.forward(t["x"], t["grid"], t["bw"], t["sw"], t["sc"], k, mode)
    D = 2.0 * y
    gx, gb, gs, gc = nat.backward(D, t["x"], t["grid"], t["bw"], t["sw"], t["sc"], k,
                                  need_x, True, True, True, mode)
    torch.cuda.synchronize()
    for tag in ("fwd", "bwd"):
        for key, buf in list(nat._ws_cache.items()):
            if key[2] == tag and mode in (nat.MODE_TC_BF16X3, nat.MODE_TC_BF16X1):
                nat.check_status(buf)
    f = lambda a: None if a is None else a.cpu().numpy()
    return f(y), f(D), f(gx), f(gb), f(gs), f(gc)


def _compare_layer(case, mode, tol, need_x=True):
    y, D, gx, gb, gs, gc = _run_layer(case, mode, need_x)
    c64 = {n: (None if v is None or isinstance(v, int) else v.astype(np.float64)) for n, v in case.items()}
    ry, _ = ko.kan_forward(c64["x"], c64["grid"], c64["bw"], c64["sw"], c64["sc"], case["k"])
    # backward is checked for the kernel's own dY so forward error does not leak in
    rgx, rgb, rgs, rgc = ko.kan_backward(D.astype(np.float64), c64["x"], c64["grid"], c64["bw"], c64["sw"],
                                         c64["sc"], case["k"])
    errs = {"y": rel_err(y, ry), "g_spline": rel_err(gs, rgs)}
    if need_x:
        errs["gx"] = rel_err(gx, rgx)
    if case["bw"] is not None:
        errs["g_base"] = rel_err(gb, rgb)
    if case["sc"] is not None:
        errs["g_scaler"] = rel_err(gc, rgc)
    bad = {n: e for n, e in errs.items() if not e < tol}
    assert not bad, f"errors above {tol}: {bad} (all: {errs})"
    return errs


def test_layer_golden_simt():
    z = load_golden("layer.npz")
    for name in [str(n) for n in z["names"]]:
        f64 = z[name + "/x"].dtype == np.float64
        t = {n: dev(z[name + "/" + n]) for n in ("x", "grid", "base_weight", "spline_weight")}
        sc = dev(z[name + "/spline_scaler"]) if name + "/spline_scaler" in z.files else None
        k = int(z[name + "/k"])
        y = nat.forward(t["x"], t["grid"], t["base_weight"], t["spline_weight"], sc, k, nat.MODE_SIMT)
        gx, gb, gs, gc = nat.backward(2.0 * y, t["x"], t["grid"], t["base_weight"], t["spline_weight"], sc, k,
                                      True, True, True, sc is not None, nat.MODE_SIMT)
        tol = TOL64 if f64 else TOL32
        assert rel_err(y.cpu().numpy(), z[name + "/y"]) < tol, name
        assert rel_err(gx.cpu().numpy(), z[name + "/gx"]) < tol, name
        assert rel_err(gb.cpu().numpy(), z[name + "/g_base_weight"]) < tol, name
        assert rel_err(gs.cpu().numpy(), z[name + "/g_spline_weight"]) < tol, name
        if sc is not None:
            assert rel_err(gc.cpu().numpy(), z[name + "/g_spline_scaler"]) < tol, name


@pytest.mark.parametrize("dtype,tol", [(np.float64, TOL64), (np.float32, TOL32)])
@pytest.mark.parametrize("shape", [
    dict(N=1, I=1, O=1, G=1, k=1),
    dict(N=257, I=19, O=70, G=5, k=3),
    dict(N=300, I=7, O=5, G=64, k=3, nonuniform=True),
    dict(N=130, I=33, O=3, G=12, k=2, scaler=False),
    dict(N=64, I=9, O=40, G=20, k=3, base=False, nonuniform=True),
    dict(N=515, I=2, O=64, G=8, k=3),
    dict(N=515, I=64, O=1, G=8, k=3),
    dict(N=1, I=300, O=37, G=5, k=3),                        # small-batch forward kernel: 1 row,
    dict(N=13, I=130, O=9, G=20, k=2, nonuniform=True),      # ragged rows / features / outputs,
    dict(N=255, I=7, O=70, G=64, k=3, base=False),           # its largest batch, no base branch
    dict(N=256, I=7, O=70, G=5, k=1, scaler=False),          # first batch of the tiled kernel
])
def test_layer_simt_vs_oracle(shape, dtype, tol):
    case = make_layer_case(dtype=dtype, seed=11, **shape)
    _compare_layer(case, nat.MODE_SIMT, tol)


@pytest.mark.parametrize("shape", [
    dict(N=512, I=2, O=64, G=8, k=3),                         # the three layers of the PINN-style network
    dict(N=1000, I=64, O=64, G=8, k=3),
    dict(N=700, I=64, O=1, G=8, k=3),
    dict(N=1111, I=70, O=130, G=20, k=2, nonuniform=True),    # ragged in rows, features, outputs
    dict(N=513, I=9, O=8, G=5, k=3, scaler=False),            # R + 1 odd, the 8-output tile
    dict(N=640, I=33, O=9, G=5, k=1, base=False, nonuniform=True),
    dict(N=900, I=5, O=200, G=60, k=3, nonuniform=True),      # one feature per chunk
    dict(N=2048, I=130, O=70, G=11, k=3),                     # 12 columns of padding in the last chunk
])
def test_layer_float64_matrix_kernels_vs_oracle(shape):
    """float64 from 512 rows on runs on the FP64 matrix instruction (dense formulation)."""
    case = make_layer_case(dtype=np.float64, seed=23, **shape)
    errs = _compare_layer(case, nat.MODE_SIMT, TOL64)
    print("dense64", shape, errs)
    _compare_layer(case, nat.MODE_AUTO, TOL64, need_x=False)


def test_fp64_matrix_instruction_fragments():
    """The fragment layout kan_dmma.cuh documents for mma.sync m8n8k4 f64, stated in numpy."""
    import ctypes
    from torchsplinekan_b200.build import SELFTEST_PATH
    lib = ctypes.CDLL(SELFTEST_PATH)
    fn = lib.kanb200_selftest_dmma_fragments
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 4
    rng = np.random.default_rng(0)
    A, B = rng.standard_normal((8, 4)), rng.standard_normal((4, 8))
    lanes = np.arange(32)
    g, t = lanes // 4, lanes % 4
    a, b = dev(A[g, t].copy()), dev(B[t, g].copy())
    c = torch.zeros(32, 4, dtype=torch.float64, device="cuda")
    assert fn(0, a.data_ptr(), b.data_ptr(), c.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    C = A @ B
    got = c.cpu().numpy()
    assert np.abs(got[:, 0] - C[g, 2 * t]).max() < 1e-14 and np.abs(got[:, 1] - C[g, 2 * t + 1]).max() < 1e-14


@pytest.mark.parametrize("shape", [
    dict(N=128, I=8, O=256, G=5, k=3),
    dict(N=300, I=40, O=70, G=5, k=3, nonuniform=True),
    dict(N=1024, I=64, O=256, G=5, k=3),
    dict(N=777, I=100, O=300, G=5, k=3, scaler=False),
    dict(N=640, I=72, O=128, G=4, k=2, nonuniform=True),
    dict(N=513, I=33, O=65, G=3, k=1, base=False),
    dict(N=2048, I=256, O=512, G=5, k=3, nonuniform=True),
    dict(N=2048, I=256, O=10, G=5, k=3),                      # narrow layers: a handful of outputs
    dict(N=1500, I=64, O=1, G=5, k=3, nonuniform=True),
    dict(N=777, I=40, O=4, G=8, k=2, scaler=False),
])
def test_layer_tensor_core_bf16x3_vs_oracle(shape):
    case = make_layer_case(dtype=np.float32, seed=5, **shape)
    errs = _compare_layer(case, nat.MODE_TC_BF16X3, TOL32)
    print("bf16x3", shape, errs)
    # both forward kernels (generated operand in shared / in tensor memory) whatever the shape picks
    try:
        for variant in (0, 1):
            nat.lib().kanb200_set_forward_variant(variant)
            _compare_layer(case, nat.MODE_TC_BF16X3, TOL32, need_x=False)
    finally:
        nat.lib().kanb200_set_forward_variant(-1)


@pytest.mark.parametrize("shape", [
    dict(N=300, I=40, O=70, G=6, k=3),                        # R = 9: two chunks per feature, 13 knots
    dict(N=515, I=33, O=130, G=8, k=3, nonuniform=True),      # R = 11
    dict(N=257, I=24, O=64, G=9, k=1, scaler=False),          # R = 10 with the 12-knot table
    dict(N=640, I=19, O=300, G=20, k=2, base=False, nonuniform=True),
    dict(N=1000, I=64, O=96, G=64, k=3, nonuniform=True),     # the widest grid: 9 chunks per feature
    dict(N=2048, I=128, O=256, G=64, k=3),
    dict(N=384, I=7, O=40, G=65, k=3),                        # G + 2k = 71, the limit
])
def test_layer_tensor_core_wide_grid_vs_oracle(shape):
    """Grids with G + k > 8: a feature owns several 8-column chunks of the contraction space."""
    case = make_layer_case(dtype=np.float32, seed=9, **shape)
    errs = _compare_layer(case, nat.MODE_TC_BF16X3, TOL32)
    print("bf16x3 wide", shape, errs)


def test_layer_tensor_core_bf16x1_stated_tolerance():
    """Single-MMA bf16 mode: operands rounded to 8 significand bits; stated tolerance 1e-2."""
    case = make_layer_case(dtype=np.float32, seed=6, N=1024, I=64, O=256, G=5, k=3)
    errs = _compare_layer(case, nat.MODE_TC_BF16X1, 1e-2)
    print("bf16x1", errs)
    assert errs["y"] > 1e-6          # it really is the reduced-precision path


def test_auto_mode_resolution():
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 65536, 1024, 1024, 5, 3) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float64, 65536, 1024, 1024, 5, 3) == nat.MODE_SIMT
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 16384, 512, 512, 64, 3) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 256, 256, 5, 3) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 16, 32, 5, 3) == nat.MODE_SIMT      # too little work
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 128, 16, 32, 5, 3) == nat.MODE_SIMT
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 32, 8, 5, 3) == nat.MODE_SIMT
    # narrow layers over long batches: the cost follows N I (outputs are padded to one tile)
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 8192, 256, 10, 5, 3) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 8192, 64, 4, 5, 3) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 8192, 4, 64, 5, 3) == nat.MODE_SIMT       # I < 8
    # the forward alone moves to the tensor cores earlier than the backward (the gather forward walks every feature)
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 256, 10, 5, 3) == nat.MODE_SIMT
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 256, 10, 5, 3, nat.OP_FORWARD) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 64, 64, 5, 3, nat.OP_FORWARD) == nat.MODE_TC_BF16X3
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 1024, 32, 8, 5, 3, nat.OP_FORWARD) == nat.MODE_SIMT
    assert nat.resolve_mode(nat.MODE_AUTO, torch.float32, 128, 784, 256, 5, 3, nat.OP_FORWARD) == nat.MODE_SIMT   # N < 256


def test_backward_skips_unrequested_outputs():
    case = make_layer_case(200, 12, 9, 5, 3, np.float32, seed=2)
    t = {n: dev(v) for n, v in case.items() if n != "k"}
    D = torch.randn(200, 9, device="cuda")
    gx, gb, gs, gc = nat.backward(D, t["x"], t["grid"], t["bw"], t["sw"], t["sc"], 3, True, False, False, False)
    assert gx is not None and gb is None and gs is None and gc is None
    gx, gb, gs, gc = nat.backward(D, t["x"], t["grid"], t["bw"], t["sw"], t["sc"], 3, False, True, True, True)
    assert gx is None and gb is not None and gs is not None and gc is not None


# ---------------------------------------------------------------------------
# regulariser statistic
# ---------------------------------------------------------------------------
def test_edge_abs_mean_matches_golden():
    z = load_golden("reg.npz")
    for name in [str(n) for n in z["names"]]:
        s, H, bw, W, ga = (dev(z[name + "/" + n]) for n in ("s", "H", "bw", "W", "ga"))
        tol = TOL64 if z[name + "/H"].dtype == np.float64 else TOL32
        a = nat.edge_abs_mean(s, H, bw, W)
        assert rel_err(a.cpu().numpy(), z[name + "/a"]) < tol, name
        a0 = nat.edge_abs_mean(None, H, None, W)
        assert rel_err(a0.cpu().numpy(), z[name + "/a_nobase"]) < tol, name
        ds, dH, dbw, dW = nat.edge_abs_mean_backward(ga, s, H, bw, W, True, True, True, True)
        for got, key in ((ds, "ds"), (dH, "dH"), (dbw, "dbw"), (dW, "dW")):
            assert rel_err(got.cpu().numpy(), z[name + "/" + key]) < tol, (name, key)


@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-11), (np.float32, 5e-5)])
@pytest.mark.parametrize("N,I,O,R", [(1000, 37, 70, 8), (333, 5, 200, 11), (129, 9, 6, 23), (64, 3, 4, 67)])
def test_edge_abs_mean_vs_oracle(N, I, O, R, dtype, tol):
    rng = np.random.default_rng(N)
    H = rng.uniform(0, 1, size=(N, I, R)).astype(dtype)
    s = rng.standard_normal((N, I)).astype(dtype)
    bw = rng.standard_normal((O, I)).astype(dtype)
    W = rng.standard_normal((O, I, R)).astype(dtype)
    ga = rng.uniform(0.5, 1.5, size=(O, I)).astype(dtype)
    a = nat.edge_abs_mean(dev(s), dev(H), dev(bw), dev(W)).cpu().numpy()
    ra = ko.edge_abs_mean(s.astype(np.float64), H.astype(np.float64), bw.astype(np.float64), W.astype(np.float64))
    assert rel_err(a, ra) < tol
    ds, dH, dbw, dW = nat.edge_abs_mean_backward(dev(ga), dev(s), dev(H), dev(bw), dev(W), True, True, True, True)
    rds, rdH, rdbw, rdW = ko.edge_abs_mean_backward(ga.astype(np.float64), s.astype(np.float64),
                                                    H.astype(np.float64), bw.astype(np.float64),
                                                    W.astype(np.float64))
    # sign(phi) may flip for |phi| at rounding level in fp32; compare in the max norm
    for got, ref in ((ds, rds), (dH, rdH), (dbw, rdbw), (dW, rdW)):
        assert rel_err(got.cpu().numpy(), ref) < max(tol, 2e-3 if dtype == np.float32 else tol)


# ---------------------------------------------------------------------------
# validation happens before any launch
# ---------------------------------------------------------------------------
def test_limits_rejected_before_launch():
    x = torch.zeros(4, 2, device="cuda")
    grid = torch.zeros(2, 73, device="cuda")       # G + 2k = 72 > 71
    with pytest.raises(RuntimeError, match=r"G \+ 2k"):
        nat.basis(x, grid, 3)
    with pytest.raises(RuntimeError, match="no CPU path"):
        nat.basis(torch.zeros(4, 2), torch.zeros(2, 12), 3)


# ---------------------------------------------------------------------------
# gradient all-reduce kernel: several ranks of one device inside a single launch
# ---------------------------------------------------------------------------
def _emulated_ranks(world, n, blocks, seed=0):
    pad = nat.allreduce_pad_bytes(world, blocks)
    stride = (n + pad // 4 + 63) // 64 * 64
    buf = torch.zeros(world, stride, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(seed)
    buf[:, :n] = torch.randn(world, n, device="cuda", generator=g)
    return buf, [buf[r].data_ptr() for r in range(world)], n * 4


@pytest.mark.parametrize("world,n,blocks", [(2, 4 * 1000, 4), (4, 4 * 123457, 8), (8, 4 * 50001, 16), (3, 8, 2)])
def test_allreduce_kernel_peer_loads_emulated_ranks(world, n, blocks):
    """Peer-load variant with all ranks' blocks co-resident in one launch: every rank's copy ends
    up with the sum taken in rank order (bit-exact), the signal pad returns to zero and can be
    reused by the next call."""
    buf, ptrs, pad_off = _emulated_ranks(world, n, blocks)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = buf[:, :n].clone()
    want = torch.zeros(n, device="cuda")
    for r in range(world):
        want = want + before[r]
    want = want * 0.5
    nat.allreduce_sum(ptrs, 0, 0, pad_off, n, 0, world, status, local_ranks=world, blocks=blocks, scale=0.5)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for r in range(world):
        assert torch.equal(buf[r, :n], want), r
    assert int(buf[:, n:].abs().sum().item()) == 0          # pad lowered again
    # second call on the result: world * 0.5 * want, same pad
    nat.allreduce_sum(ptrs, 0, 0, pad_off, n, 0, world, status, local_ranks=world, blocks=blocks, scale=1.0)
    torch.cuda.synchronize()
    want2 = torch.zeros(n, device="cuda")
    for r in range(world):
        want2 = want2 + want
    assert int(status.item()) == 0 and torch.equal(buf[0, :n], want2) and torch.equal(buf[world - 1, :n], want2)


def test_allreduce_kernel_missing_rank_times_out_with_status():
    """A rank that never launches: the waits of the others run out (limit set to half a second
    here), the kernel returns with status 1 and the context stays usable."""
    world, n, blocks = 2, 4 * 256, 2
    buf, ptrs, pad_off = _emulated_ranks(world, n, blocks)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = buf.clone()
    nat.allreduce_set_wait_limit_ms(500)
    try:
        nat.allreduce_sum(ptrs, 0, 0, pad_off, n, 0, world, status, local_ranks=1, blocks=blocks)   # rank 0 only
        torch.cuda.synchronize()
    finally:
        nat.allreduce_set_wait_limit_ms(10000)
    assert int(status.item()) == 1
    assert torch.equal(buf[:, :n], before[:, :n])            # nothing was reduced
    assert float(torch.ones(4, device="cuda").sum()) == 4.0  # the device still answers


def test_allreduce_argument_checks():
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    buf = torch.zeros(1024, device="cuda")
    with pytest.raises(RuntimeError, match="world size"):
        nat.allreduce_sum([buf.data_ptr()] * 17, 0, 0, 2048, 64, 0, 17, status)
    with pytest.raises(RuntimeError, match="multiple of 4"):
        nat.allreduce_sum([buf.data_ptr()], 0, 0, 2048, 63, 0, 1, status)
    with pytest.raises(RuntimeError, match="overlaps"):
        nat.allreduce_sum([buf.data_ptr()], 0, 0, 128, 64, 0, 1, status)
    with pytest.raises(RuntimeError, match="peer loads"):
        nat.allreduce_sum([buf.data_ptr()] * 2, buf.data_ptr(), 0, 2048, 64, 0, 2, status, local_ranks=2)


def test_allreduce_kernel_ranges_small_blocks_emulated_ranks():
    """Three ranges of the allocation in one launch with 128-thread blocks (the configuration that
    shares the SMs with a tensor-core kernel); data between the ranges is left alone."""
    world, blocks, n = 4, 8, 4 * 30000
    buf, ptrs, pad_off = _emulated_ranks(world, n, blocks, seed=3)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = buf[:, :n].clone()
    ranges = [(0, 4 * 5000), (4 * 4 * 6000, 4 * 7001), (4 * 4 * 20000, 4 * 3)]      # (byte offset, floats)
    nat.allreduce_sum_ranges(ptrs, 0, ranges, pad_off, 0, world, status, local_ranks=world, blocks=blocks,
                             threads=128)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = before.clone()
    for off, cnt in ranges:
        lo = off // 4
        tot = torch.zeros(cnt, device="cuda")
        for r in range(world):
            tot = tot + before[r, lo:lo + cnt]
        want[:, lo:lo + cnt] = tot
    assert torch.equal(buf[:, :n], want)
    with pytest.raises(RuntimeError, match="between 1 and 4 ranges"):
        nat.allreduce_sum_ranges(ptrs, 0, ranges + ranges, pad_off, 0, world, status, local_ranks=world)


# ---------------------------------------------------------------------------
# edge statistic straight from x (tensor cores)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("N,I,O,G,k,base,custom_s", [
    (4096, 64, 256, 5, 3, True, False), (1000, 37, 130, 5, 3, True, False), (2048, 16, 64, 4, 2, False, False),
    (3000, 24, 300, 5, 3, True, True), (512, 8, 16, 7, 1, True, False)])
def test_edge_abs_mean_from_x_tensor_cores(N, I, O, G, k, base, custom_s):
    """a[o,i] from x (basis never stored) against the float64 dense evaluation; non-uniform knots,
    a share of inputs exactly on knots and outside the knot range, ragged tiles."""
    case = make_layer_case(N, I, O, G, k, np.float32, seed=N + I, nonuniform=True, base=base)
    x, grid = dev(case["x"]), dev(case["grid"])
    W = dev(case["sw"] * case["sc"][:, :, None])
    bw = dev(case["bw"]) if base else None
    s = torch.tanh(x) if custom_s else None
    a = nat.edge_abs_mean_x(x, s, grid, bw, W, k, nat.MODE_TC_BF16X3)
    torch.cuda.synchronize()
    for key, buf in list(nat._ws_cache.items()):
        if key[2] == "edge_x":
            nat.check_status(buf)
    x64 = case["x"].astype(np.float64)
    H = ko.compute_basis(x64, case["grid"].astype(np.float64), k)
    phi = np.einsum("nir,oir->noi", H, (case["sw"] * case["sc"][:, :, None]).astype(np.float64))
    if base:
        sv = np.tanh(x64) if custom_s else x64 / (1.0 + np.exp(-x64))
        phi = phi + sv[:, None, :] * case["bw"].astype(np.float64)[None]
    want = np.abs(phi).mean(0)
    assert rel_err(a.cpu().numpy(), want) < TOL32


@pytest.mark.parametrize("dtype,tol", [(np.float32, 2e-5), (np.float64, 1e-11)])
@pytest.mark.parametrize("N,I,O,G,k,base,custom_s", [
    (700, 20, 50, 5, 3, True, False), (333, 9, 70, 12, 2, True, True), (520, 12, 33, 30, 3, False, False),
    (300, 6, 40, 4, 1, True, False)])
def test_edge_abs_mean_from_x_fma_kernels_and_backward(N, I, O, G, k, base, custom_s, dtype, tol):
    """Forward (FMA-pipe route) and all gradients of the from-x edge statistic against the operators
    that work on the materialised basis (themselves checked against the oracle and the golden file
    above): a, dW, dbw agree directly; gx = basis_grad(dH) (+ ds silu'(x)); ds for custom base values."""
    case = make_layer_case(N, I, O, G, k, dtype, seed=N + I + G, nonuniform=True, base=base)
    tdt = torch.float32 if dtype == np.float32 else torch.float64
    x, grid = dev(case["x"]), dev(case["grid"])
    W = dev(case["sw"] * case["sc"][:, :, None])
    bw = dev(case["bw"]) if base else None
    s_custom = torch.tanh(x) if (custom_s and base) else None
    s_dense = (s_custom if s_custom is not None else torch.nn.functional.silu(x)) if base else None
    rng = np.random.default_rng(5)
    ga = dev(rng.uniform(0.1, 1.0, size=(O, I)).astype(dtype))
    H = nat.basis(x, grid, k)
    a_ref = nat.edge_abs_mean(s_dense, H, bw, W)
    ds_ref, dH_ref, dbw_ref, dW_ref = nat.edge_abs_mean_backward(ga, s_dense, H, bw, W, True, True, True, True)
    gx_ref = nat.basis_grad(x, grid, k, dH_ref)
    if base and s_custom is None:
        sig = torch.sigmoid(x)
        gx_ref = gx_ref + ds_ref * (sig * (1 + x * (1 - sig)))
    a = nat.edge_abs_mean_x(x, s_custom, grid, bw, W, k, nat.MODE_SIMT)
    gx, ds, dbw, dW = nat.edge_abs_mean_x_backward(ga, x, s_custom, grid, bw, W, k, mode=nat.MODE_SIMT)
    torch.cuda.synchronize()
    f = lambda t: t.double().cpu().numpy()
    assert rel_err(f(a), f(a_ref)) < tol
    assert rel_err(f(dW), f(dW_ref)) < tol
    assert rel_err(f(gx), f(gx_ref)) < tol
    if base:
        assert rel_err(f(dbw), f(dbw_ref)) < tol
    if s_custom is not None:
        assert rel_err(f(ds), f(ds_ref)) < tol
    else:
        assert ds is None
    assert x.dtype == tdt


def _edge_backward_dense64(case, ga, base):
    """float64 dense evaluation of the edge statistic's gradients: (phi, gx, dbw, dW)."""
    k = case["k"]
    x = case["x"].astype(np.float64)
    g64 = case["grid"].astype(np.float64)
    W = (case["sw"] * case["sc"][:, :, None]).astype(np.float64)
    H = ko.compute_basis(x, g64, k)
    dHdx = ko.compute_basis_derivative(x, g64, k)
    phi = np.einsum("nir,oir->noi", H, W)
    sig = 1.0 / (1.0 + np.exp(-x))
    if base:
        bw = case["bw"].astype(np.float64)
        phi = phi + (x * sig)[:, None, :] * bw[None]
    sg = np.sign(phi) * (ga.astype(np.float64) / x.shape[0])[None]
    dW = np.einsum("noi,nir->oir", sg, H)
    gx = np.einsum("noi,oir,nir->ni", sg, W, dHdx)
    dbw = None
    if base:
        dbw = np.einsum("noi,ni->oi", sg, x * sig)
        gx = gx + np.einsum("noi,oi->ni", sg, bw) * (sig * (1 + x * (1 - sig)))
    return phi, gx, dbw, dW


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_edge_penalty_one_launch_matches_dense_formulation(dtype):
    """kanb200_edge_penalty (value and closed-form gradient of the regulariser's scalar head in one
    launch) against autograd through the dense tensor formulation (reference_backend.py:149-170):
    generic edge means, some exactly zero, all zero, a statistic of a realistic size; and the
    autograd function that uses it."""
    from torchsplinekan_b200 import _native as nat, fused
    from torchsplinekan_b200.dense_backend import regularization_from_edge_means
    torch.manual_seed(0)
    cases = [torch.rand(5, 7, dtype=dtype) + 0.01,
             torch.cat([torch.zeros(2, 7, dtype=dtype), torch.rand(3, 7, dtype=dtype)]),
             torch.zeros(3, 4, dtype=dtype),
             torch.rand(256, 784, dtype=dtype) * 0.05,
             torch.cat([torch.zeros(40, 300, dtype=dtype), torch.rand(60, 300, dtype=dtype)])]     # two-launch form with dead entries
    tol = 1e-13 if dtype == torch.float64 else 2e-6
    for a0 in cases:
        a = a0.clone().requires_grad_()
        want_v = regularization_from_edge_means(a, 0.7, 1.3)
        (want_g,) = torch.autograd.grad(want_v, a)
        got_v, got_g = nat.edge_penalty(a0.cuda(), 0.7, 1.3)
        scale = max(1.0, float(want_v.detach().abs()))
        assert abs(float(got_v) - float(want_v)) <= tol * scale
        gscale = max(1.0, float(want_g.abs().max()))
        assert float((got_g.cpu() - want_g).abs().max()) <= tol * gscale * 4
        only_v, none_g = nat.edge_penalty(a0.cuda(), 0.7, 1.3, need_grad=False)
        assert none_g is None and float(only_v) == float(got_v)
        # the single-block form (no workspace) and the two-launch form agree
        one_v, one_g = nat.edge_penalty(a0.cuda(), 0.7, 1.3, scratch=False)
        assert abs(float(one_v) - float(want_v)) <= tol * scale
        assert float((one_g.cpu() - want_g).abs().max()) <= tol * gscale * 4
        b = a0.cuda().requires_grad_()
        out = fused.penalty_from_edge_means(b, 0.7, 1.3)
        (gb,) = torch.autograd.grad(out * 2.0, b)
        assert float((gb.cpu() - 2.0 * want_g).abs().max()) <= tol * gscale * 8
    if dtype == torch.float64:
        a = (torch.rand(4, 3, dtype=dtype, device="cuda") + 0.05).requires_grad_()
        f = lambda t: fused.penalty_from_edge_means(t, 0.7, 1.3)
        assert torch.autograd.gradcheck(f, (a,)) and torch.autograd.gradgradcheck(f, (a,))


@pytest.mark.parametrize("N,I,O,G,k,base", [
    (1024, 16, 256, 5, 3, True), (777, 37, 130, 5, 3, True), (2048, 8, 64, 4, 2, False), (300, 5, 16, 7, 1, True),
    (4096, 64, 256, 5, 3, True)])
def test_edge_backward_tensor_cores_fixed_signs(N, I, O, G, k, base):
    """Gradients of the from-x edge statistic on the tensor cores where the sign of every phi is
    beyond doubt (coefficients and base weights of one sign per output, inputs in (0, 1) so that
    SiLU is positive): sign tile, both chained products, scaling and the ragged edges are checked
    at float32 accuracy against the float64 dense evaluation."""
    case = make_layer_case(N, I, O, G, k, np.float32, seed=N + O, nonuniform=True, base=base)
    rng = np.random.default_rng(N)
    flip = np.where(np.arange(O) % 3 == 0, -1.0, 1.0).astype(np.float32)
    case["x"] = rng.uniform(0.02, 0.98, size=case["x"].shape).astype(np.float32)
    case["sw"] = (np.abs(case["sw"]) + 0.05) * flip[:, None, None]
    case["sc"] = np.abs(case["sc"]) + 0.05
    if base:
        case["bw"] = (np.abs(case["bw"]) + 0.05) * flip[:, None]
    ga = rng.uniform(0.1, 1.0, size=(O, I)).astype(np.float32)
    phi, gx_ref, dbw_ref, dW_ref = _edge_backward_dense64(case, ga, base)
    assert np.abs(phi).min() > 1e-4
    x, grid = dev(case["x"]), dev(case["grid"])
    W = dev(case["sw"] * case["sc"][:, :, None])
    bw = dev(case["bw"]) if base else None
    gx, ds, dbw, dW = nat.edge_abs_mean_x_backward(dev(ga), x, None, grid, bw, W, k, mode=nat.MODE_TC_BF16X3)
    torch.cuda.synchronize()
    for key, buf in list(nat._ws_cache.items()):
        if key[2] == "edge_x":
            nat.check_status(buf)
    f = lambda t: t.double().cpu().numpy()
    errs = {"dW": rel_err(f(dW), dW_ref), "gx": rel_err(f(gx), gx_ref)}
    if base:
        errs["dbw"] = rel_err(f(dbw), dbw_ref)
    print("edge backward (tensor cores)", (N, I, O), errs)
    assert all(e < 2e-5 for e in errs.values()), errs
    # parameter gradients alone (no input gradient: the third product is skipped)
    _, _, dbw2, dW2 = nat.edge_abs_mean_x_backward(dev(ga), x, None, grid, bw, W, k, need_x=False,
                                                   mode=nat.MODE_TC_BF16X3)
    assert torch.equal(dW2, dW) and (not base or torch.equal(dbw2, dbw))


@pytest.mark.parametrize("N,I,O", [(2048, 32, 256), (1500, 20, 70)])
def test_edge_backward_tensor_cores_random_signs(N, I, O):
    """Random coefficients: phi changes sign from sample to sample.  Where |phi| is at rounding level
    two evaluations may disagree on the sign, and each such sample moves an entry by 2 ga / N times a
    basis value, so the comparison is in the relative L2 norm and in the share of entries that agree.
    The tensor-core kernel forms phi from split-bf16 operands (about 5e-6 of its terms) and, by
    default, evaluates every phi below 2e-5 of a bound on its terms again in float32 before taking
    the sign: its gradients then are as close to float64 as those of the float32 FMA kernels
    (measured: relative L2 3e-7 .. 8e-7).  With the re-check switched off a few more samples near
    phi = 0 fall on the other side (7e-5 / 3e-5 / 2e-4 for dW / dbw / gx, 99.9 % of entries within 2e-5)."""
    G, k = 5, 3
    case = make_layer_case(N, I, O, G, k, np.float32, seed=3 * N + O, nonuniform=True, base=True)
    rng = np.random.default_rng(O)
    ga = rng.uniform(0.1, 1.0, size=(O, I)).astype(np.float32)
    _, gx_ref, dbw_ref, dW_ref = _edge_backward_dense64(case, ga, True)
    x, grid = dev(case["x"]), dev(case["grid"])
    W, bw = dev(case["sw"] * case["sc"][:, :, None]), dev(case["bw"])
    f = lambda t: t.double().cpu().numpy()
    gx_f, _, dbw_f, dW_f = nat.edge_abs_mean_x_backward(dev(ga), x, None, grid, bw, W, k, mode=nat.MODE_SIMT)
    assert nat.get_edge_sign_recheck()
    try:
        for recheck, l2_bound, share in ((True, 5e-6, 0.9999), (False, 5e-4, 0.995)):
            nat.set_edge_sign_recheck(recheck)
            gx, ds, dbw, dW = nat.edge_abs_mean_x_backward(dev(ga), x, None, grid, bw, W, k, mode=nat.MODE_TC_BF16X3)
            torch.cuda.synchronize()
            for name, got, fma, want in (("dW", dW, dW_f, dW_ref), ("dbw", dbw, dbw_f, dbw_ref), ("gx", gx, gx_f, gx_ref)):
                l2 = np.linalg.norm(f(got) - want) / np.linalg.norm(want)
                l2_fma = np.linalg.norm(f(fma) - want) / np.linalg.norm(want)
                close = np.mean(np.abs(f(got) - want) <= 2e-5 * np.abs(want).max())
                print(f"edge backward random signs, re-check {recheck}, {name}: rel L2 {l2:.2e} "
                      f"(FMA kernels {l2_fma:.2e}), entries within 2e-5: {close:.4f}")
                assert l2 < max(l2_bound, 3 * l2_fma) and close > share
    finally:
        nat.set_edge_sign_recheck(True)


@pytest.mark.parametrize("shape", [
    dict(N=257, I=1024, O=64, G=5, k=3), dict(N=3000, I=24, O=520, G=20, k=2, nonuniform=True),
    dict(N=130, I=40, O=1024, G=5, k=3, nonuniform=True)])
def test_layer_tensor_core_general_weights(shape):
    """Spline-dominated weights (the reference's initialisation makes the base branch dominate y and
    hides accumulation error): 1024 features in one tile, a wide grid, many outputs."""
    _compare_layer(make_layer_case(dtype=np.float32, seed=11, **shape), nat.MODE_TC_BF16X3, TOL32)


@pytest.mark.parametrize("N,I,O,G,k,base,scaler", [
    (1024, 64, 640, 5, 3, True, True),      # two output tiles + remainder: shared-memory operand kernel
    (777, 37, 130, 5, 3, True, False),      # one output tile: tensor-memory operand kernel, ragged everything
    (512, 24, 300, 4, 2, False, True),      # no base branch
    (2048, 16, 64, 20, 3, True, True),      # wide grid: three chunks per feature
])
def test_forward_prepared_equals_forward_bit_for_bit(N, I, O, G, k, base, scaler):
    """kanb200_prepare_forward + kanb200_forward_prepared (knot table and weight image built once,
    contraction alone per call: the form export_inference's frozen layers use,
    spline_kan/kan_linear.py:471-496) against kanb200_forward in the same tensor-core mode: identical
    bits, for several calls on one prepared buffer and for both MMA modes."""
    from torchsplinekan_b200 import _native as nat
    case = make_layer_case(N, I, O, G, k, np.float32, seed=31, nonuniform=True, scaler=scaler, base=base)
    x, grid, sw = dev(case["x"]), dev(case["grid"]), dev(case["sw"])
    bw, sc = dev(case["bw"]), dev(case["sc"])
    prepared = nat.prepare_forward(grid, bw, sw, sc, k)
    assert prepared is not None and prepared.dtype == torch.uint8
    for mode in (nat.MODE_TC_BF16X3, nat.MODE_TC_BF16X1):
        want = nat.forward(x, grid, bw, sw, sc, k, mode)
        for _ in range(2):
            got = nat.forward_prepared(x, prepared, O, G, k, base, mode)
            assert torch.equal(got, want)
    half = nat.forward_prepared(x[: N // 2 + 3], prepared, O, G, k, base, nat.MODE_TC_BF16X3)
    assert torch.equal(half, nat.forward(x[: N // 2 + 3].contiguous(), grid, bw, sw, sc, k, nat.MODE_TC_BF16X3))
    # float64 has no prepared form
    assert nat.prepare_forward(grid.double(), None if bw is None else bw.double(), sw.double(),
                               None if sc is None else sc.double(), k) is None
    with pytest.raises(RuntimeError):
        nat.forward_prepared(x, prepared[: prepared.numel() // 2].contiguous(), O, G, k, base, nat.MODE_TC_BF16X3)


@pytest.mark.parametrize("N,I,O,G,k", [
    (300, 256, 40, 5, 3),        # 36 column blocks = 2 chains, tensor-memory operand kernel, ragged rows
    (130, 784, 300, 5, 3),       # 111 blocks = 5 chains, shared-memory operand kernel (two output tiles)
    (1000, 200, 520, 4, 2),      # 3 output tiles (a pair and a single one), 2 chains
    (256, 24, 64, 64, 3),        # wide grid: 9 chunks per feature
])
def test_forward_small_batch_chains_as_work_items(N, I, O, G, k):
    """Small batches: the chains of 24 column blocks of a tile run as separate work items whose partial
    results are added in fixed order by a second kernel.  Against the float64 oracle (stated 1e-5),
    and bit-identical to the same call with a workspace too small for the partial results, where a
    tile's chains run one after the other inside one work item."""
    from torchsplinekan_b200 import _native as nat
    case = make_layer_case(N, I, O, G, k, np.float32, seed=41, nonuniform=True)
    x, grid, bw, sw, sc = dev(case["x"]), dev(case["grid"]), dev(case["bw"]), dev(case["sw"]), dev(case["sc"])
    y = nat.forward(x, grid, bw, sw, sc, k, nat.MODE_TC_BF16X3)
    want = oracle_step(case, need_x=False)[0]
    assert rel_err(y.cpu().numpy().astype(np.float64), want) < 1e-5
    full = nat.workspace_bytes(nat.OP_FORWARD, nat.MODE_TC_BF16X3, torch.float32, N, I, O, G, k)
    prepared = nat.prepare_forward(grid, bw, sw, sc, k)
    assert full > 256 + prepared.numel()                      # room for the partial results was asked for
    y2 = torch.empty_like(y)
    small = torch.zeros(256, dtype=torch.uint8, device=x.device)
    lib = nat.lib()
    rc = lib.kanb200_forward_prepared(0, nat.MODE_TC_BF16X3, x.data_ptr(), prepared.data_ptr(), prepared.numel(), 1,
                                      y2.data_ptr(), N, I, O, G, k, small.data_ptr(), small.numel(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    assert torch.equal(nat.forward(x, grid, bw, sw, sc, k, nat.MODE_TC_BF16X3), y)      # and from run to run


@pytest.mark.parametrize("N,I,O,G,k,dtype,tol", [
    (32768, 24, 1, 8, 3, np.float64, TOL64),      # scalar output, eleven basis functions (16-slot variant)
    (40000, 9, 4, 5, 3, np.float32, TOL32),       # four outputs, ragged last block
    (32768, 17, 3, 4, 2, np.float64, TOL64),
    (33000, 6, 2, 12, 1, np.float32, TOL32),
])
def test_narrow_layer_kernels(N, I, O, G, k, dtype, tol):
    """Layers with a handful of outputs and many samples (scalar heads: KAN[2,64,64,1]'s last layer) take
    the narrow-layer kernels in AUTO mode: forward and all gradients against the float64 oracle on a
    slice of the rows and against the gather kernels on all of them."""
    from torchsplinekan_b200 import _native as nat
    case = make_layer_case(N, I, O, G, k, dtype, seed=51, nonuniform=True)
    x, grid, bw, sw, sc = dev(case["x"]), dev(case["grid"]), dev(case["bw"]), dev(case["sw"]), dev(case["sc"])
    y = nat.forward(x, grid, bw, sw, sc, k, nat.MODE_AUTO)
    D = 2.0 * y
    got = nat.backward(D, x, grid, bw, sw, sc, k, True, True, True, True, nat.MODE_AUTO)
    ys = nat.forward(x, grid, bw, sw, sc, k, nat.MODE_SIMT)
    want = nat.backward(D, x, grid, bw, sw, sc, k, True, True, True, True, nat.MODE_SIMT)
    f = lambda t: t.double().cpu().numpy()
    assert rel_err(f(y), f(ys)) < tol
    for a, b in zip(got, want):
        assert rel_err(f(a), f(b)) < tol * 4
    # oracle on the first 512 rows (forward and input gradient are row-wise)
    sub = {n: (v[:512] if n == "x" else v) for n, v in case.items()}
    yo, Do, gxo = oracle_step(sub)[:3]
    assert rel_err(f(y[:512]), yo) < tol
    assert rel_err(f(got[0][:512]), gxo) < tol * 4
    # without parameter gradients no workspace is needed
    gx_only = nat.backward(D, x, grid, bw, sw, sc, k, True, False, False, False, nat.MODE_AUTO)
    assert torch.equal(gx_only[0], got[0]) and gx_only[1] is None
