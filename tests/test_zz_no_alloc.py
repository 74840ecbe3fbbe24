"""The allocation-free variant of the edge statistic (kanb200_edge_abs_mean_noalloc).

It serves hosts that cannot give the library a workspace at call time because all of their
device memory is planned ahead (a serving process with a static memory plan, an operator plugin
that only ever receives its input and output tensors).  The partial sums then live in a 4 MiB
buffer compiled into the library.  The test calls the entry point through the C ABI twice in a
row -- the second call reuses the buffer with the first call's leftovers in it -- and compares with
the ordinary entry point, which gets a fresh workspace.  This file sorts last so that a run that
stops at the first failure has already seen every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

nat = pytest.importorskip("torchsplinekan_b200._native")


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _noalloc(s, H, bw, W):
    N, I, R = H.shape
    O = W.shape[0]
    a = torch.full((O, I), float("nan"), dtype=H.dtype, device=H.device)
    code = nat.F32 if H.dtype == torch.float32 else nat.F64
    with torch.cuda.device(H.device):
        rc = nat.lib().kanb200_edge_abs_mean_noalloc(code, _p(s), _p(H), _p(bw), _p(W), _p(a), N, I, O, R,
                                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, a


def _case(N, I, O, R, dtype, seed, base=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    H = torch.rand(N, I, R, device="cuda", dtype=dtype, generator=g)
    W = torch.randn(O, I, R, device="cuda", dtype=dtype, generator=g)
    s = torch.randn(N, I, device="cuda", dtype=dtype, generator=g) if base else None
    bw = torch.randn(O, I, device="cuda", dtype=dtype, generator=g) if base else None
    return s, H, bw, W


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.float64, 1e-13)])
def test_two_calls_in_a_row_match_the_workspace_entry_point(dtype, tol):
    # first call: many splits, fills a good part of the built-in buffer
    first = _case(4000, 64, 96, 8, dtype, seed=1)
    # second call: different shape and no base branch, so stale partial sums of the first call
    # sit in and around the region it uses
    second = _case(700, 40, 33, 11, dtype, seed=2, base=False)
    for s, H, bw, W in (first, second):
        rc, a = _noalloc(s, H, bw, W)
        assert rc == 0, nat.last_error()
        want = nat.edge_abs_mean(s, H, bw, W)
        torch.cuda.synchronize()
        assert torch.isfinite(a).all()
        err = (a - want).abs().max().item() / want.abs().max().item()
        assert err <= tol, err


def test_shapes_beyond_the_built_in_buffer_are_refused():
    # 2048 x 2048 edges need 16 MiB of partial sums, four times the built-in buffer.  Real
    # (zero) operands of the right sizes are passed, so even a wrong size check could not make a
    # kernel read out of bounds.
    N, I, O, R = 64, 2048, 2048, 8
    H = torch.zeros(N, I, R, device="cuda")
    W = torch.zeros(O, I, R, device="cuda")
    rc, _ = _noalloc(None, H, None, W)
    assert rc == nat.EWORKSPACE
    assert "4194304" in nat.last_error() and "workspace" in nat.last_error()
