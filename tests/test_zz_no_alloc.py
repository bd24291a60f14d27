"""The scratch-free RMSNorm backward (ctdk_rmsnorm_bwd_static) against the regular entry point.

It exists for hosts that cannot pass scratch memory and cannot let the library allocate: a
trainer whose own arena already owns all of HBM, or a step loop that must not contain
cudaMalloc / cudaFree because they stall every stream. Both entry points run the same kernels,
only the home of the per-CTA dw partial rows differs, so dx must be bit-identical and dw equal
up to the summation order of the partial rows (the static variant caps the grid at 256 CTAs).
The check is made on two calls in a row because every call shares the one built-in array and
sees what the previous call left in it. This file is collected last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_both(rows, H, seed, accumulate, add_to_dx, offset=0, want_inputs=False):
    """offset: floats by which the dx buffer is shifted off its 16-byte alignment."""
    from emberlm_b200 import lib
    g = torch.Generator(device="cuda").manual_seed(seed)
    dy = torch.randn(rows, H, device="cuda", generator=g)
    x = torch.randn(rows, H, device="cuda", generator=g)
    w = torch.rand(H, device="cuda", generator=g) + 0.5
    dx0 = torch.randn(rows * H + offset, device="cuda", generator=g)[offset:].view(rows, H)
    dw0 = torch.randn(H, device="cuda", generator=g)
    s = torch.cuda.current_stream().cuda_stream
    dx_a, dw_a = _clone_like(dx0, offset), dw0.clone()
    scratch = torch.empty(lib.raw().ctdk_rmsnorm_bwd_scratch_floats(H), device="cuda")
    lib.call("ctdk_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), dx_a.data_ptr(), dw_a.data_ptr(),
             scratch.data_ptr(), rows, H, 1e-5, int(accumulate), int(add_to_dx), s)
    dx_b, dw_b = _clone_like(dx0, offset), dw0.clone()
    lib.call("ctdk_rmsnorm_bwd_static", dy.data_ptr(), x.data_ptr(), w.data_ptr(), dx_b.data_ptr(),
             dw_b.data_ptr(), rows, H, 1e-5, int(accumulate), int(add_to_dx), s)
    torch.cuda.synchronize()
    if want_inputs:
        return dx_a, dw_a, dx_b, dw_b, (dy, x, w, dx0, dw0)
    return dx_a, dw_a, dx_b, dw_b


def _clone_like(t, offset):
    """A copy of t with the same (mis)alignment as the original buffer."""
    if offset == 0:
        return t.clone()
    buf = torch.empty(t.numel() + offset, device=t.device, dtype=t.dtype)
    out = buf[offset:].view(t.shape)
    out.copy_(t)
    return out


def test_static_scratch_variant_matches_regular_entry_point_twice_in_a_row():
    # second call: fewer rows and a narrower H than the first, so stale partial rows and stale
    # columns from call one are still sitting in the array
    for rows, H, seed, acc, add in [(3000, 960, 1, False, False), (37, 576, 2, True, True)]:
        dx_a, dw_a, dx_b, dw_b = _call_both(rows, H, seed, acc, add)
        assert torch.equal(dx_a, dx_b)
        np.testing.assert_allclose(dw_b.cpu().numpy(), dw_a.cpu().numpy(), atol=1e-4 * np.sqrt(rows), rtol=1e-4)


def test_static_scratch_variant_widest_row_unaligned_pointer_and_oracle():
    """The widest accepted row (H = 4096: four float4 per thread, last row and column of the
    built-in array in use with 300 > 256 rows), a dx pointer 4 bytes off its 16-byte alignment
    with H % 4 == 0 (the scalar kernel), and the static entry point directly against the numpy
    oracle (oracle/ops.py rms_norm_backward)."""
    from oracle import ops as oo
    for rows, H, seed, acc, add, off in [(300, 4096, 4, False, True, 0), (50, 960, 5, True, False, 1)]:
        dx_a, dw_a, dx_b, dw_b, (dy, x, w, dx0, dw0) = _call_both(rows, H, seed, acc, add, offset=off, want_inputs=True)
        assert torch.equal(dx_a, dx_b)
        np.testing.assert_allclose(dw_b.cpu().numpy(), dw_a.cpu().numpy(), atol=1e-4 * np.sqrt(rows), rtol=1e-4)
        rdx, rdw = oo.rms_norm_backward(dy.cpu().numpy(), x.cpu().numpy(), w.cpu().numpy(), 1e-5)
        want_dx = rdx + (dx0.cpu().numpy() if add else 0.0)
        want_dw = rdw + (dw0.cpu().numpy() if acc else 0.0)
        np.testing.assert_allclose(dx_b.cpu().numpy(), want_dx, atol=2e-5, rtol=2e-5)
        np.testing.assert_allclose(dw_b.cpu().numpy(), want_dw, atol=1e-4 * np.sqrt(rows), rtol=1e-4)


def test_static_scratch_variant_generic_width_and_limits():
    from emberlm_b200 import lib
    dx_a, dw_a, dx_b, dw_b = _call_both(50, 6, 3, False, False)   # scalar kernel path
    assert torch.equal(dx_a, dx_b)
    np.testing.assert_allclose(dw_b.cpu().numpy(), dw_a.cpu().numpy(), atol=1e-4, rtol=1e-4)
    t = torch.zeros(4, 8192, device="cuda")
    w = torch.ones(8192, device="cuda")
    rc = lib.raw().ctdk_rmsnorm_bwd_static(t.data_ptr(), t.data_ptr(), w.data_ptr(), t.data_ptr(), w.data_ptr(),
                                           4, 8192, 1e-5, 0, 0, None)
    assert rc == lib.CTDK_EINVAL and "exceeds the built-in scratch" in lib.last_error()
