"""The allocation-free normalisation entry point, ``gn_norm_forward_static_f32``.

Some callers may not allocate device memory at all — a host application that has frozen its
memory plan, a plug-in called from another program's execution loop, a process under a hard
memory cap — and have no workspace to pass either. For them the library carries the scratch
of the whole-grid normalisation inside its own image. This test calls that entry point
through the C ABI twice in a row (the second call finds the first call's leftovers in the
shared scratch) and checks each result against the workspace-taking entry point.

The file name sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, x, gamma, beta, eps=1e-5):
    B, P = x.shape[0], x[0].numel()
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.empty_like(x)
    ws = torch.empty(max(int(lib.gn_norm_workspace_bytes(B, P)), 256), dtype=torch.uint8, device=x.device)
    rc = lib.gn_norm_forward_f32(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), want.data_ptr(), None, B, P,
                                 eps, ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, lib.gn_status_string(rc)
    got = torch.full_like(x, float("nan"))
    rc = lib.gn_norm_forward_static_f32(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), got.data_ptr(), B, P,
                                        eps, stream)
    assert rc == 0, lib.gn_status_string(rc)
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_norm_matches_workspace_norm_twice():
    from gridnet_b200._lib import lib

    g = torch.Generator().manual_seed(7)
    shape = (16, 24, 32)
    gamma = (1 + 0.2 * torch.randn(shape, generator=g)).cuda()
    beta = (0.3 * torch.randn(shape, generator=g)).cuda()
    # first call: 7 samples; second call: a different batch size and different data, so stale
    # partials of the first call sit in the shared scratch when it starts
    for B, scale, shift in ((7, 3.0, 1.5), (3, 0.5, -4.0)):
        x = (scale * torch.randn(B, *shape, generator=g) + shift).cuda()
        got, want = _both(lib, x, gamma, beta)
        assert torch.isfinite(got).all()
        # same kernels, same reduction order: the two entry points agree to the last bit, which is
        # well inside the 1e-4 relative / 1e-5 absolute bar the other tests use
        assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
        assert torch.equal(got, want)
        ref = torch.nn.functional.layer_norm(x, shape, gamma, beta, 1e-5)
        assert torch.allclose(got, ref, rtol=1e-4, atol=1e-5)


def test_static_scratch_norm_with_several_slices_per_sample():
    """Grids of 16384 positions and more are summed in several slices per sample, so the [sample][slice] layout
    inside the built-in scratch is in use; two calls in a row, bit-for-bit against the workspace entry point."""
    from gridnet_b200._lib import lib

    g = torch.Generator().manual_seed(11)
    shape = (32, 32, 64)  # 65536 positions
    gamma = (1 + 0.2 * torch.randn(shape, generator=g)).cuda()
    beta = (0.3 * torch.randn(shape, generator=g)).cuda()
    for B in (5, 9):
        x = (2.0 * torch.randn(B, *shape, generator=g) + 0.7).cuda()
        got, want = _both(lib, x, gamma, beta)
        assert torch.equal(got, want)
        assert torch.allclose(got, torch.nn.functional.layer_norm(x, shape, gamma, beta, 1e-5), rtol=1e-4, atol=1e-5)


def test_static_scratch_norm_limits():
    from gridnet_b200._lib import lib

    cap = lib.gn_norm_static_max_batch()
    assert cap == 256
    shape = (4, 4, 4)
    gamma = torch.ones(shape, device="cuda")
    beta = torch.zeros(shape, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # one sample too many: refused with a clear status, output untouched
    x = torch.randn(cap + 1, *shape, device="cuda")
    y = torch.full_like(x, 5.0)
    rc = lib.gn_norm_forward_static_f32(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), cap + 1, 64,
                                        1e-5, stream)
    assert rc == -9 and b"limit" in lib.gn_status_string(rc)
    torch.cuda.synchronize()
    assert (y == 5.0).all()
    # exactly at the limit works
    x = torch.randn(cap, *shape, device="cuda")
    got, want = _both(lib, x, gamma, beta)
    assert torch.equal(got, want)
    assert lib.gn_norm_forward_static_f32(None, None, None, None, 1, 64, 1e-5, stream) == -1
    assert lib.gn_norm_forward_static_f32(None, None, None, None, 0, 64, 1e-5, stream) == 0
