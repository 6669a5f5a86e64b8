"""GPU parity of the whole-grid normalisation and of the fused model loop
(step + LayerNorm, gridnet/scripts/train_mnist.py:62-64) against the CPU oracle, the
golden vectors, and — at the benchmark's full size — against size-independent
properties (fused == unfused composition, batch independence, determinism)."""
import os

import numpy as np
import pytest
import torch

from oracle import gridnet_oracle as orc

from conftest import GOLDEN
from util import assert_close

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def model_params(seed, shape):
    """Model-style parameters: weights N(0, 1/27) (gridnet/__init__.py:42-45); bias, residual
    scale, gamma, beta perturbed around their initial values so that every term is exercised."""
    r = np.random.default_rng(seed)
    f = np.float32
    w = (r.standard_normal((27, *shape)) / np.sqrt(27)).astype(f)
    b = (0.1 * r.standard_normal(shape)).astype(f)
    s = (1 + 0.1 * r.standard_normal(shape)).astype(f)
    gamma = (1 + 0.1 * r.standard_normal(shape)).astype(f)
    beta = (0.1 * r.standard_normal(shape)).astype(f)
    return w, b, s, gamma, beta


def face_input(seed, B, shape):
    x = np.zeros((B, *shape), np.float32)
    x[..., 0] = np.random.default_rng(seed).standard_normal((B, *shape[:2]))
    return x


@pytest.mark.parametrize("B,shape", [(3, (16, 16, 16)), (2, (8, 24, 40)), (5, (4, 4, 4)), (1, (32, 32, 32))])
def test_grid_norm_forward_backward(B, shape):
    from gridnet_b200 import GridNormOp

    r = np.random.default_rng(20)
    x = (3 * r.standard_normal((B, *shape)) + 1.5).astype(np.float32)
    gamma = (1 + 0.2 * r.standard_normal(shape)).astype(np.float32)
    beta = (0.3 * r.standard_normal(shape)).astype(np.float32)
    gy = r.standard_normal(x.shape).astype(np.float32)
    y64 = orc.layernorm_forward(x.astype(np.float64), gamma.astype(np.float64), beta.astype(np.float64))
    gx64, gg64, gb64 = orc.layernorm_backward(x.astype(np.float64), gamma.astype(np.float64), gy.astype(np.float64))
    tx, tg, tb = (dev(a).requires_grad_(True) for a in (x, gamma, beta))
    y = GridNormOp.apply(tx, tg, tb, 1e-5)
    assert_close(y.detach().cpu().numpy(), y64, None, "norm forward")
    gx, gg, gb = torch.autograd.grad(y, (tx, tg, tb), dev(gy))
    assert_close(gx.cpu().numpy(), gx64, None, "norm gx")
    assert_close(gg.cpu().numpy(), gg64, None, "norm ggamma")
    assert_close(gb.cpu().numpy(), gb64, None, "norm gbeta")
    # and against torch's own LayerNorm on the device (what the reference's models call)
    ty = torch.nn.functional.layer_norm(tx, shape, tg, tb, 1e-5)
    assert torch.allclose(y, ty, rtol=1e-4, atol=1e-5)


def test_golden_outer_loop():
    from gridnet_b200 import outer_forward

    z = np.load(os.path.join(GOLDEN, "outer_loop.npz"))
    bs, inner, outer = (int(v) for v in z["meta"])
    args = [dev(z[k]) for k in ("w", "b", "s", "gamma", "beta", "x")]
    got = outer_forward(*args, inner, outer, bs).cpu().numpy()
    assert_close(got, z["y64"], z["y32"], "golden outer loop")


@pytest.mark.parametrize(
    "name,B,shape,bs,inner,outer",
    [
        ("C1 MNIST-shaped, full", 8, (32, 32, 32), 8, 2, 8),
        ("C2 shape, reduced batch", 2, (64, 64, 64), 8, 4, 12),
        ("C4 shape (block 4), reduced", 2, (32, 32, 32), 4, 8, 4),
        ("non-cubic", 3, (8, 16, 24), 8, 3, 5),
        ("single block", 2, (8, 8, 8), 8, 2, 3),
        ("odd batch, one sample per CTA", 1, (16, 16, 16), 8, 1, 2),
    ],
)
def test_outer_forward_matches_oracle(name, B, shape, bs, inner, outer):
    from gridnet_b200 import outer_forward

    w, b, s, gamma, beta = model_params(21, shape)
    if name.startswith("C1"):
        # MNIST-style input: 28x28 pixels in [0,1] zero-padded onto the [..., 0] face
        # (gridnet/scripts/train_mnist.py:59-60)
        x = np.zeros((B, *shape), np.float32)
        x[:, 2:30, 2:30, 0] = np.random.default_rng(22).random((B, 28, 28))
    else:
        x = face_input(22, B, shape)
    a64 = [a.astype(np.float64) for a in (w, b, s, gamma, beta, x)]
    ref64 = orc.outer_forward(*a64, inner, outer, bs)
    ref32 = orc.outer_forward(w, b, s, gamma, beta, x, inner, outer, bs)
    got = outer_forward(*(dev(a) for a in (w, b, s, gamma, beta, x)), inner, outer, bs).cpu().numpy()
    assert_close(got, ref64, ref32, name)


def test_outer_forward_edge_cases():
    from gridnet_b200 import outer_forward

    shape = (8, 8, 8)
    w, b, s, gamma, beta = (dev(a) for a in model_params(23, shape))
    x = dev(face_input(24, 2, shape))
    assert torch.equal(outer_forward(w, b, s, gamma, beta, x, 2, 0, 8), x)  # no outer steps
    e = torch.empty(0, *shape, device="cuda")
    assert outer_forward(w, b, s, gamma, beta, e, 2, 3, 8).shape == e.shape
    # zero inner iterations: the loop is LayerNorm applied `outer` times
    got = outer_forward(w, b, s, gamma, beta, x, 0, 2, 8)
    want = x
    for _ in range(2):
        want = torch.nn.functional.layer_norm(want, shape, gamma, beta, 1e-5)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    with pytest.raises(AssertionError):
        outer_forward(w, b, s, gamma[:4], beta, x, 2, 2, 8)


def test_full_size_properties_c2():
    """The benchmark configuration at full size (64^3, block 8, 4 inner x 12 outer, batch 64): too slow
    for the scalar oracle in float64 at full batch, so parity is carried by properties."""
    from gridnet_b200 import GridnetCudaOp, GridNormOp, outer_forward

    shape, B, bs, inner, outer = (64, 64, 64), 64, 8, 4, 12
    w, b, s, gamma, beta = (dev(a) for a in model_params(25, shape))
    x = dev(face_input(26, B, shape))
    y = outer_forward(w, b, s, gamma, beta, x, inner, outer, bs)
    assert torch.isfinite(y).all()
    # (1) deterministic: a second run is bit-identical
    assert torch.equal(y, outer_forward(w, b, s, gamma, beta, x, inner, outer, bs))
    # (2) the fused loop equals the unfused composition of the two public ops
    h = x
    for _ in range(outer):
        h = GridnetCudaOp.apply(w, b, s, h, inner, bs, 1e-5, False, "silu")
        h = GridNormOp.apply(h, gamma, beta, 1e-5)
    assert torch.allclose(y, h, rtol=1e-4, atol=1e-5), (y - h).abs().max().item()
    # (3) samples are independent: any sub-batch gives the same rows
    sub = outer_forward(w, b, s, gamma, beta, x[5:8].contiguous(), inner, outer, bs)
    assert torch.allclose(y[5:8], sub, rtol=1e-5, atol=1e-6)
    # (4) every sample is normalised: mean beta-ish, variance gamma-ish (gamma, beta near 1, 0)
    flat = ((y - beta) / gamma).flatten(1)
    assert flat.mean(1).abs().max() < 1e-3
    assert (flat.var(1, unbiased=False) - 1).abs().max() < 1e-2
    # (5) three samples against the float64 oracle
    a64 = [t.cpu().numpy().astype(np.float64) for t in (w, b, s, gamma, beta)]
    idx = [0, 31, 63]
    x64 = x[idx].cpu().numpy().astype(np.float64)
    ref64 = orc.outer_forward(*a64, x64, inner, outer, bs)
    ref32 = orc.outer_forward(*(a.astype(np.float32) for a in a64), x64.astype(np.float32), inner, outer, bs)
    assert_close(y[idx].cpu().numpy(), ref64, ref32, "C2 full size, sampled rows")


@pytest.mark.parametrize("B,shape,inner,outer,act", [
    (64, (16, 16, 16), 4, 3, "silu"),      # one full group; blocks on every face of the grid
    (5, (16, 16, 16), 2, 3, "silu"),       # mostly padding: the zero-padded last group
    (70, (8, 16, 24), 3, 2, "tanh"),       # two groups, non-cubic grid, odd inner count
    (64, (8, 8, 8), 1, 2, "leaky_relu"),   # a single block (only stale halo), one inner iteration
    (128, (24, 8, 16), 2, 2, "relu"),      # two full groups, z is the long axis
])
def test_large_batch_kernel_matches_patch_kernel_and_oracle(B, shape, inner, outer, act):
    """The large-batch step kernel (lanes own samples, a block split over a cluster of two CTAs, activations
    interleaved by 64 samples) must give the same fused loop as the register-patch kernel and the oracle."""
    from gridnet_b200 import outer_forward, outer_forward_failed, outer_forward_workspace
    from gridnet_b200._lib import lib

    w, b, s, gamma, beta = model_params(27, shape)
    x = face_input(28, B, shape)
    x[:, 1::3, ::2, 1:] = 0.3 * np.random.default_rng(31).standard_normal(x[:, 1::3, ::2, 1:].shape)
    args = [dev(a) for a in (w, b, s, gamma, beta, x)]
    ws = outer_forward_workspace(B, shape, 8, args[0].device)
    try:
        assert lib.gn_config_set(b"outer_kernel", 1) == 0
        base = outer_forward(*args, inner, outer, 8, act)
        assert lib.gn_config_set(b"outer_kernel", 2) == 0
        got = outer_forward(*args, inner, outer, 8, act, workspace=ws)
        again = outer_forward(*args, inner, outer, 8, act, workspace=ws)
    finally:
        lib.gn_config_set(b"outer_kernel", 0)
    assert not outer_forward_failed(ws, B, shape, 8)
    assert torch.equal(got, again), "two runs differ"
    assert torch.allclose(got, base, rtol=2e-5, atol=2e-6), (got - base).abs().max().item()
    a64 = [a.astype(np.float64) for a in (w, b, s, gamma, beta, x)]
    assert_close(got.cpu().numpy(), orc.outer_forward(*a64, inner, outer, 8, activation=act), None,
                 f"large-batch kernel B={B}")


@pytest.mark.parametrize("B,shape,inner,outer,act", [
    (8, (32, 32, 32), 2, 8, "silu"),       # the MNIST-shaped configuration in full
    (5, (16, 16, 16), 3, 2, "tanh"),       # samples that do not divide over the CTAs
    (1, (8, 8, 8), 1, 1, "relu"),          # one block, one sample, one step
    (3, (8, 24, 16), 2, 5, "leaky_relu"),  # non-cubic grid
])
def test_persistent_kernel_matches_step_by_step_loop_and_oracle(B, shape, inner, outer, act):
    """The whole loop as one cooperative kernel (what small problems get by default) against the loop of one
    launch per outer step and against the oracle; two runs give the same bits."""
    from gridnet_b200 import outer_forward, outer_forward_failed, outer_forward_workspace
    from gridnet_b200._lib import lib

    w, b, s, gamma, beta = model_params(81, shape)
    x = face_input(82, B, shape)
    args = [dev(a) for a in (w, b, s, gamma, beta, x)]
    ws = outer_forward_workspace(B, shape, 8, args[0].device)
    try:
        assert lib.gn_config_set(b"outer_kernel", 1) == 0
        base = outer_forward(*args, inner, outer, 8, act)
        assert lib.gn_config_set(b"outer_kernel", 3) == 0
        got = outer_forward(*args, inner, outer, 8, act, workspace=ws)
        again = outer_forward(*args, inner, outer, 8, act, workspace=ws)
    finally:
        lib.gn_config_set(b"outer_kernel", 0)
    assert not outer_forward_failed(ws, B, shape, 8)
    assert torch.equal(got, again)
    assert torch.allclose(got, base, rtol=2e-5, atol=2e-6), (got - base).abs().max().item()
    auto = outer_forward(*args, inner, outer, 8, act)  # small problems take the persistent kernel by themselves
    assert torch.equal(auto, got)
    a64 = [a.astype(np.float64) for a in (w, b, s, gamma, beta, x)]
    assert_close(got.cpu().numpy(), orc.outer_forward(*a64, inner, outer, 8, activation=act), None, f"persistent kernel B={B}")


def test_packed_parameters_are_rebuilt_when_parameters_change():
    """A reused workspace keeps the re-ordered parameters of the large-batch kernel; changing a parameter in place,
    passing another parameter tensor, or scribbling over the workspace must all lead to a rebuild."""
    from gridnet_b200 import outer_forward, outer_forward_workspace

    shape, B, inner, outer = (16, 16, 16), 64, 2, 2
    w, b, s, gamma, beta = (dev(a) for a in model_params(71, shape))
    x = dev(face_input(72, B, shape))
    ws = outer_forward_workspace(B, shape, 8, x.device)
    fresh = lambda *p: outer_forward(*p, x, inner, outer, 8)  # no workspace given: always rebuilt
    y1 = outer_forward(w, b, s, gamma, beta, x, inner, outer, 8, workspace=ws)
    assert torch.equal(y1, outer_forward(w, b, s, gamma, beta, x, inner, outer, 8, workspace=ws))  # reused
    with torch.no_grad():
        w.mul_(1.5)  # in place: same tensor, new version
    y2 = outer_forward(w, b, s, gamma, beta, x, inner, outer, 8, workspace=ws)
    assert torch.equal(y2, fresh(w, b, s, gamma, beta)) and not torch.equal(y2, y1)
    gamma2 = gamma * 0.5  # another tensor
    y3 = outer_forward(w, b, s, gamma2, beta, x, inner, outer, 8, workspace=ws)
    assert torch.equal(y3, fresh(w, b, s, gamma2, beta)) and not torch.equal(y3, y2)
    ws.fill_(7)  # the caller used the memory for something else in between
    y4 = outer_forward(w, b, s, gamma2, beta, x, inner, outer, 8, workspace=ws)
    assert torch.equal(y4, y3)


def test_large_batch_step_building_blocks():
    """gn_pair64_* through the C ABI: interleave -> one step without normalisation -> de-interleave equals the
    plain step op; interleave -> de-interleave is the identity."""
    from gridnet_b200 import GridnetCudaOp
    from gridnet_b200.backend_cuda import pair64_deinterleave, pair64_interleave, pair64_pack_weights, pair64_step

    B, shape, inner = 64, (16, 8, 24), 3
    w, b, s, _, _ = model_params(33, shape)
    x = np.random.default_rng(34).standard_normal((B, *shape)).astype(np.float32)
    tw, tb, ts, tx = (dev(a) for a in (w, b, s, x))
    xi = pair64_interleave(tx)
    assert torch.equal(pair64_deinterleave(xi, B, shape), tx)
    packed = pair64_pack_weights(tw, tb, ts)
    yi = torch.empty_like(xi)
    flag = torch.zeros(1, dtype=torch.int32, device=tx.device)
    pair64_step(packed, xi, yi, B, shape, inner, "silu", error_flag=flag)
    got = pair64_deinterleave(yi, B, shape)
    assert int(flag.item()) == 0
    want = GridnetCudaOp.apply(tw, tb, ts, tx, inner, 8, 1e-5, False, "silu")
    assert torch.allclose(got, want, rtol=2e-5, atol=2e-6), (got - want).abs().max().item()
    ref = orc.step_forward(w.astype(np.float64), b.astype(np.float64), s.astype(np.float64), x.astype(np.float64),
                           inner, 8, normalize=False, activation="silu")
    assert_close(got.cpu().numpy(), ref, None, "large-batch single step")


def test_outer_forward_reports_no_device_failure():
    from gridnet_b200 import outer_forward, outer_forward_failed, outer_forward_workspace

    shape, B = (16, 16, 16), 4
    w, b, s, gamma, beta = (dev(a) for a in model_params(29, shape))
    x = dev(face_input(30, B, shape))
    ws = outer_forward_workspace(B, shape, 8, x.device)
    ws.fill_(255)  # the flag must be cleared by the call itself
    outer_forward(w, b, s, gamma, beta, x, 2, 3, 8, workspace=ws)
    assert not outer_forward_failed(ws, B, shape, 8)


def test_grid_norm_with_more_than_65535_samples():
    """The batch sits in the first grid dimension of the norm kernels, so it is not capped at 65535."""
    from gridnet_b200 import GridNormOp

    B, shape = 70001, (4, 4, 4)
    g = torch.Generator(device="cuda").manual_seed(5)
    x = 2 * torch.randn(B, *shape, device="cuda", generator=g) + 0.5
    gamma = 1 + 0.1 * torch.randn(shape, device="cuda", generator=g)
    beta = 0.1 * torch.randn(shape, device="cuda", generator=g)
    y = GridNormOp.apply(x, gamma, beta, 1e-5)
    ref = torch.nn.functional.layer_norm(x, shape, gamma, beta, 1e-5)
    assert torch.allclose(y, ref, rtol=1e-4, atol=1e-5)
    idx = [0, 1, 65535, 65536, B - 1]
    want = orc.layernorm_forward(x[idx].cpu().numpy().astype(np.float64), gamma.cpu().numpy().astype(np.float64),
                                 beta.cpu().numpy().astype(np.float64))
    assert_close(y[idx].cpu().numpy(), want, None, "norm, large batch")


def test_forward_on_planes_beyond_the_register_prefetch_limit():
    """A grid whose (N, K) plane is too large for the 20-bit offsets of the plain-load path still takes the tuned
    forward kernel when bulk tensor copies apply (and stays correct): 8 x 344 x 344, one sample."""
    from gridnet_b200 import GridnetCudaOp
    from gridnet_b200._lib import lib

    shape = (8, 344, 344)
    r = np.random.default_rng(41)
    w = (r.standard_normal((27, *shape)) / np.sqrt(27)).astype(np.float32)
    b = (0.1 * r.standard_normal(shape)).astype(np.float32)
    s = (1 + 0.1 * r.standard_normal(shape)).astype(np.float32)
    x = r.standard_normal((1, *shape)).astype(np.float32)
    tw, tb, ts, tx = (dev(a) for a in (w, b, s, x))
    got = GridnetCudaOp.apply(tw, tb, ts, tx, 2, 8, 1e-5, False, "silu")
    # the fused entry point only exists on the tuned path: it must accept this shape now
    y2 = torch.empty_like(tx)
    rc = lib.gn_step_forward_fused_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), y2.data_ptr(), None, None,
                                       None, None, 1, *shape, 2, 8, 2, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.gn_status_string(rc)
    assert torch.equal(got, y2)
    ref = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), 2, 8, normalize=False, activation="silu")
    assert_close(got.cpu().numpy(), ref, None, "large plane")


def test_device_failure_reports_can_be_seen():
    """The host side of the bounded-wait contract: a set flag is what the accessors report. Nothing here makes a
    kernel's wait run out; the flag in the workspace and the library's status word are written by hand."""
    import gridnet_b200 as gb
    from gridnet_b200._lib import lib

    shape, B = (16, 16, 16), 4
    w, b, s, gamma, beta = (dev(a) for a in model_params(29, shape))
    x = dev(face_input(30, B, shape))
    ws = gb.outer_forward_workspace(B, shape, 8, x.device)
    gb.outer_forward(w, b, s, gamma, beta, x, 2, 3, 8, workspace=ws)
    assert not gb.outer_forward_failed(ws, B, shape, 8)
    off = int(lib.gn_outer_forward_error_flag_offset(B, *shape, 8))
    ws[off:off + 4].view(torch.int32).fill_(1)  # what a kernel does when its wait gives up
    assert gb.outer_forward_failed(ws, B, shape, 8)
    gb.outer_forward(w, b, s, gamma, beta, x, 2, 3, 8, workspace=ws)  # the next call clears it
    assert not gb.outer_forward_failed(ws, B, shape, 8)

    # the status word of the entry points that have no workspace
    gb.device_status(clear=True)
    y = gb.GridnetCudaOp.apply(w, b, s, x, 2, 8, 1e-5, False, "silu")  # tuned forward, bulk tile copies
    y2 = gb.GatedGridnetCudaOp.apply(torch.stack([w, w], 1).contiguous(), torch.stack([b, b]).contiguous(), x, 2, 8, "tanh")
    assert torch.isfinite(y).all() and torch.isfinite(y2).all()
    assert gb.device_status(clear=False) is False
    assert lib.gn_device_status_set(1) == 0
    assert gb.device_status(clear=False) is True  # not cleared by reading with clear=False
    assert gb.device_status(clear=True) is True
    assert gb.device_status(clear=True) is False


@pytest.mark.parametrize("name,shape,B,bs,inner", [("C3", (128, 128, 128), 16, 8, 2), ("C4", (64, 64, 64), 128, 4, 8)])
def test_full_size_step_gradients(name, shape, B, bs, inner):
    """One outer step of the forward + backward configurations on their full grids (C4 at its full batch,
    C3 at 16 of its 256 samples: the kernels walk the batch sample by sample, so the batch size only changes
    how CTAs split it). The scalar oracle is too slow here, so parity is carried by properties: the tuned
    four-kernel backward against the independent one-kernel backward, bit-reproducibility, independence of
    the samples, and two samples against the float64 oracle."""
    from gridnet_b200 import GridnetCudaOp
    from gridnet_b200._lib import lib

    w, b, s, _, _ = (dev(a) for a in model_params(61, shape))
    g = torch.Generator(device="cuda").manual_seed(62)
    x = torch.randn(B, *shape, device="cuda", generator=g)
    gy = torch.randn(B, *shape, device="cuda", generator=g)
    M, N, K = shape
    stream = torch.cuda.current_stream().cuda_stream

    def backward(tuned, xs, gys):
        n = xs.shape[0]
        outs = [torch.empty_like(t) for t in (w, b, s, xs)]
        if tuned:
            need = lib.gn_step_backward_workspace_bytes(n, M, N, K, inner, bs, 0, 4)
            assert need > 0
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            rc = lib.gn_step_backward_ws_f32(w.data_ptr(), b.data_ptr(), s.data_ptr(), xs.data_ptr(), gys.data_ptr(),
                                             *(t.data_ptr() for t in outs), n, M, N, K, inner, bs, 1e-5, 0, 2,
                                             ws.data_ptr(), ws.numel(), stream)
            assert rc == 0 and int(ws.view(torch.int32)[lib.gn_step_backward_error_flag_offset(n, M, N, K, inner) // 4]) == 0
        else:
            rc = lib.gn_step_backward_f32(w.data_ptr(), b.data_ptr(), s.data_ptr(), xs.data_ptr(), gys.data_ptr(),
                                          *(t.data_ptr() for t in outs), n, M, N, K, inner, bs, 1e-5, 0, 2, stream)
            assert rc == 0
        return outs

    tuned = backward(True, x, gy)
    again = backward(True, x, gy)
    plain = backward(False, x, gy)
    for name_, a, a2, p in zip(("gw", "gb", "gs", "gx"), tuned, again, plain):
        assert torch.isfinite(a).all(), name_
        assert torch.equal(a, a2), name_  # no atomics: bit-reproducible
        scale = p.abs().max().item()
        assert (a - p).abs().max().item() <= 2e-4 * scale, (name_, (a - p).abs().max().item(), scale)
    # grad_x of a sample does not depend on the rest of the batch
    sub = backward(True, x[3:5].contiguous(), gy[3:5].contiguous())
    assert torch.allclose(tuned[3][3:5], sub[3], rtol=1e-5, atol=1e-6 * tuned[3].abs().max().item())
    # forward and grad_x of two samples against the float64 oracle (parameter gradients of those two
    # samples alone come with it)
    idx = [0, B - 1]
    a64 = [t.cpu().numpy().astype(np.float64) for t in (w, b, s)]
    x64, gy64 = (t[idx].cpu().numpy().astype(np.float64) for t in (x, gy))
    y = GridnetCudaOp.apply(w, b, s, x, inner, bs, 1e-5, False, "silu")
    ref_y = orc.step_forward(*a64, x64, inner, bs, 1e-5, False, "silu")
    ref_y32 = orc.step_forward(*(a.astype(np.float32) for a in a64), x64.astype(np.float32), inner, bs, 1e-5, False, "silu")
    assert_close(y[idx].cpu().numpy(), ref_y, ref_y32, f"{name} forward, sampled rows")
    ref_g = orc.step_backward(*a64, x64, gy64, inner, bs, 1e-5, False, "silu")
    ref_g32 = orc.step_backward(*(a.astype(np.float32) for a in a64), x64.astype(np.float32), gy64.astype(np.float32),
                                inner, bs, 1e-5, False, "silu")
    two = backward(True, x[idx].contiguous(), gy[idx].contiguous())
    for name_, a, r, n32 in zip(("gw", "gb", "gs", "gx"), two, ref_g, ref_g32):
        assert_close(a.cpu().numpy(), r, n32, f"{name} {name_}, two samples")
