"""Module wrappers and the host-buffer pipeline on the GPU: the fused model loop equals the
step-by-step composition with autograd, reference-style state dicts load, training gradients
flow through both ops, and HostPipelinedForward returns what outer_forward returns."""
import numpy as np
import pytest
import torch

from oracle import gridnet_oracle as orc

pytestmark = pytest.mark.gpu


def test_model_fused_inference_equals_training_path_and_oracle():
    import gridnet_b200 as gb

    torch.manual_seed(0)
    shape = (16, 16, 16)
    dev = torch.device("cuda")
    model = gb.GridnetModel(shape, inner_iters=2, outer_iters=3, block_size=8, device=dev)
    with torch.no_grad():
        model.network.bias.normal_(0, 0.1)
        model.norm.weight.normal_(1, 0.1)
        model.norm.bias.normal_(0, 0.1)
    assert set(model.state_dict()) == {"network.weight", "network.bias", "network.residual_scale", "norm.weight", "norm.bias"}
    x = torch.zeros(3, *shape, device=dev)
    x[..., 0] = torch.randn(3, 16, 16, device=dev)
    with torch.no_grad():
        fused = model(x)
    stepwise = model(x)  # grad enabled: GridnetCudaOp + GridNormOp per outer step
    assert stepwise.requires_grad
    assert torch.allclose(fused, stepwise, rtol=1e-4, atol=1e-5)
    sd = {k: v.detach().cpu().numpy().astype(np.float64) for k, v in model.state_dict().items()}
    want = orc.outer_forward(sd["network.weight"], sd["network.bias"], sd["network.residual_scale"], sd["norm.weight"],
                             sd["norm.bias"], x.cpu().numpy().astype(np.float64), 2, 3, 8)
    err = np.abs(fused.cpu().numpy() - want)
    assert (err <= 1e-5 + 1e-4 * np.abs(want)).all()
    # a training step: the gradients of all five parameters and of the input against the oracle's chain
    # step_backward o layernorm_backward over the three outer steps (float64 oracle, float32 oracle for the noise)
    from util import assert_close

    gy = torch.linspace(-1, 1, stepwise.numel(), device=dev).view_as(stepwise).contiguous()
    xg = x.clone().requires_grad_(True)
    out = model(xg)
    names = ["network.weight", "network.bias", "network.residual_scale", "norm.weight", "norm.bias"]
    params = dict(model.named_parameters())
    grads = torch.autograd.grad(out, [params[n] for n in names] + [xg], gy)
    args64 = [sd[n] for n in names] + [x.cpu().numpy().astype(np.float64), gy.cpu().numpy().astype(np.float64)]
    want64 = orc.outer_backward(*args64, 2, 3, 8)
    want32 = orc.outer_backward(*(a.astype(np.float32) for a in args64), 2, 3, 8)
    for name, g, r64, r32 in zip(names + ["input"], grads, want64, want32):
        assert_close(g.cpu().numpy(), r64, r32, f"model gradient of {name}")
    # the fused training node against the step-by-step composition of the two autograd ops (same library kernels
    # underneath, different order of a few float32 operations), with the forward stash on and off
    for keep in (False, True):
        previous = gb.keep_forward_stash(keep)
        try:
            xs = x.clone().requires_grad_(True)
            h = xs
            for _ in range(3):
                h = model.norm(model.network(h))
            want = torch.autograd.grad(h, [params[n] for n in names] + [xs], gy)
            xf = x.clone().requires_grad_(True)
            outf = model(xf)
            got = torch.autograd.grad(outf, [params[n] for n in names] + [xf], gy)
        finally:
            gb.keep_forward_stash(previous)
        assert torch.allclose(outf, h, rtol=1e-5, atol=1e-6)
        for name, a, c in zip(names + ["input"], got, want):
            assert torch.allclose(a, c, rtol=1e-3, atol=1e-4 * (1 + c.abs().max().item())), (name, keep, (a - c).abs().max().item())


@pytest.mark.parametrize("block,shape,B", [(8, (16, 8, 24), 5), (4, (8, 16, 8), 3)])
def test_fused_training_loop_op(block, shape, B):
    """FusedLoopTrainOp directly: both block sizes, odd batch, a non-cubic grid, zero outer iterations, and
    gradients against the float64 oracle chain."""
    import gridnet_b200 as gb
    from util import assert_close

    r = np.random.default_rng(61)
    f = np.float32
    w = (r.standard_normal((27, *shape)) / np.sqrt(27)).astype(f)
    b = (0.1 * r.standard_normal(shape)).astype(f)
    s = (1 + 0.1 * r.standard_normal(shape)).astype(f)
    ga = (1 + 0.1 * r.standard_normal(shape)).astype(f)
    be = (0.1 * r.standard_normal(shape)).astype(f)
    x = r.standard_normal((B, *shape)).astype(f)
    gy = r.standard_normal((B, *shape)).astype(f)
    inner, outer = 2, 3
    leaves = [torch.from_numpy(a).cuda().requires_grad_(True) for a in (w, b, s, ga, be, x)]
    assert gb.FusedLoopTrainOp.supported(leaves[0], leaves[5], inner, block)
    y = gb.FusedLoopTrainOp.apply(*leaves, inner, outer, block, "silu", 1e-5)
    grads = torch.autograd.grad(y, leaves, torch.from_numpy(gy).cuda())
    a64 = [a.astype(np.float64) for a in (w, b, s, ga, be, x)]
    assert_close(y.detach().cpu().numpy(), orc.outer_forward(*a64, inner, outer, block), None, "fused training forward")
    want64 = orc.outer_backward(*a64, gy.astype(np.float64), inner, outer, block)
    want32 = orc.outer_backward(w, b, s, ga, be, x, gy, inner, outer, block)
    for name, g, r64, r32 in zip(("weight", "bias", "scale", "gamma", "beta", "input"), grads, want64, want32):
        assert_close(g.cpu().numpy(), r64, r32, f"fused training gradient of {name} (block {block})")
    y0 = gb.FusedLoopTrainOp.apply(*leaves, inner, 0, block, "silu", 1e-5)
    assert torch.equal(y0, leaves[5])


def test_gated_model_and_readout_run():
    import gridnet_b200 as gb

    dev = torch.device("cuda")
    shape = (8, 8, 8)
    model = gb.GridnetModel(shape, 2, 2, 4, dev, activation="tanh", gated=True)
    ro = gb.Readout(shape, 10, dev)
    x = torch.randn(2, *shape, device=dev)
    out = ro(model(x))
    assert out.shape == (2, 10)
    out.sum().backward()
    assert model.network.weight.grad.abs().sum() > 0
    with pytest.raises(RuntimeError):
        gb.gridnet_step(torch.zeros(27, *shape), torch.zeros(shape), torch.zeros(shape), torch.zeros(1, *shape), 1, 8)


def test_host_pipelined_forward_matches_outer_forward():
    import gridnet_b200 as gb

    g = torch.Generator().manual_seed(3)
    shape, B = (16, 16, 16), 4
    w = (torch.randn(27, *shape, generator=g) / 27 ** 0.5).cuda()
    b = (0.1 * torch.randn(shape, generator=g)).cuda()
    s = torch.ones(shape).cuda()
    gamma = (1 + 0.1 * torch.randn(shape, generator=g)).cuda()
    beta = (0.1 * torch.randn(shape, generator=g)).cuda()
    hx = [torch.randn(B, *shape, generator=g).pin_memory() for _ in range(5)]
    hy = [torch.empty(B, *shape).pin_memory() for _ in range(5)]
    pipe = gb.HostPipelinedForward(w, b, s, gamma, beta, B, 2, 3, 8)
    for xi, yi in zip(hx, hy):  # more batches than buffer sets: buffers are reused
        pipe.submit(xi, yi)
    pipe.synchronize()
    for xi, yi in zip(hx, hy):
        want = gb.outer_forward(w, b, s, gamma, beta, xi.cuda(), 2, 3, 8).cpu()
        assert torch.equal(yi, want)


@pytest.mark.parametrize("block", [8, 4])
def test_fused_loop_variants_equal_the_step_by_step_composition(block):
    """Per-step parameters (with gradients, through FusedLoopSeparateTrainOp) and the residual form (without,
    through fused_loop_forward) against the composition of the step op and the norm op, which the other tests pin
    to the oracle (gridnet/scripts/train_imagenet.py:76-86)."""
    import gridnet_b200 as gb

    g = torch.Generator().manual_seed(17)
    shape, B, inner, outer = (16, 8, 16), 3, 2, 3
    dev = "cuda"
    mk = lambda *sz, scale=1.0, shift=0.0: (shift + scale * torch.randn(*sz, generator=g)).to(dev)
    plist = [(mk(27, *shape, scale=27 ** -0.5), mk(*shape, scale=0.1), mk(*shape, scale=0.1, shift=1.0))
             for _ in range(outer)]
    gamma, beta = mk(*shape, scale=0.1, shift=1.0), mk(*shape, scale=0.1)
    x, gy = mk(B, *shape), mk(B, *shape)

    def composition(leaves_p, ga, be, xin, residual):
        h = xin
        for w, b, s in leaves_p:
            if residual:
                n = gb.GridNormOp.apply(h, ga, be, 1e-5)
                h = h + (gb.GridnetCudaOp.apply(w, b, s, n, inner, block, 1e-5, False, "silu") - n)
            else:
                h = gb.GridNormOp.apply(gb.GridnetCudaOp.apply(w, b, s, h, inner, block, 1e-5, False, "silu"), ga, be, 1e-5)
        return h

    # inference, both forms
    with torch.no_grad():
        for residual in (False, True):
            want = composition(plist, gamma, beta, x, residual)
            got = gb.fused_loop_forward(plist, gamma, beta, x, inner, block, "silu", 1e-5, outer_residual=residual)
            assert torch.allclose(got, want, rtol=1e-4, atol=1e-5), (residual, (got - want).abs().max().item())
        assert torch.equal(gb.fused_loop_forward([], gamma, beta, x, inner, block, "silu", 1e-5, outer_residual=True), x)

    # training with per-step parameters
    def leaves():
        ps = [tuple(t.clone().requires_grad_(True) for t in p) for p in plist]
        return ps, gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True), x.clone().requires_grad_(True)

    ps, ga, be, xl = leaves()
    flat = [t for p in ps for t in p]
    want_y = composition(ps, ga, be, xl, False)
    want = torch.autograd.grad(want_y, [ga, be, xl] + flat, gy)
    ps, ga, be, xl = leaves()
    flat = [t for p in ps for t in p]
    got_y = gb.FusedLoopSeparateTrainOp.apply(ga, be, xl, inner, block, "silu", 1e-5, *flat)
    got = torch.autograd.grad(got_y, [ga, be, xl] + flat, gy)
    assert torch.allclose(got_y, want_y, rtol=1e-4, atol=1e-5)
    for i, (a, c) in enumerate(zip(got, want)):
        assert torch.allclose(a, c, rtol=1e-3, atol=1e-4 * (1 + c.abs().max().item())), (i, (a - c).abs().max().item())

    # training in the residual form: per-step parameters, then one shared set, with the stash forced on and off
    for shared in (False, True):
        for keep in (True, False):
            previous = gb.keep_forward_stash(keep)
            try:
                ps, ga, be, xl = leaves()
                if shared:
                    ps = [ps[0]] * outer
                uniq = list(ps[0]) if shared else [t for p in ps for t in p]
                want_y = composition(ps, ga, be, xl, True)
                want = torch.autograd.grad(want_y, [ga, be, xl] + uniq, gy)
                ps, ga, be, xl = leaves()
                if shared:
                    ps = [ps[0]] * outer
                uniq = list(ps[0]) if shared else [t for p in ps for t in p]
                got_y = gb.FusedLoopResidualTrainOp.apply(ga, be, xl, inner, block, "silu", 1e-5, outer, *uniq)
                got = torch.autograd.grad(got_y, [ga, be, xl] + uniq, gy)
            finally:
                gb.keep_forward_stash(previous)
            assert torch.allclose(got_y, want_y, rtol=1e-4, atol=1e-5), (shared, keep)
            for i, (a, c) in enumerate(zip(got, want)):
                assert torch.allclose(a, c, rtol=1e-3, atol=1e-4 * (1 + c.abs().max().item())), \
                    (shared, keep, i, (a - c).abs().max().item())
    y0 = gb.FusedLoopResidualTrainOp.apply(gamma, beta, x, inner, block, "silu", 1e-5, 0, *plist[0])
    assert torch.equal(y0, x)


@pytest.mark.parametrize("name,grid,block,inner,outer,B", [("C3", 128, 8, 2, 16, 1), ("C4", 64, 4, 8, 16, 2)])
def test_training_configurations_at_their_own_grid_and_depth(name, grid, block, inner, outer, B):
    """The two forward + backward configurations of the benchmark at their own grid size, block size and
    iteration counts (128^3 / 8 / 2 x 16 and 64^3 / 4 / 8 x 16), one or two samples of the batch (samples only meet
    in the parameter gradients, which are sums over them): the fused training node's output and all six gradients
    against the float64 oracle's chain rule over the whole loop, the float32 oracle giving the noise floor."""
    import gridnet_b200 as gb
    from util import assert_close

    r = np.random.default_rng(73)
    f = np.float32
    shape = (grid, grid, grid)
    w = (r.standard_normal((27, *shape)) / np.sqrt(27)).astype(f)
    b = np.zeros(shape, f)
    s = np.ones(shape, f)
    ga = (1 + 0.05 * r.standard_normal(shape)).astype(f)
    be = (0.05 * r.standard_normal(shape)).astype(f)
    x = np.zeros((B, *shape), f)
    x[..., 0] = r.standard_normal((B, grid, grid))  # the input face, as in the benchmark
    gy = r.standard_normal((B, *shape)).astype(f)
    leaves = [torch.from_numpy(a).cuda().requires_grad_(True) for a in (w, b, s, ga, be, x)]
    assert gb.FusedLoopTrainOp.supported(leaves[0], leaves[5], inner, block)
    y = gb.FusedLoopTrainOp.apply(*leaves, inner, outer, block, "silu", 1e-5)
    grads = torch.autograd.grad(y, leaves, torch.from_numpy(gy).cuda())
    assert not gb.device_status(clear=True)
    a64 = [a.astype(np.float64) for a in (w, b, s, ga, be, x)]
    y64 = orc.outer_forward(*a64, inner, outer, block)
    y32 = orc.outer_forward(w, b, s, ga, be, x, inner, outer, block)
    assert_close(y.detach().cpu().numpy(), y64, y32, f"{name} forward")
    want64 = orc.outer_backward(*a64, gy.astype(np.float64), inner, outer, block)
    want32 = orc.outer_backward(w, b, s, ga, be, x, gy, inner, outer, block)
    # noise factor 3 instead of 2: the comparison is between the MAXIMA of two realisations of float32 rounding
    # noise over up to 5.7e7 elements after 32 chained stencil passes (gradients up to 4e3 in magnitude; measured:
    # the float32 oracle's worst error 1.3e-3, ours 3.0e-3, i.e. 7e-7 of max|ref|; 25 against 29 elements outside)
    for label, g, r64, r32 in zip(("weight", "bias", "scale", "gamma", "beta", "input"), grads, want64, want32):
        assert_close(g.cpu().numpy(), r64, r32, f"{name} gradient of {label}", noise_factor=3.0)
