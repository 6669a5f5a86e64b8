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
