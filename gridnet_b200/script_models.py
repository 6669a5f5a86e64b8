"""The two model classes the reference's training scripts define around the grid update, with the
same constructor keywords, attribute names and parameter names, so that their checkpoints
(``torch.save(model.state_dict())``, gridnet/scripts/train_imagenet.py:171-179) load with a plain
``load_state_dict``:

* :class:`MnistModel`     gridnet/scripts/train_mnist.py:16-65
* :class:`ImageNetModel`  gridnet/scripts/train_imagenet.py:18-87 (``outer_residual``, ``separate_params``)

The grid update and the whole-grid normalisation run through the CUDA library (the autograd ops when
gradients are needed, the fused loop otherwise); the patch embedding (a strided ``Conv2d`` written onto
the first K-planes) and the readout (last K-plane -> LayerNorm -> Linear) are the small dense layers
either side of the path and stay plain torch.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .backend_cuda import (FusedLoopResidualTrainOp, FusedLoopSeparateTrainOp, FusedLoopTrainOp, fused_loop_forward,
                           outer_forward)
from .modules import GatedGridnet, Gridnet, GridNorm, Readout


def _wants_grad(module: nn.Module, *tensors: torch.Tensor) -> bool:
    return torch.is_grad_enabled() and (any(t.requires_grad for t in tensors)
                                        or any(p.requires_grad for p in module.parameters()))


def _plain_loop(network: nn.Module, norm: GridNorm, h: torch.Tensor, outer_iters: int, owner: nn.Module) -> torch.Tensor:
    """``for _ in range(outer_iters): h = norm(network(h))``: one fused call when nothing needs a gradient, one
    autograd node over the whole loop when something does and the tuned kernels apply."""
    plain = isinstance(network, Gridnet) and not network.normalize and h.dtype == torch.float32
    if plain and not _wants_grad(owner, h):
        return outer_forward(network.weight, network.bias, network.residual_scale, norm.weight, norm.bias,
                             h.contiguous(), network.inner_iterations, outer_iters, network.block_size,
                             network.activation, norm.eps)
    if plain and FusedLoopTrainOp.supported(network.weight, h, network.inner_iterations, network.block_size):
        return FusedLoopTrainOp.apply(network.weight, network.bias, network.residual_scale, norm.weight, norm.bias, h,
                                      network.inner_iterations, outer_iters, network.block_size, network.activation,
                                      norm.eps)
    for _ in range(outer_iters):
        h = norm(network(h))
    return h


class MnistModel(nn.Module):
    """gridnet/scripts/train_mnist.py:16-65: a 32^3 grid, the 28x28 image written onto the first K-plane of a
    learned initial state, ``outer_iters`` x (network, LayerNorm), readout of the last K-plane."""

    def __init__(self, inner_iters: int, outer_iters: int, init_scale: float, residual_scale: float, gated: bool,
                 remember_bias: float, activation: str, device):
        super().__init__()
        self.outer_iters = outer_iters
        self.device = device
        self.init_in = nn.Parameter(torch.randn(32, 32, 32, device=device))
        if gated:
            self.network = GatedGridnet((32, 32, 32), inner_iters, 8, init_scale=init_scale, device=device,
                                        activation=activation)
            with torch.no_grad():
                self.network.bias[1].fill_(remember_bias)
        else:
            self.network = Gridnet((32, 32, 32), inner_iters, 8, init_scale=init_scale, residual_scale=residual_scale,
                                   device=device, normalize=False, activation=activation)
        self.norm = GridNorm((32, 32, 32), device=device)
        self.readout = Readout((32, 32, 32), out_channels=10, device=device)

    def forward(self, batch: torch.Tensor) -> torch.Tensor:
        batch = batch.reshape(-1, 28, 28)
        init_acts = self.init_in[None].repeat(batch.shape[0], 1, 1, 1)
        init_acts[:, 2:-2, 2:-2, 0] = batch
        return self.readout(_plain_loop(self.network, self.norm, init_acts, self.outer_iters, self))


class ImageNetModel(nn.Module):
    """gridnet/scripts/train_imagenet.py:18-87. ``grid_size`` must divide 256 (the image side); the patch
    embedding writes ``emb_channels`` K-planes; ``separate_params`` gives every outer iteration its own
    network (``networks.<i>.*`` in the state dict, ``network.*`` otherwise); ``outer_residual`` replaces
    ``h = norm(net(h))`` by ``n = norm(h); h = h + (net(n) - n)``."""

    def __init__(self, *, inner_iters: int, outer_iters: int, outer_residual: bool, init_scale: float,
                 residual_scale: float, emb_channels: int, grid_size: int, activation: str, separate_params: bool,
                 device):
        super().__init__()
        assert 256 % grid_size == 0
        self.outer_iters = outer_iters
        self.outer_residual = outer_residual
        self.emb_channels = emb_channels
        self.device = device
        self.init_in = nn.Parameter(torch.randn(grid_size, grid_size, grid_size, device=device))

        def make_model() -> Gridnet:
            return Gridnet((grid_size,) * 3, inner_iters, 8, init_scale=init_scale, residual_scale=residual_scale,
                           device=device, normalize=False, activation=activation)

        self.separate_params = separate_params
        if self.separate_params:
            self.networks = nn.ModuleList([make_model() for _ in range(outer_iters)])
        else:
            self.network = make_model()
        self.patch_emb = nn.Conv2d(3, emb_channels, kernel_size=256 // grid_size, stride=256 // grid_size,
                                   device=device)
        self.norm = GridNorm((grid_size,) * 3, device=device)
        self.readout = Readout((grid_size,) * 3, out_channels=1000, device=device)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        init_acts = self.init_in[None].repeat(images.shape[0], 1, 1, 1)
        init_acts[:, :, :, : self.emb_channels] = self.patch_emb(images).permute(0, 2, 3, 1)
        h = init_acts
        if not self.separate_params and not self.outer_residual:
            return self.readout(_plain_loop(self.network, self.norm, h, self.outer_iters, self))
        nets = list(self.networks) if self.separate_params else [self.network] * self.outer_iters
        first = nets[0] if nets else None
        if first is not None and h.dtype == torch.float32 and not first.normalize and \
                FusedLoopTrainOp.supported(first.weight, h, first.inner_iterations, first.block_size):
            # the loop variants run fused too: per-step parameters and the residual form, with and without gradients
            plist = [(n.weight, n.bias, n.residual_scale) for n in nets]
            if not _wants_grad(self, h):
                return self.readout(fused_loop_forward(plist, self.norm.weight, self.norm.bias, h, first.inner_iterations,
                                                       first.block_size, first.activation, self.norm.eps,
                                                       outer_residual=self.outer_residual))
            flat = [t for ps in (plist if self.separate_params else plist[:1]) for t in ps]
            if self.outer_residual:
                return self.readout(FusedLoopResidualTrainOp.apply(self.norm.weight, self.norm.bias, h,
                                                                   first.inner_iterations, first.block_size,
                                                                   first.activation, self.norm.eps, self.outer_iters,
                                                                   *flat))
            return self.readout(FusedLoopSeparateTrainOp.apply(self.norm.weight, self.norm.bias, h,
                                                               first.inner_iterations, first.block_size,
                                                               first.activation, self.norm.eps,
                                                               *[t for ps in plist for t in ps]))
        for i in range(self.outer_iters):
            net = self.networks[i] if self.separate_params else self.network
            if self.outer_residual:
                norm_h = self.norm(h)
                h = h + (net(norm_h) - norm_h)
            else:
                h = self.norm(net(h))
        return self.readout(h)
