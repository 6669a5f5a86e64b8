"""Module-level wrappers with the reference's constructor arguments and parameter names
(gridnet/__init__.py:21-121), so reference ``state_dict``s load unchanged, plus the model loop
the reference's scripts write by hand (gridnet/scripts/train_mnist.py:57-65).

Everything computes through the CUDA library; parameters on another device raise, because
this package has no CPU or PyTorch implementation of the update.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch
import torch.nn as nn

from .backend_cuda import FusedLoopTrainOp, GatedGridnetCudaOp, GridnetCudaOp, GridNormOp, outer_forward


def _need_cuda(t: torch.Tensor, what: str) -> None:
    if t.device.type != "cuda":
        raise RuntimeError(f"{what} is on {t.device}; gridnet_b200 only runs on CUDA devices (no fallback)")


def gridnet_step(weight, bias, residual_scale, init_activations, inner_iterations: int, block_size: int,
                 eps: float = 1e-5, normalize: bool = True, activation: str = "silu") -> torch.Tensor:
    """Same arguments as the reference's ``gridnet_step`` (gridnet/__init__.py:124-194)."""
    _need_cuda(weight, "weight")
    return GridnetCudaOp.apply(weight, bias, residual_scale, init_activations, inner_iterations, block_size, eps,
                               normalize, activation)


def gated_gridnet_step(weight, bias, init_activations, inner_iterations: int, block_size: int,
                       activation: str = "tanh") -> torch.Tensor:
    """Same arguments as the reference's ``gated_gridnet_step`` (gridnet/__init__.py:197-255)."""
    _need_cuda(weight, "weight")
    return GatedGridnetCudaOp.apply(weight, bias, init_activations, inner_iterations, block_size, activation)


class Gridnet(nn.Module):
    """gridnet/__init__.py:21-64."""

    def __init__(self, shape: Tuple[int, int, int], inner_iterations: int, block_size: int, device,
                 dtype: torch.dtype = torch.float32, eps: float = 1e-5, init_scale: float = 1.0,
                 residual_scale: float = 1.0, normalize: bool = True, activation: str = "silu"):
        super().__init__()
        self.shape, self.inner_iterations, self.block_size = tuple(shape), inner_iterations, block_size
        self.eps, self.normalize, self.activation = eps, normalize, activation
        self.weight = nn.Parameter(torch.randn(27, *shape, device=device, dtype=dtype) * (init_scale / math.sqrt(27)))
        self.bias = nn.Parameter(torch.zeros(*shape, device=device, dtype=dtype))
        self.residual_scale = nn.Parameter(torch.ones(*shape, device=device, dtype=dtype) * residual_scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return gridnet_step(self.weight, self.bias, self.residual_scale, x, self.inner_iterations, self.block_size,
                            self.eps, self.normalize, self.activation)


class GatedGridnet(nn.Module):
    """gridnet/__init__.py:67-99."""

    def __init__(self, shape: Tuple[int, int, int], inner_iterations: int, block_size: int, device,
                 dtype: torch.dtype = torch.float32, init_scale: float = 1.0, activation: str = "tanh"):
        super().__init__()
        self.shape, self.inner_iterations, self.block_size, self.activation = tuple(shape), inner_iterations, block_size, activation
        self.weight = nn.Parameter(torch.randn(27, 2, *shape, device=device, dtype=dtype) * (init_scale / math.sqrt(27)))
        self.bias = nn.Parameter(torch.zeros(2, *shape, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return gated_gridnet_step(self.weight, self.bias, x, self.inner_iterations, self.block_size, self.activation)


class GridNorm(nn.Module):
    """``nn.LayerNorm(shape)`` over the whole grid with the same parameter names (weight, bias)."""

    def __init__(self, shape: Tuple[int, int, int], device, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(*shape, device=device))
        self.bias = nn.Parameter(torch.zeros(*shape, device=device))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return GridNormOp.apply(x, self.weight, self.bias, self.eps)


class Readout(nn.Module):
    """gridnet/__init__.py:102-121: the last ``output_layers`` K-planes -> LayerNorm -> Linear (plain torch:
    the only dense layer around the path, and tiny)."""

    def __init__(self, grid_shape: Tuple[int, int, int], out_channels: int, device, dtype: torch.dtype = torch.float32,
                 output_layers: int = 1):
        super().__init__()
        size = grid_shape[0] * grid_shape[1] * output_layers
        self.output_layers = output_layers
        self.norm = nn.LayerNorm(size, device=device, dtype=dtype)
        self.proj = nn.Linear(size, out_channels, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(self.norm(x[:, :, :, -self.output_layers:].flatten(1)))


class GridnetModel(nn.Module):
    """The loop of the reference's scripts: ``for _ in range(outer_iters): h = network(h); h = norm(h)``
    (gridnet/scripts/train_mnist.py:62-64), with submodules named ``network`` and ``norm`` as there.

    A plain float32 network with per-block normalisation off runs fused: with gradients disabled as ONE call
    (:func:`outer_forward`), with gradients as one autograd node over the whole loop (:class:`FusedLoopTrainOp`:
    statistics out of the step kernels, normalisation on load, only raw step outputs saved). Everything else is
    the step-by-step composition of the two autograd ops."""

    def __init__(self, shape: Tuple[int, int, int], inner_iters: int, outer_iters: int, block_size: int, device,
                 init_scale: float = 1.0, residual_scale: float = 1.0, activation: str = "silu", gated: bool = False,
                 normalize: bool = False):
        super().__init__()
        self.outer_iters = outer_iters
        if gated:
            self.network = GatedGridnet(shape, inner_iters, block_size, device, init_scale=init_scale,
                                        activation=activation)
        else:
            self.network = Gridnet(shape, inner_iters, block_size, device, init_scale=init_scale,
                                   residual_scale=residual_scale, normalize=normalize, activation=activation)
        self.norm = GridNorm(shape, device)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        net = self.network
        plain = isinstance(net, Gridnet) and not net.normalize and h.dtype == torch.float32
        with_grad = torch.is_grad_enabled() and (h.requires_grad or any(p.requires_grad for p in self.parameters()))
        if plain and not with_grad:
            return outer_forward(net.weight, net.bias, net.residual_scale, self.norm.weight, self.norm.bias,
                                 h.contiguous(), net.inner_iterations, self.outer_iters, net.block_size, net.activation,
                                 self.norm.eps)
        if plain and FusedLoopTrainOp.supported(net.weight, h, net.inner_iterations, net.block_size):
            return FusedLoopTrainOp.apply(net.weight, net.bias, net.residual_scale, self.norm.weight, self.norm.bias, h,
                                          net.inner_iterations, self.outer_iters, net.block_size, net.activation,
                                          self.norm.eps)
        for _ in range(self.outer_iters):
            h = self.norm(net(h))
        return h
