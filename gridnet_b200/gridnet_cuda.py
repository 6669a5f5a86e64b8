"""Module-shaped stand-in for the reference's native extension ``gridnet_cuda``.

Same four functions, same positional arguments and the same contract as the
pybind11 module in src/gridnet_cuda.cpp:188-194: tensors must be CUDA and
contiguous (RuntimeError otherwise), outputs are caller-allocated, nothing is
returned. Work is queued on torch's current stream (the reference launches on
the legacy default stream, src/gridnet_cuda_kernels.cu:761).

The gradient outputs are overwritten; the reference accumulates into tensors its
caller zeroes first (gridnet/backend_cuda.py:78-81), which gives the same values.
"""
from __future__ import annotations

import torch

from ._lib import GN_ERR_UNSUPPORTED, GridnetB200Error, activation_id, check, lib


def _check_input(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise GridnetB200Error(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise GridnetB200Error(f"{name} must be contiguous")


def _suffix(t: torch.Tensor) -> str:
    if t.dtype == torch.float32:
        return "f32"
    if t.dtype == torch.float64:
        return "f64"
    raise GridnetB200Error(f"unsupported dtype {t.dtype}: float32 and float64 only")


def _same(ts, names):
    for t, n in zip(ts, names):
        _check_input(t, n)
        if t.dtype != ts[0].dtype or t.device != ts[0].device:
            raise GridnetB200Error(f"{n}: dtype/device differs from {names[0]}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def forward(weight, bias, scale, initActivations, outActivations, innerIterations, blockSize, eps,
            normalize, activation) -> None:
    _same((weight, bias, scale, initActivations, outActivations),
          ("weight", "bias", "scale", "initActivations", "outActivations"))
    B, M, N, K = initActivations.shape
    fn = getattr(lib, "gn_step_forward_" + _suffix(weight))
    with torch.cuda.device(weight.device):
        check(fn(weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), initActivations.data_ptr(),
                 outActivations.data_ptr(), B, M, N, K, int(innerIterations), int(blockSize), float(eps),
                 int(bool(normalize)), activation_id(activation), _stream(weight)))


def backward(weight, bias, scale, initActivations, outGrads, weightGradOut, biasGradOut, scaleGradOut,
             activationsGradOut, innerIterations, blockSize, eps, normalize, activation) -> None:
    _same((weight, bias, scale, initActivations, outGrads, weightGradOut, biasGradOut, scaleGradOut,
           activationsGradOut),
          ("weight", "bias", "scale", "initActivations", "outGrads", "weightGradOut", "biasGradOut",
           "scaleGradOut", "activationsGradOut"))
    B, M, N, K = initActivations.shape
    sfx = _suffix(weight)
    with torch.cuda.device(weight.device):
        need = 0
        if sfx == "f32" and B > 0:
            need = int(lib.gn_step_backward_workspace_bytes(B, M, N, K, int(innerIterations), int(blockSize),
                                                            int(bool(normalize)), 4))
        if need:
            # scratch for the tuned four-kernel path (torch's caching allocator, stream ordered)
            ws = torch.empty(need, dtype=torch.uint8, device=weight.device)
            check(lib.gn_step_backward_ws_f32(
                weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), initActivations.data_ptr(), outGrads.data_ptr(),
                weightGradOut.data_ptr(), biasGradOut.data_ptr(), scaleGradOut.data_ptr(),
                activationsGradOut.data_ptr(), B, M, N, K, int(innerIterations), int(blockSize), float(eps),
                int(bool(normalize)), activation_id(activation), ws.data_ptr(), ws.numel(), _stream(weight)))
            return
        fn = getattr(lib, "gn_step_backward_" + sfx)
        check(fn(weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), initActivations.data_ptr(),
                 outGrads.data_ptr(), weightGradOut.data_ptr(), biasGradOut.data_ptr(),
                 scaleGradOut.data_ptr(), activationsGradOut.data_ptr(), B, M, N, K, int(innerIterations),
                 int(blockSize), float(eps), int(bool(normalize)), activation_id(activation),
                 _stream(weight)))


def forward_with_stash(weight, bias, scale, initActivations, outActivations, innerIterations, blockSize, activation):
    """:func:`forward` (normalize off, float32) that also keeps what the backward pass would otherwise
    recompute. Returns the stash tensor, or ``None`` (after running the ordinary forward) where the
    tuned path does not apply. Not part of the reference's module: it always recomputes."""
    _same((weight, bias, scale, initActivations, outActivations),
          ("weight", "bias", "scale", "initActivations", "outActivations"))
    B, M, N, K = initActivations.shape
    need = 0
    if weight.dtype == torch.float32 and B > 0:
        need = int(lib.gn_step_stash_bytes(B, M, N, K, int(innerIterations), int(blockSize)))
    with torch.cuda.device(weight.device):
        if need:
            stash = torch.empty(need, dtype=torch.uint8, device=weight.device)
            rc = lib.gn_step_forward_stash_f32(
                weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), initActivations.data_ptr(),
                outActivations.data_ptr(), B, M, N, K, int(innerIterations), int(blockSize), activation_id(activation),
                stash.data_ptr(), stash.numel(), _stream(weight))
            if rc == 0:
                return stash
            if rc != GN_ERR_UNSUPPORTED:  # anything but "the tuned path does not apply here"
                check(rc)
    forward(weight, bias, scale, initActivations, outActivations, innerIterations, blockSize, 1e-5, False, activation)
    return None


def backward_with_stash(weight, bias, scale, initActivations, outGrads, weightGradOut, biasGradOut, scaleGradOut,
                        activationsGradOut, innerIterations, blockSize, activation, stash) -> None:
    """:func:`backward` for a step whose forward pass went through :func:`forward_with_stash`."""
    _same((weight, bias, scale, initActivations, outGrads, weightGradOut, biasGradOut, scaleGradOut,
           activationsGradOut),
          ("weight", "bias", "scale", "initActivations", "outGrads", "weightGradOut", "biasGradOut",
           "scaleGradOut", "activationsGradOut"))
    B, M, N, K = initActivations.shape
    with torch.cuda.device(weight.device):
        need = int(lib.gn_step_backward_stash_workspace_bytes(B, M, N, K, int(innerIterations), int(blockSize)))
        ws = torch.empty(need, dtype=torch.uint8, device=weight.device)
        check(lib.gn_step_backward_stash_f32(
            weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), initActivations.data_ptr(), outGrads.data_ptr(),
            weightGradOut.data_ptr(), biasGradOut.data_ptr(), scaleGradOut.data_ptr(), activationsGradOut.data_ptr(),
            B, M, N, K, int(innerIterations), int(blockSize), activation_id(activation), stash.data_ptr(), stash.numel(),
            ws.data_ptr(), ws.numel(), _stream(weight)))


def forward_gated(weight, bias, initActivations, outActivations, innerIterations, blockSize,
                  activation) -> None:
    _same((weight, bias, initActivations, outActivations),
          ("weight", "bias", "initActivations", "outActivations"))
    B, M, N, K = initActivations.shape
    fn = getattr(lib, "gn_gated_forward_" + _suffix(weight))
    with torch.cuda.device(weight.device):
        check(fn(weight.data_ptr(), bias.data_ptr(), initActivations.data_ptr(), outActivations.data_ptr(),
                 B, M, N, K, int(innerIterations), int(blockSize), activation_id(activation),
                 _stream(weight)))


def backward_gated(weight, bias, initActivations, outGrads, weightGradOut, biasGradOut, activationsGradOut,
                   innerIterations, blockSize, activation) -> None:
    _same((weight, bias, initActivations, outGrads, weightGradOut, biasGradOut, activationsGradOut),
          ("weight", "bias", "initActivations", "outGrads", "weightGradOut", "biasGradOut",
           "activationsGradOut"))
    B, M, N, K = initActivations.shape
    fn = getattr(lib, "gn_gated_backward_" + _suffix(weight))
    with torch.cuda.device(weight.device):
        need = 0
        if _suffix(weight) == "f32" and B > 0:
            need = int(lib.gn_gated_backward_workspace_bytes(B, M, N, K, int(innerIterations), int(blockSize), 4))
        if need:
            # scratch for the tuned four-kernel path (torch's caching allocator, stream ordered)
            ws = torch.empty(need, dtype=torch.uint8, device=weight.device)
            check(lib.gn_gated_backward_ws_f32(
                weight.data_ptr(), bias.data_ptr(), initActivations.data_ptr(), outGrads.data_ptr(),
                weightGradOut.data_ptr(), biasGradOut.data_ptr(), activationsGradOut.data_ptr(), B, M, N, K,
                int(innerIterations), int(blockSize), activation_id(activation), ws.data_ptr(), ws.numel(),
                _stream(weight)))
            return
        check(fn(weight.data_ptr(), bias.data_ptr(), initActivations.data_ptr(), outGrads.data_ptr(),
                 weightGradOut.data_ptr(), biasGradOut.data_ptr(), activationsGradOut.data_ptr(), B, M, N, K,
                 int(innerIterations), int(blockSize), activation_id(activation), _stream(weight)))
