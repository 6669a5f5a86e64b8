"""The drop-in boundary seen from the reference's side: its own ``gridnet`` package, imported unchanged from the
reference tree with ``gridnet_cuda`` replaced by this package's module of the same shape, picks up its CUDA ops
(gridnet/__init__.py:14-18) and reaches this library's argument validation through them. Skipped where the
reference tree is not present."""
import importlib
import os
import sys

import pytest
import torch

REFERENCE = os.environ.get("GRIDNET_REFERENCE", "/root/reference")


@pytest.fixture()
def reference_gridnet():
    if not os.path.isdir(os.path.join(REFERENCE, "gridnet")):
        pytest.skip("reference tree not present")
    import gridnet_b200

    saved = {k: sys.modules.get(k) for k in list(sys.modules) if k == "gridnet" or k.startswith("gridnet.")}
    saved["gridnet_cuda"] = sys.modules.get("gridnet_cuda")
    for k in list(saved):
        sys.modules.pop(k, None)
    sys.modules["gridnet_cuda"] = gridnet_b200.gridnet_cuda
    sys.path.insert(0, REFERENCE)
    sys.dont_write_bytecode, old_flag = True, sys.dont_write_bytecode  # the reference tree is read-only
    try:
        yield importlib.import_module("gridnet")
    finally:
        sys.dont_write_bytecode = old_flag
        sys.path.remove(REFERENCE)
        for k in [k for k in sys.modules if k == "gridnet" or k.startswith("gridnet.") or k == "gridnet_cuda"]:
            sys.modules.pop(k, None)
        for k, v in saved.items():
            if v is not None:
                sys.modules[k] = v


def test_reference_package_picks_up_the_replacement_extension(reference_gridnet):
    gridnet = reference_gridnet
    import gridnet_b200

    assert gridnet.GridnetCudaOp is not None and gridnet.GatedGridnetCudaOp is not None
    assert sys.modules["gridnet.backend_cuda"].gridnet_cuda is gridnet_b200.gridnet_cuda
    # the reference's op runs its own assertions, then calls forward() of the replacement module: with CPU
    # tensors that call must end in this library's check (src/gridnet_cuda.cpp:6-10 raises the same way)
    shape = (8, 8, 8)
    w, b, s = torch.randn(27, *shape), torch.randn(shape), torch.randn(shape)
    x = torch.randn(2, *shape)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        gridnet.GridnetCudaOp.apply(w, b, s, x, 2, 8, 1e-5, False, "silu")
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        gridnet.GatedGridnetCudaOp.apply(torch.randn(27, 2, *shape), torch.randn(2, *shape), x, 2, 8, "tanh")
    # the reference's own assertions still come first
    with pytest.raises(AssertionError):
        gridnet.GridnetCudaOp.apply(w, b, s, torch.randn(2, 8, 8, 12), 2, 8, 1e-5, False, "silu")


@pytest.mark.gpu
def test_reference_modules_run_on_the_replacement_extension(reference_gridnet):
    """On a GPU box that also has the reference tree: the reference's Gridnet module, unmodified, computes through
    this library and agrees with its own PyTorch path."""
    gridnet = reference_gridnet
    dev = torch.device("cuda")
    torch.manual_seed(0)
    net = gridnet.Gridnet((16, 16, 16), 2, 8, dev, normalize=False, activation="silu")
    x = torch.randn(3, 16, 16, 16, device=dev)
    got = net(x)
    want = sys.modules["gridnet.backend_torch"].gridnet_step_pytorch(
        net.weight, net.bias, net.residual_scale, x, 2, 8, net.eps, False, "silu")
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
