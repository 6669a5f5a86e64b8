"""CPU-side checks of the boundary: the shared library loads, exports every symbol
the header declares, and the op surface validates its arguments like the reference
(gridnet/backend_cuda.py:19-52) before anything touches a GPU."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "gridnet_b200.h")).read()
    return sorted(set(re.findall(r"GN_API[^;(]*?\b(gn_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from gridnet_b200 import _lib

    names = _header_symbols()
    assert len(names) >= 18
    dll = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(dll, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signature table and header disagree"


def test_status_strings_and_activation_names():
    from gridnet_b200._lib import lib

    assert lib.gn_status_string(0) == b"ok"
    for code in range(-9, 0):
        assert lib.gn_status_string(code) not in (b"ok", b"unknown status")
    assert [lib.gn_activation_from_name(n) for n in (b"relu", b"leaky_relu", b"silu", b"tanh")] == [0, 1, 2, 3]
    assert lib.gn_activation_from_name(b"gelu") == -1
    assert lib.gn_version() >= 1
    assert lib.gn_step_backward_max_inner(8, 4) >= 32
    assert lib.gn_step_backward_max_inner(8, 8) >= 32
    assert lib.gn_step_backward_max_inner(3, 4) == -1


def test_argument_errors_need_no_gpu():
    # validation order of the C ABI: geometry first, so these return before any CUDA call
    from gridnet_b200._lib import lib

    f = lib.gn_step_forward_f32
    assert f(None, None, None, None, None, 1, 8, 8, 8, 1, 3, 1e-5, 0, 2, None) == -2  # block 3
    assert f(None, None, None, None, None, 1, 8, 8, 12, 1, 8, 1e-5, 0, 2, None) == -2  # 12 % 8
    assert f(None, None, None, None, None, 1, 8, 8, 8, 1, 8, 1e-5, 0, 7, None) == -4  # activation
    assert f(None, None, None, None, None, 1, 8, 8, 8, -1, 8, 1e-5, 0, 2, None) == -5  # inner
    assert f(None, None, None, None, None, 1, 8, 8, 8, 1, 8, 1e-5, 0, 2, None) == -1  # NULL pointers
    assert f(None, None, None, None, None, 0, 8, 8, 8, 1, 8, 1e-5, 0, 2, None) == 0  # empty batch
    assert lib.gn_outer_forward_workspace_bytes(64, 64, 64, 64, 8) >= 2 * 64 * 64**3 * 4


def test_op_surface_assertions_match_reference():
    from gridnet_b200 import GatedGridnetCudaOp, GridnetCudaOp

    shape = (8, 8, 8)
    w, b, s = torch.zeros(27, *shape), torch.zeros(shape), torch.zeros(shape)
    x = torch.zeros(2, *shape)
    with pytest.raises(AssertionError):  # block size does not divide the grid
        GridnetCudaOp.apply(w, b, s, x, 1, 3, 1e-5, False, "silu")
    with pytest.raises(AssertionError):  # weight shape
        GridnetCudaOp.apply(w[:26], b, s, x, 1, 8, 1e-5, False, "silu")
    with pytest.raises(AssertionError):  # dtype mismatch
        GridnetCudaOp.apply(w, b.double(), s, x, 1, 8, 1e-5, False, "silu")
    with pytest.raises(AssertionError):
        GatedGridnetCudaOp.apply(w, torch.zeros(2, *shape), x, 1, 8, "tanh")
    # empty batch: a clone, no kernel (gridnet/backend_cuda.py:51-52)
    e = torch.zeros(0, *shape)
    out = GridnetCudaOp.apply(w, b, s, e, 1, 8, 1e-5, False, "silu")
    assert out.shape == e.shape and out.data_ptr() != e.data_ptr() or out.numel() == 0
    # CPU tensors are rejected by the extension layer, as CHECK_CUDA does (src/gridnet_cuda.cpp:6)
    with pytest.raises(RuntimeError):
        GridnetCudaOp.apply(w, b, s, x, 1, 8, 1e-5, False, "silu")
    with pytest.raises(RuntimeError):
        GatedGridnetCudaOp.apply(torch.zeros(27, 2, *shape), torch.zeros(2, *shape), x, 1, 8, "tanh")


def test_no_fallback_when_library_is_missing(tmp_path, monkeypatch):
    # the loader must fail loudly instead of degrading to another implementation
    import importlib

    from gridnet_b200 import _lib

    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(ImportError):
        _lib._load()
    importlib.reload(_lib)
