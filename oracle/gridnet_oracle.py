"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE, not product code).

Only the test suite, the smoke test and the benchmark's CPU-baseline / reference
arm may import this module. It wraps ``oracle/libgridnet_oracle.so`` (built by
``oracle/Makefile`` from ``gridnet_oracle.c``), a plain-C restatement of

* ``gridnet/backend_torch.py:9-142``  (``gridnet_step_pytorch``),
* ``gridnet/backend_torch.py:145-267`` (``gated_gridnet_step_pytorch``),
* the gradients torch.autograd derives from them, and
* ``torch.nn.LayerNorm`` over the whole grid, which the reference's models apply
  after every outer step (``gridnet/scripts/train_mnist.py:54,62-64``).

Parity status: PINNED. ``tests/test_oracle_golden.py`` checks every function here
against vectors produced by the reference's own Python code
(``tests/golden/make_golden.py`` imports it and writes ``tests/golden/*.npz``)
and against the reference's two known-answer tests
(``gridnet/backend_torch_test.py:10-60``).

All arrays are C-contiguous numpy arrays of float32 or float64.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgridnet_oracle.so")

ACTIVATIONS = {"relu": 0, "leaky_relu": 1, "silu": 2, "tanh": 3}

_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with gcc if the shared object is missing or stale."""
    src = [os.path.join(_HERE, f) for f in ("gridnet_oracle.c", "gridnet_oracle_impl.inc", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH)
    if not stale:
        t = os.path.getmtime(_LIB_PATH)
        stale = any(os.path.getmtime(s) > t for s in src)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libgridnet_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.gno_max_threads.restype = ctypes.c_int
    return _lib


def max_threads() -> int:
    return int(lib().gno_max_threads())


def set_threads(n: int) -> None:
    lib().gno_set_threads(ctypes.c_int(int(n)))


def _sfx(dtype) -> str:
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle supports float32/float64, got {dtype}")


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"], "oracle needs C-contiguous arrays"
    return a.ctypes.data_as(ctypes.c_void_p)


def _same(dtype, *arrs):
    return [np.ascontiguousarray(a, dtype=dtype) for a in arrs]


def _check(x, block_size):
    B, M, N, K = x.shape
    if M % block_size or N % block_size or K % block_size:
        raise AssertionError(f"block_size={block_size} incompatible with {x.shape}")
    return B, M, N, K


def step_forward(weight, bias, scale, x, inner, block_size, eps=1e-5, normalize=True, activation="silu"):
    dt = np.asarray(x).dtype
    weight, bias, scale, x = _same(dt, weight, bias, scale, x)
    B, M, N, K = _check(x, block_size)
    assert weight.shape == (27, M, N, K) and bias.shape == (M, N, K) and scale.shape == (M, N, K)
    y = np.empty_like(x)
    if B:
        getattr(lib(), "gno_step_forward_" + _sfx(dt))(
            _p(weight), _p(bias), _p(scale), _p(x), _p(y), B, M, N, K, int(inner), int(block_size),
            ctypes.c_double(eps), int(bool(normalize)), ACTIVATIONS[activation])
    return y


def step_backward(weight, bias, scale, x, gy, inner, block_size, eps=1e-5, normalize=True, activation="silu"):
    """Returns (grad_weight, grad_bias, grad_scale, grad_x)."""
    dt = np.asarray(x).dtype
    weight, bias, scale, x, gy = _same(dt, weight, bias, scale, x, gy)
    B, M, N, K = _check(x, block_size)
    gw, gb, gs, gx = np.empty_like(weight), np.empty_like(bias), np.empty_like(scale), np.empty_like(x)
    getattr(lib(), "gno_step_backward_" + _sfx(dt))(
        _p(weight), _p(bias), _p(scale), _p(x), _p(gy), _p(gw), _p(gb), _p(gs), _p(gx), B, M, N, K,
        int(inner), int(block_size), ctypes.c_double(eps), int(bool(normalize)), ACTIVATIONS[activation])
    return gw, gb, gs, gx


def gated_forward(weight, bias, x, inner, block_size, activation="tanh"):
    dt = np.asarray(x).dtype
    weight, bias, x = _same(dt, weight, bias, x)
    B, M, N, K = _check(x, block_size)
    assert weight.shape == (27, 2, M, N, K) and bias.shape == (2, M, N, K)
    y = np.empty_like(x)
    if B:
        getattr(lib(), "gno_gated_forward_" + _sfx(dt))(
            _p(weight), _p(bias), _p(x), _p(y), B, M, N, K, int(inner), int(block_size),
            ACTIVATIONS[activation])
    return y


def gated_backward(weight, bias, x, gy, inner, block_size, activation="tanh"):
    """Returns (grad_weight, grad_bias, grad_x)."""
    dt = np.asarray(x).dtype
    weight, bias, x, gy = _same(dt, weight, bias, x, gy)
    B, M, N, K = _check(x, block_size)
    gw, gb, gx = np.empty_like(weight), np.empty_like(bias), np.empty_like(x)
    getattr(lib(), "gno_gated_backward_" + _sfx(dt))(
        _p(weight), _p(bias), _p(x), _p(gy), _p(gw), _p(gb), _p(gx), B, M, N, K, int(inner),
        int(block_size), ACTIVATIONS[activation])
    return gw, gb, gx


def layernorm_forward(x, gamma, beta, eps=1e-5):
    dt = np.asarray(x).dtype
    x, gamma, beta = _same(dt, x, gamma, beta)
    B = x.shape[0]
    P = int(np.prod(x.shape[1:]))
    y = np.empty_like(x)
    if B:
        getattr(lib(), "gno_layernorm_forward_" + _sfx(dt))(
            _p(x), _p(gamma), _p(beta), _p(y), B, ctypes.c_long(P), ctypes.c_double(eps))
    return y


def layernorm_backward(x, gamma, gy, eps=1e-5):
    """Returns (grad_x, grad_gamma, grad_beta)."""
    dt = np.asarray(x).dtype
    x, gamma, gy = _same(dt, x, gamma, gy)
    B = x.shape[0]
    P = int(np.prod(x.shape[1:]))
    gx, gg, gb = np.empty_like(x), np.empty_like(gamma), np.empty_like(gamma)
    getattr(lib(), "gno_layernorm_backward_" + _sfx(dt))(
        _p(x), _p(gamma), _p(gy), _p(gx), _p(gg), _p(gb), B, ctypes.c_long(P), ctypes.c_double(eps))
    return gx, gg, gb


def outer_forward(weight, bias, scale, gamma, beta, x, inner, outer, block_size, eps=1e-5,
                  normalize=False, activation="silu", ln_eps=1e-5):
    """``outer`` repetitions of (step, whole-grid LayerNorm): the model loop of
    gridnet/scripts/train_mnist.py:62-64."""
    h = np.asarray(x)
    for _ in range(outer):
        h = step_forward(weight, bias, scale, h, inner, block_size, eps, normalize, activation)
        h = layernorm_forward(h, gamma, beta, ln_eps)
    return h


def outer_backward(weight, bias, scale, gamma, beta, x, gy, inner, outer, block_size, eps=1e-5, normalize=False,
                   activation="silu", ln_eps=1e-5):
    """Gradient of :func:`outer_forward` for an upstream gradient ``gy`` on its result: the composition
    ``step_backward o layernorm_backward`` walked from the last outer step to the first, parameter gradients
    summed over the steps (shared parameters). Returns (grad_weight, grad_bias, grad_scale, grad_gamma,
    grad_beta, grad_x)."""
    h = np.asarray(x)
    step_in, norm_in = [], []
    for _ in range(outer):
        step_in.append(h)
        s = step_forward(weight, bias, scale, h, inner, block_size, eps, normalize, activation)
        norm_in.append(s)
        h = layernorm_forward(s, gamma, beta, ln_eps)
    g = np.asarray(gy, dtype=h.dtype)
    gw = gb = gs = gg = gbt = None
    for k in reversed(range(outer)):
        g, dg, dbt = layernorm_backward(norm_in[k], gamma, g, ln_eps)
        dw, db, ds, g = step_backward(weight, bias, scale, step_in[k], g, inner, block_size, eps, normalize, activation)
        if gw is None:
            gw, gb, gs, gg, gbt = dw, db, ds, dg, dbt
        else:
            gw, gb, gs, gg, gbt = gw + dw, gb + db, gs + ds, gg + dg, gbt + dbt
    return gw, gb, gs, gg, gbt, g
