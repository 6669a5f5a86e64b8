"""Pins the CPU oracle: every oracle function against vectors produced by the
reference's own Python code (tests/golden/make_golden.py), plus the reference's
two known-answer tests (gridnet/backend_torch_test.py:10-60)."""
import os

import numpy as np
import pytest

from oracle import gridnet_oracle as orc

from conftest import GOLDEN


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


def _cases(npz):
    return sorted({k.split("_")[0] for k in npz.files if k.endswith("_meta")})


def _relerr(a, b):
    return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-300))


def test_step_forward_matches_reference_vectors():
    z = _load("step_forward.npz")
    for c in _cases(z):
        bs, inner, norm = (int(v) for v in z[f"{c}_meta"])
        act = str(z[f"{c}_act"])
        args = [z[f"{c}_{k}"] for k in ("w", "b", "s", "x")]
        y64 = orc.step_forward(*[a.astype(np.float64) for a in args], inner, bs, 1e-5, bool(norm), act)
        assert _relerr(y64, z[f"{c}_y64"]) < 1e-12, c
        y32 = orc.step_forward(*args, inner, bs, 1e-5, bool(norm), act)
        assert y32.dtype == np.float32
        # float32 against the reference's float32 run: the same rounding noise on both sides
        np.testing.assert_allclose(y32, z[f"{c}_y32"], rtol=1e-4, atol=2e-5, err_msg=c)
        np.testing.assert_allclose(y32, z[f"{c}_y64"], rtol=1e-4, atol=2e-5, err_msg=c)


def test_step_backward_matches_reference_autograd():
    z = _load("step_backward.npz")
    for c in _cases(z):
        bs, inner, norm = (int(v) for v in z[f"{c}_meta"])
        act = str(z[f"{c}_act"])
        w, b, s, x, gy = (z[f"{c}_{k}"].astype(np.float64) for k in ("w", "b", "s", "x", "gy"))
        got = orc.step_backward(w, b, s, x, gy, inner, bs, 1e-5, bool(norm), act)
        for name, g in zip(("gw", "gb", "gs", "gx"), got):
            assert _relerr(g, z[f"{c}_{name}"]) < 1e-11, (c, name)


def test_gated_matches_reference_vectors():
    z = _load("gated.npz")
    for c in _cases(z):
        bs, inner = (int(v) for v in z[f"{c}_meta"])
        act = str(z[f"{c}_act"])
        w, b, x, gy = (z[f"{c}_{k}"] for k in ("w", "b", "x", "gy"))
        y32 = orc.gated_forward(w, b, x, inner, bs, act)
        np.testing.assert_allclose(y32, z[f"{c}_y32"], rtol=1e-4, atol=1e-5, err_msg=c)
        w, b, x, gy = (a.astype(np.float64) for a in (w, b, x, gy))
        assert _relerr(orc.gated_forward(w, b, x, inner, bs, act), z[f"{c}_y64"]) < 1e-12, c
        got = orc.gated_backward(w, b, x, gy, inner, bs, act)
        for name, g in zip(("gw", "gb", "gx"), got):
            assert _relerr(g, z[f"{c}_{name}"]) < 1e-11, (c, name)


def test_outer_loop_and_layernorm_match_reference_vectors():
    z = _load("outer_loop.npz")
    bs, inner, outer = (int(v) for v in z["meta"])
    a = [z[k] for k in ("w", "b", "s", "gamma", "beta", "x")]
    y64 = orc.outer_forward(*[v.astype(np.float64) for v in a], inner, outer, bs)
    assert _relerr(y64, z["y64"]) < 1e-11
    y32 = orc.outer_forward(*a, inner, outer, bs)
    np.testing.assert_allclose(y32, z["y32"], rtol=1e-4, atol=1e-5)
    gam, bet = z["gamma"].astype(np.float64), z["beta"].astype(np.float64)
    lx, lgy = z["ln_x"].astype(np.float64), z["ln_gy"].astype(np.float64)
    assert _relerr(orc.layernorm_forward(lx, gam, bet), z["ln_y"]) < 1e-12
    gx, gg, gb = orc.layernorm_backward(lx, gam, lgy)
    assert _relerr(gx, z["ln_gx"]) < 1e-11
    assert _relerr(gg, z["ln_gg"]) < 1e-11
    assert _relerr(gb, z["ln_gb"]) < 1e-12


@pytest.mark.parametrize("shape,bs", [((16, 16, 16), 8), ((32, 64, 128), 8)])
def test_zero_iterations_is_identity(shape, bs):
    # gridnet/backend_torch_test.py:10-25
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, *shape), dtype=np.float32)
    w = rng.standard_normal((27, *shape), dtype=np.float32)
    b = rng.standard_normal(shape, dtype=np.float32)
    y = orc.step_forward(w, b, np.ones(shape, np.float32), x, 0, bs)
    assert np.array_equal(y, x)


@pytest.mark.parametrize("shape,bs", [((16, 16, 16), 8), ((32, 64, 128), 8)])
def test_zero_weights_closed_form(shape, bs):
    # gridnet/backend_torch_test.py:28-60: with zero weights and bias every
    # iteration adds silu(0) * 0.31 = 0 to every voxel
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, *shape), dtype=np.float32)
    w = np.zeros((27, *shape), np.float32)
    b = np.zeros(shape, np.float32)
    s = np.full(shape, 0.31, np.float32)
    y = orc.step_forward(w, b, s, x, 10, bs)
    np.testing.assert_allclose(y, x, rtol=0, atol=0)
    # non-zero bias: each voxel moves by 10 * silu(bias) * 0.31
    b = rng.standard_normal(shape, dtype=np.float32)
    y = orc.step_forward(w, b, s, x, 10, bs, normalize=True)
    want = x + 10 * (b / (1 + np.exp(-b.astype(np.float64)))) * 0.31
    np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-5)


def test_empty_batch_and_bad_block():
    shape = (8, 8, 8)
    w = np.zeros((27, *shape), np.float32)
    b = np.zeros(shape, np.float32)
    y = orc.step_forward(w, b, b, np.zeros((0, *shape), np.float32), 2, 8)
    assert y.shape == (0, *shape)
    with pytest.raises(AssertionError):
        orc.step_forward(w, b, b, np.zeros((1, *shape), np.float32), 2, 3)


def test_outer_backward_matches_finite_differences():
    """The oracle's chain rule over the model loop (step_backward o layernorm_backward, shared parameters summed)
    against central differences of outer_forward, float64, one random entry of every argument."""
    r = np.random.default_rng(0)
    shape, B = (8, 8, 8), 2
    w = r.standard_normal((27, *shape)) / np.sqrt(27)
    b, s = 0.1 * r.standard_normal(shape), 1 + 0.1 * r.standard_normal(shape)
    ga, be = 1 + 0.1 * r.standard_normal(shape), 0.1 * r.standard_normal(shape)
    x, gy = r.standard_normal((B, *shape)), r.standard_normal((B, *shape))
    args = [w, b, s, ga, be, x]
    grads = orc.outer_backward(*args, gy, 2, 2, 4)
    eps = 1e-6
    for ai in range(6):
        idx = tuple(int(r.integers(0, d)) for d in args[ai].shape)
        ap, am = [a.copy() for a in args], [a.copy() for a in args]
        ap[ai][idx] += eps
        am[ai][idx] -= eps
        fd = float(((orc.outer_forward(*ap, 2, 2, 4) - orc.outer_forward(*am, 2, 2, 4)) * gy).sum()) / (2 * eps)
        assert abs(fd - grads[ai][idx]) <= 1e-6 * (1 + abs(fd)), (ai, fd, grads[ai][idx])
