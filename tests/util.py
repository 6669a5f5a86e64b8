"""Helpers shared by the test modules: seeded inputs and the tolerance policy."""
import numpy as np

# The parity bar for float32 results against the float64 oracle:
# |ours - ref| <= ATOL + RTOL * |ref| elementwise.
RTOL = 1e-4
ATOL = 1e-5


def rng_inputs(seed, B, shape, gated=False, dtype=np.float32, unit_scale=False):
    """randn inputs like gridnet/backend_cuda_test.py:23-26 (all-randn parameters), or
    with ``unit_scale`` the model initialisation of gridnet/__init__.py:42-49
    (weights N(0, 1/27), bias 0, residual scale 1)."""
    r = np.random.default_rng(seed)
    x = r.standard_normal((B, *shape)).astype(dtype)
    if gated:
        w = r.standard_normal((27, 2, *shape)).astype(dtype)
        b = r.standard_normal((2, *shape)).astype(dtype)
        if unit_scale:
            w = (w / np.sqrt(27)).astype(dtype)
        return w, b, x
    w = r.standard_normal((27, *shape)).astype(dtype)
    b = r.standard_normal(shape).astype(dtype)
    s = r.standard_normal(shape).astype(dtype)
    if unit_scale:
        w = (w / np.sqrt(27)).astype(dtype)
        b = np.zeros(shape, dtype)
        s = np.ones(shape, dtype)
    return w, b, s, x


def assert_close(ours, ref64, ref32=None, what="", rtol=RTOL, atol=ATOL, noise_factor=2.0):
    """Elementwise 1e-4 relative / 1e-5 absolute against the float64 oracle.

    Deep inner loops amplify float32 rounding noise, and gradients that are sums with
    cancellation carry an error that scales with the summands, not with the (small) result:
    the float32 ORACLE itself then shows errors against float64 of the size of our miss
    (measured for the reference's own float32 path at 8 and more inner iterations). Only
    when ``ref32`` is given, elements outside the bar are accepted if our worst error is at
    most ``noise_factor`` (2) times the float32 oracle's worst error on the same tensor, at most
    0.1 % of the elements (plus that factor times the oracle's own share) are outside, and the
    worst error stays below 3e-4 of max|ref|. A test that needs a larger factor passes it and
    says why."""
    ours = np.asarray(ours, dtype=np.float64)
    ref64 = np.asarray(ref64, dtype=np.float64)
    assert ours.shape == ref64.shape, (what, ours.shape, ref64.shape)
    assert np.isfinite(ours).all(), f"{what}: non-finite values"
    err = np.abs(ours - ref64)
    tol = atol + rtol * np.abs(ref64)
    bad = err > tol
    if not bad.any():
        return
    detail = ""
    if ref32 is not None:
        noise = np.abs(np.asarray(ref32, dtype=np.float64) - ref64)
        bad32 = noise > tol
        scale = np.abs(ref64).max() + 1e-30
        if (err.max() <= noise_factor * noise.max() and bad.mean() <= noise_factor * bad32.mean() + 1e-3
                and err.max() / scale < 3e-4):
            return
        detail = (f" [float32 oracle: {int(bad32.sum())} outside, worst {noise.max():.3e};"
                  f" ours worst {err.max():.3e}, max|ref| {scale:.3e}]")
    i = np.unravel_index(np.argmax(err * bad), err.shape)
    raise AssertionError(
        f"{what}: {int(bad.sum())}/{bad.size} elements outside tolerance; worst at {i}: "
        f"ours={ours[i]!r} ref={ref64[i]!r} err={err[i]:.3e} tol={tol[i]:.3e}{detail}")


# ---- the reference scripts' model classes (tests/golden/make_script_model_fixtures.py, tests/test_script_models.py)
SCRIPT_MODEL_CONFIGS = {
    "mnist": ("mnist", dict(inner_iters=2, outer_iters=3, init_scale=1.0, residual_scale=1.0, gated=False,
                            remember_bias=1.0, activation="silu")),
    "mnist_gated": ("mnist", dict(inner_iters=2, outer_iters=2, init_scale=1.0, residual_scale=1.0, gated=True,
                                  remember_bias=1.0, activation="tanh")),
    "imagenet_plain": ("imagenet", dict(inner_iters=2, outer_iters=2, outer_residual=False, init_scale=1.0,
                                        residual_scale=0.5, emb_channels=4, grid_size=32, activation="leaky_relu",
                                        separate_params=False)),
    "imagenet_residual_separate": ("imagenet", dict(inner_iters=2, outer_iters=2, outer_residual=True, init_scale=1.0,
                                                    residual_scale=0.5, emb_channels=4, grid_size=32,
                                                    activation="leaky_relu", separate_params=True)),
}


def fill_state_dict(model, seed: int) -> None:
    """Overwrites every entry of ``model.state_dict()`` (in sorted name order) with seeded values that keep
    the activations tame: grid weights N(0, 0.2^2), scales 1 + 0.1 N, everything else 0.1 N."""
    import torch

    rng = np.random.default_rng(seed)
    sd = model.state_dict()
    with torch.no_grad():
        for name in sorted(sd):
            t = sd[name]
            v = rng.standard_normal(tuple(t.shape)).astype(np.float32)
            if name.endswith("residual_scale") or (name.endswith("norm.weight")):
                v = 1.0 + 0.1 * v
            elif t.dim() >= 4 and t.shape[0] == 27:
                v = 0.2 * v
            else:
                v = 0.1 * v
            t.copy_(torch.from_numpy(v).to(t.device))


def script_model_inputs(kind: str, seed: int):
    import torch

    rng = np.random.default_rng(seed)
    if kind == "mnist":
        return torch.from_numpy(rng.random((3, 1, 28, 28)).astype(np.float32))
    return torch.from_numpy(rng.standard_normal((2, 3, 256, 256)).astype(np.float32))
