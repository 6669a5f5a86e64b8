"""GPU parity: the CUDA path (through the C ABI, via the reference-shaped op
surface) against the CPU oracle and the committed golden vectors.

Layout follows the reference's own GPU tests (gridnet/backend_cuda_test.py): same
shapes, both block sizes, both normalize values, float32 forward and float64
gradients, plus the edge cases listed in each test."""
import os

import numpy as np
import pytest
import torch

from oracle import gridnet_oracle as orc

from conftest import GOLDEN
from util import assert_close, rng_inputs

pytestmark = pytest.mark.gpu


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def ops():
    from gridnet_b200 import GatedGridnetCudaOp, GridnetCudaOp

    return GridnetCudaOp, GatedGridnetCudaOp


# ------------------------------------------------------------------ plain forward
@pytest.mark.parametrize(
    "shape,block_size,normalize",
    [
        ((16, 16, 16), 8, True),
        ((32, 64, 128), 8, True),
        ((32, 64, 128), 4, True),
        ((32, 16, 8), 4, False),
        ((24, 16, 32), 4, False),  # tuned block-4 path: eight blocks per CTA region
        ((12, 4, 20), 4, False),   # sides not multiples of 8: the one-thread-per-neuron kernel
        ((32, 16, 8), 8, False),
        ((32, 64, 128), 8, False),
        ((8, 8, 8), 8, False),
        ((8, 24, 40), 8, False),
        ((4, 4, 4), 4, True),
    ],
)
def test_forward_equivalence(shape, block_size, normalize):
    # gridnet/backend_cuda_test.py:9-36 (all-randn parameters, B = 2, 2 inner iterations, silu)
    Op, _ = ops()
    w, b, s, x = rng_inputs(1, 2, shape)
    ref64 = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), 2, block_size, 1e-5, normalize, "silu")
    ref32 = orc.step_forward(w, b, s, x, 2, block_size, 1e-5, normalize, "silu")
    got = Op.apply(dev(w), dev(b), dev(s), dev(x), 2, block_size, 1e-5, normalize, "silu").cpu().numpy()
    assert np.abs(got - ref64).max() < 2e-4  # the reference's own bar
    assert_close(got, ref64, ref32, f"forward {shape}/{block_size}/{normalize}")


@pytest.mark.parametrize("activation", ["relu", "leaky_relu", "silu", "tanh"])
@pytest.mark.parametrize("block_size,normalize", [(8, False), (4, False), (8, True)])
def test_forward_activations(activation, block_size, normalize):
    Op, _ = ops()
    shape = (16, 8, 24)
    w, b, s, x = rng_inputs(2, 3, shape)
    ref64 = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), 3, block_size, 1e-5, normalize, activation)
    ref32 = orc.step_forward(w, b, s, x, 3, block_size, 1e-5, normalize, activation)
    got = Op.apply(dev(w), dev(b), dev(s), dev(x), 3, block_size, 1e-5, normalize, activation).cpu().numpy()
    assert_close(got, ref64, ref32, f"{activation}/{block_size}/{normalize}")


@pytest.mark.parametrize("inner", [1, 2, 8, 9, 32])
@pytest.mark.parametrize("batch", [1, 5])
def test_forward_inner_depth_and_odd_batches(inner, batch):
    # model-like parameters (weights N(0, 1/27), unit scale) so that deep inner loops stay finite
    Op, _ = ops()
    shape = (16, 16, 8)
    w, b, s, x = rng_inputs(3, batch, shape, unit_scale=True)
    ref64 = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), inner, 8, 1e-5, False, "silu")
    ref32 = orc.step_forward(w, b, s, x, inner, 8, 1e-5, False, "silu")
    got = Op.apply(dev(w), dev(b), dev(s), dev(x), inner, 8, 1e-5, False, "silu").cpu().numpy()
    assert_close(got, ref64, ref32, f"inner={inner} B={batch}")


@pytest.mark.parametrize("inner", [1, 8, 9])
@pytest.mark.parametrize("batch", [1, 5])
def test_forward_block4_inner_depth_and_odd_batches(inner, batch):
    """Block 4 through the tuned kernel (grid sides multiples of 8): the compile-time inner count 8, a
    run-time one, and batches that leave CTAs with a single sample."""
    Op, _ = ops()
    shape = (16, 24, 8)
    w, b, s, x = rng_inputs(5, batch, shape, unit_scale=True)
    ref64 = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), inner, 4, 1e-5, False, "silu")
    ref32 = orc.step_forward(w, b, s, x, inner, 4, 1e-5, False, "silu")
    got = Op.apply(dev(w), dev(b), dev(s), dev(x), inner, 4, 1e-5, False, "silu").cpu().numpy()
    assert_close(got, ref64, ref32, f"block 4 inner={inner} B={batch}")


def test_forward_float64_matches_oracle_tightly():
    Op, _ = ops()
    for bs, norm in ((8, True), (4, False), (8, False), (4, True)):
        w, b, s, x = rng_inputs(4, 2, (8, 16, 8), dtype=np.float64)
        ref = orc.step_forward(w, b, s, x, 2, bs, 1e-5, norm, "silu")
        got = Op.apply(dev(w), dev(b), dev(s), dev(x), 2, bs, 1e-5, norm, "silu").cpu().numpy()
        assert np.abs(got - ref).max() < 1e-10 * (1 + np.abs(ref).max())


def test_known_answers():
    # gridnet/backend_torch_test.py:10-60
    Op, _ = ops()
    shape = (16, 16, 16)
    w, b, s, x = rng_inputs(5, 2, shape)
    out = Op.apply(dev(w), dev(b), dev(np.ones_like(s)), dev(x), 0, 8, 1e-5, True, "silu")
    assert torch.equal(out.cpu(), torch.from_numpy(x))
    zw = np.zeros_like(w)
    sc = np.full(shape, 0.31, np.float32)
    for norm in (True, False):
        out = Op.apply(dev(zw), dev(b), dev(sc), dev(x), 10, 8, 1e-5, norm, "silu").cpu().numpy()
        want = x + 10 * (b / (1 + np.exp(-b.astype(np.float64)))) * 0.31
        np.testing.assert_allclose(out, want, rtol=1e-5, atol=1e-5)


def test_boundary_and_interior_blocks_see_the_right_halo():
    # one hot voxel per sample placed at a block corner: its influence must cross into every
    # neighbouring block through the halo, and stop at the grid boundary
    Op, _ = ops()
    shape = (24, 24, 24)
    w, b, s, _ = rng_inputs(6, 1, shape, unit_scale=True)
    x = np.zeros((4, *shape), np.float32)
    x[0, 8, 8, 8] = 1.0   # interior corner shared by 8 blocks
    x[1, 0, 0, 0] = 1.0   # grid corner
    x[2, 23, 15, 16] = 1.0
    x[3, 7, 23, 0] = 1.0
    ref = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), 2, 8, 1e-5, False, "silu")
    got = Op.apply(dev(w), dev(b), dev(s), dev(x), 2, 8, 1e-5, False, "silu").cpu().numpy()
    assert_close(got, ref, None, "hot voxel")


def test_golden_forward_vectors():
    Op, _ = ops()
    z = np.load(os.path.join(GOLDEN, "step_forward.npz"))
    for c in sorted({k.split("_")[0] for k in z.files if k.endswith("_meta")}):
        bs, inner, norm = (int(v) for v in z[f"{c}_meta"])
        act = str(z[f"{c}_act"])
        w, b, s, x = (z[f"{c}_{k}"] for k in ("w", "b", "s", "x"))
        got = Op.apply(dev(w), dev(b), dev(s), dev(x), inner, bs, 1e-5, bool(norm), act).cpu().numpy()
        assert_close(got, z[f"{c}_y64"], z[f"{c}_y32"], f"golden forward {c}")


# ----------------------------------------------------------------- plain backward
def _grads(Op, w, b, s, x, gy, inner, bs, norm, act, dtype):
    tw, tb, ts, tx = (dev(a, dtype).requires_grad_(True) for a in (w, b, s, x))
    out = Op.apply(tw, tb, ts, tx, inner, bs, 1e-5, norm, act)
    gs, gb, gw, gx = torch.autograd.grad(out, (ts, tb, tw, tx), dev(gy, dtype))
    return [g.cpu().numpy() for g in (gw, gb, gs, gx)]


@pytest.mark.parametrize(
    "shape,inner_iters,block_size,normalize",
    [
        ((16, 16, 16), 1, 8, True),
        ((16, 16, 16), 2, 8, True),
        ((32, 64, 128), 2, 8, True),
        ((32, 64, 128), 2, 4, True),
        ((32, 16, 8), 2, 4, False),
        ((32, 16, 8), 2, 8, False),
    ],
)
def test_grad_equivalence_float64(shape, inner_iters, block_size, normalize):
    # gridnet/backend_cuda_test.py:61-110: float64, grads w.r.t. scales, biases, weights, inputs
    Op, _ = ops()
    w, b, s, x = rng_inputs(7, 2, shape, dtype=np.float64)
    gy = np.random.default_rng(8).standard_normal(x.shape)
    want = orc.step_backward(w, b, s, x, gy, inner_iters, block_size, 1e-5, normalize, "silu")
    got = _grads(Op, w, b, s, x, gy, inner_iters, block_size, normalize, "silu", torch.float64)
    for name, g, r in zip(("weights", "biases", "scales", "inputs"), got, want):
        err = np.abs(g - r).max()
        assert err < 3e-4, f"MAE in {name}: {err}"  # the reference's bar
        assert err < 1e-9 * (1 + np.abs(r).max()), f"{name}: {err}"


@pytest.mark.parametrize("activation", ["relu", "leaky_relu", "silu", "tanh"])
@pytest.mark.parametrize("block_size,normalize,inner", [(8, False, 2), (8, False, 1), (8, False, 5), (4, False, 3), (8, True, 2), (4, True, 1)])
def test_grad_float32(activation, block_size, normalize, inner):
    Op, _ = ops()
    shape = (8, 16, 16)
    w, b, s, x = rng_inputs(9, 3, shape, unit_scale=not normalize)
    if not normalize:
        b = (0.1 * np.random.default_rng(10).standard_normal(shape)).astype(np.float32)
    gy = np.random.default_rng(11).standard_normal(x.shape).astype(np.float32)
    a64 = [a.astype(np.float64) for a in (w, b, s, x, gy)]
    want = orc.step_backward(*a64, inner, block_size, 1e-5, normalize, activation)
    noise = orc.step_backward(w, b, s, x, gy, inner, block_size, 1e-5, normalize, activation)
    got = _grads(Op, w, b, s, x, gy, inner, block_size, normalize, activation, torch.float32)
    for name, g, r, n in zip(("gw", "gb", "gs", "gx"), got, want, noise):
        assert_close(g, r, n, f"{name} {activation}/{block_size}/{normalize}")


@pytest.mark.parametrize("inner", [8, 9, 32])
def test_grad_deep_inner(inner):
    # stash boundaries of the reference kernel (8 / 16 / 32, src/gridnet_cuda_kernels.cu:829-836)
    Op, _ = ops()
    shape = (8, 8, 16)
    w, b, s, x = rng_inputs(12, 2, shape, unit_scale=True, dtype=np.float64)
    w *= 0.5
    gy = np.random.default_rng(13).standard_normal(x.shape)
    want = orc.step_backward(w, b, s, x, gy, inner, 8, 1e-5, False, "silu")
    got = _grads(Op, w, b, s, x, gy, inner, 8, False, "silu", torch.float64)
    for name, g, r in zip(("gw", "gb", "gs", "gx"), got, want):
        assert np.abs(g - r).max() < 1e-9 * (1 + np.abs(r).max()), name


def test_golden_backward_vectors():
    Op, _ = ops()
    z = np.load(os.path.join(GOLDEN, "step_backward.npz"))
    for c in sorted({k.split("_")[0] for k in z.files if k.endswith("_meta")}):
        bs, inner, norm = (int(v) for v in z[f"{c}_meta"])
        act = str(z[f"{c}_act"])
        w, b, s, x, gy = (z[f"{c}_{k}"].astype(np.float64) for k in ("w", "b", "s", "x", "gy"))
        got = _grads(Op, w, b, s, x, gy, inner, bs, bool(norm), act, torch.float64)
        for name, g in zip(("gw", "gb", "gs", "gx"), got):
            r = z[f"{c}_{name}"]
            assert np.abs(g - r).max() < 1e-9 * (1 + np.abs(r).max()), (c, name)


def test_backward_overwrites_its_outputs():
    # gradient buffers handed to the extension may hold garbage: every element is written
    from gridnet_b200 import gridnet_cuda

    shape = (8, 8, 8)
    w, b, s, x = rng_inputs(14, 2, shape, dtype=np.float64)
    gy = np.random.default_rng(15).standard_normal(x.shape)
    want = orc.step_backward(w, b, s, x, gy, 2, 8, 1e-5, False, "silu")
    bufs = [torch.full(a.shape, 7.0, dtype=torch.float64, device="cuda") for a in (w, b, s, x)]
    gridnet_cuda.backward(dev(w), dev(b), dev(s), dev(x), dev(gy), *bufs, 2, 8, 1e-5, False, "silu")
    for g, r in zip(bufs, want):
        assert np.abs(g.cpu().numpy() - r).max() < 1e-9 * (1 + np.abs(r).max())


# -------------------------------------------------------------------------- gated
@pytest.mark.parametrize("shape,block_size", [((16, 16, 16), 8), ((32, 64, 128), 8), ((32, 64, 128), 4)])
def test_forward_equivalence_gated(shape, block_size):
    # gridnet/backend_cuda_test.py:39-58
    _, Gated = ops()
    w, b, x = rng_inputs(16, 2, shape, gated=True)
    ref64 = orc.gated_forward(*(a.astype(np.float64) for a in (w, b, x)), 2, block_size, "tanh")
    ref32 = orc.gated_forward(w, b, x, 2, block_size, "tanh")
    got = Gated.apply(dev(w), dev(b), dev(x), 2, block_size, "tanh").cpu().numpy()
    assert np.abs(got - ref64).max() < 2e-4
    assert_close(got, ref64, ref32, f"gated {shape}/{block_size}")


@pytest.mark.parametrize("activation", ["relu", "leaky_relu", "silu", "tanh"])
@pytest.mark.parametrize("inner,batch", [(1, 1), (3, 5), (8, 9)])
def test_gated_forward_tuned_kernel_details(activation, inner, batch):
    """The tuned gated forward (float32, block 8): every activation, inner counts that end on either
    ping-pong tile, batches that leave CTAs with one sample, a non-cubic grid with corner blocks."""
    _, Gated = ops()
    shape = (8, 24, 16)
    w, b, x = rng_inputs(18, batch, shape, gated=True)
    w = (w / 3).astype(np.float32)  # keeps eight iterations tame
    ref64 = orc.gated_forward(*(a.astype(np.float64) for a in (w, b, x)), inner, 8, activation)
    ref32 = orc.gated_forward(w, b, x, inner, 8, activation)
    got = Gated.apply(dev(w), dev(b), dev(x), inner, 8, activation).cpu().numpy()
    assert_close(got, ref64, ref32, f"gated {activation} inner={inner} B={batch}")


@pytest.mark.parametrize(
    "shape,inner_iters,block_size",
    [((16, 16, 16), 1, 8), ((16, 16, 16), 2, 8), ((32, 64, 128), 2, 8), ((32, 64, 128), 2, 4)],
)
def test_grad_equivalence_gated(shape, inner_iters, block_size):
    # gridnet/backend_cuda_test.py:113-152
    _, Gated = ops()
    w, b, x = rng_inputs(17, 2, shape, gated=True, dtype=np.float64)
    gy = np.random.default_rng(18).standard_normal(x.shape)
    want = orc.gated_backward(w, b, x, gy, inner_iters, block_size, "tanh")
    tw, tb, tx = (dev(a).requires_grad_(True) for a in (w, b, x))
    out = Gated.apply(tw, tb, tx, inner_iters, block_size, "tanh")
    gb, gw, gx = torch.autograd.grad(out, (tb, tw, tx), dev(gy))
    for name, g, r in zip(("weights", "biases", "inputs"), (gw, gb, gx), want):
        g = g.cpu().numpy()
        assert np.isfinite(g).all()
        err = np.abs(g - r).max()
        assert err < 3e-4, f"MAE in {name}: {err}"
        assert err < 1e-9 * (1 + np.abs(r).max()), name


@pytest.mark.parametrize("block_size", [8, 4])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_gated_gradients_with_zero_inner_iterations(block_size, dtype):
    """inner_iters = 0 is the identity: grad_x = grad_y exactly (every cell, also the ones other threads own),
    parameter gradients zero. Checked repeatedly, since the fault this guards against was a race."""
    _, Gated = ops()
    shape = (16, 16, 24)
    w, b, x = rng_inputs(19, 3, shape, gated=True, dtype=dtype)
    gy = np.random.default_rng(20).standard_normal(x.shape).astype(dtype)
    want = orc.gated_backward(w.astype(np.float64), b.astype(np.float64), x.astype(np.float64), gy.astype(np.float64), 0,
                              block_size, "tanh")
    for _ in range(5):
        tw, tb, tx = (dev(a).requires_grad_(True) for a in (w, b, x))
        out = Gated.apply(tw, tb, tx, 0, block_size, "tanh")
        assert torch.equal(out, tx)
        gw, gb, gx = torch.autograd.grad(out, (tw, tb, tx), dev(gy))
        assert torch.equal(gx, dev(gy))
        assert not gw.any() and not gb.any()
        for g, r in zip((gw, gb, gx), want):
            assert np.array_equal(g.cpu().numpy().astype(np.float64), r)


def test_golden_gated_vectors():
    _, Gated = ops()
    z = np.load(os.path.join(GOLDEN, "gated.npz"))
    for c in sorted({k.split("_")[0] for k in z.files if k.endswith("_meta")}):
        bs, inner = (int(v) for v in z[f"{c}_meta"])
        act = str(z[f"{c}_act"])
        w, b, x, gy = (z[f"{c}_{k}"] for k in ("w", "b", "x", "gy"))
        got = Gated.apply(dev(w), dev(b), dev(x), inner, bs, act).cpu().numpy()
        assert_close(got, z[f"{c}_y64"], z[f"{c}_y32"], f"golden gated {c}")
        tw, tb, tx = (dev(a, torch.float64).requires_grad_(True) for a in (w, b, x))
        out = Gated.apply(tw, tb, tx, inner, bs, act)
        gw, gb, gx = torch.autograd.grad(out, (tw, tb, tx), dev(gy, torch.float64))
        for name, g in zip(("gw", "gb", "gx"), (gw, gb, gx)):
            r = z[f"{c}_{name}"]
            assert np.abs(g.cpu().numpy() - r).max() < 1e-9 * (1 + np.abs(r).max()), (c, name)


# ------------------------------------------------------------------- error paths
def test_extension_layer_errors():
    # RuntimeError for non-contiguous tensors and unknown activations, as the reference's
    # C++ layer raises (src/gridnet_cuda.cpp:6-10, src/activations.h:15-16)
    from gridnet_b200 import gridnet_cuda

    Op, _ = ops()
    shape = (8, 8, 8)
    w, b, s, x = (dev(a) for a in rng_inputs(19, 2, shape))
    with pytest.raises(RuntimeError, match="unknown activation"):
        Op.apply(w, b, s, x, 1, 8, 1e-5, False, "gelu")
    y = torch.empty_like(x)
    xt = x.transpose(1, 2)
    with pytest.raises(RuntimeError, match="contiguous"):
        gridnet_cuda.forward(w, b, s, xt, y, 1, 8, 1e-5, False, "silu")
    from gridnet_b200._lib import lib

    big = lib.gn_step_backward_max_inner(8, 8) + 1
    tw = w.double().requires_grad_(True)
    # (double precision: the one-kernel backward with its shared-memory stash; the tuned float paths
    # have no such limit)
    out = Op.apply(tw, b.double(), s.double(), x.double(), big, 8, 1e-5, True, "relu")
    with pytest.raises(RuntimeError, match="inner"):
        out.sum().backward()
    # an empty batch returns a clone without launching anything
    e = torch.empty(0, *shape, device="cuda")
    assert Op.apply(w, b, s, e, 1, 8, 1e-5, False, "silu").shape == e.shape
    # a non-contiguous upstream gradient is accepted (made contiguous by the op)
    tx = x.clone().requires_grad_(True)
    out = Op.apply(w, b, s, tx, 1, 8, 1e-5, False, "silu")
    out.transpose(1, 2).contiguous().transpose(1, 2).backward(torch.ones_like(out))
    assert torch.isfinite(tx.grad).all()


def test_forward_with_unaligned_activations_uses_the_plain_load_path():
    # TMA tile fetch needs a 16-byte aligned activation tensor; a view that starts 4 bytes into a
    # buffer makes the tuned kernel fall back to plain loads, which must give the same result
    Op, _ = ops()
    shape = (16, 24, 16)
    w, b, s, x = rng_inputs(40, 3, shape, unit_scale=True)
    ref64 = orc.step_forward(*(a.astype(np.float64) for a in (w, b, s, x)), 4, 8, 1e-5, False, "silu")
    store = torch.zeros(x.size + 1, device="cuda")
    xv = store[1:].view(x.shape)
    xv.copy_(torch.from_numpy(x))
    assert xv.data_ptr() % 16 == 4 and xv.is_contiguous()
    got_unaligned = Op.apply(dev(w), dev(b), dev(s), xv, 4, 8, 1e-5, False, "silu")
    got_aligned = Op.apply(dev(w), dev(b), dev(s), dev(x), 4, 8, 1e-5, False, "silu")
    assert torch.equal(got_unaligned, got_aligned)
    assert_close(got_aligned.cpu().numpy(), ref64, None, "unaligned x")


@pytest.mark.parametrize("block", [8, 4])
def test_keep_forward_stash_gives_identical_gradients(block):
    """The autograd op with the memory-for-time switch on: same output and the same gradient bits, also when
    the graph is differentiated twice (the second pass has no stash left and recomputes)."""
    import gridnet_b200 as gb

    Op, _ = ops()
    shape, B, inner = (16, 24, 8), 3, 4
    w, b, s, x = rng_inputs(51, B, shape, unit_scale=True)
    gy = dev(np.random.default_rng(52).standard_normal(x.shape).astype(np.float32))

    def run():
        t = [dev(a).requires_grad_(True) for a in (w, b, s, x)]
        y = Op.apply(*t, inner, block, 1e-5, False, "silu")
        g1 = torch.autograd.grad(y, t, gy, retain_graph=True)
        g2 = torch.autograd.grad(y, t, gy)
        return y.detach(), g1, g2

    default = gb.keep_forward_stash(False)  # recompute, like the reference
    try:
        y0, ga, gb2 = run()
        assert gb.keep_forward_stash(True) is False
        y1, gc, gd = run()
    finally:
        gb.keep_forward_stash(default)
    assert default is None and torch.equal(y0, y1)  # the package default decides from the free memory
    for a, b_, c, d in zip(ga, gb2, gc, gd):
        assert torch.equal(a, b_) and torch.equal(a, c) and torch.equal(a, d)


@pytest.mark.parametrize("block", [8, 4])
def test_tuned_backward_equals_one_kernel_backward(block):
    """float32, normalize off: the four-kernel path (with workspace) against the one-kernel path
    (without) and the float64 oracle, on a grid with interior, face, edge and corner blocks, an odd
    batch, and through the C ABI directly."""
    from gridnet_b200._lib import lib

    shape, B, inner = (24, 16, 32), 5, 3
    w, b, s, x = rng_inputs(41, B, shape, unit_scale=True)
    b = (0.1 * np.random.default_rng(42).standard_normal(shape)).astype(np.float32)
    s = (1 + 0.1 * np.random.default_rng(43).standard_normal(shape)).astype(np.float32)
    gy = np.random.default_rng(44).standard_normal(x.shape).astype(np.float32)
    want = orc.step_backward(*(a.astype(np.float64) for a in (w, b, s, x, gy)), inner, block, 1e-5, False, "silu")
    noise = orc.step_backward(w, b, s, x, gy, inner, block, 1e-5, False, "silu")
    tw, tb, ts, tx, tgy = (dev(a) for a in (w, b, s, x, gy))
    M, N, K = shape
    stream = torch.cuda.current_stream().cuda_stream
    outs = {}
    for tag in ("plain", "tuned", "tuned again"):
        g = [torch.full_like(t, 3.0) for t in (tw, tb, ts, tx)]
        if tag == "plain":
            rc = lib.gn_step_backward_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                          *(t.data_ptr() for t in g), B, M, N, K, inner, block, 1e-5, 0, 2, stream)
        else:
            need = lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, block, 0, 4)
            assert need > 0
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            rc = lib.gn_step_backward_ws_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                             *(t.data_ptr() for t in g), B, M, N, K, inner, block, 1e-5, 0, 2,
                                             ws.data_ptr(), ws.numel(), stream)
        assert rc == 0, lib.gn_status_string(rc)
        outs[tag] = [t.cpu().numpy() for t in g]
        if tag != "plain":
            # an int inside the workspace reports a bounded wait that gave up
            off = lib.gn_step_backward_error_flag_offset(B, M, N, K, inner)
            assert 0 < off <= need - 4 and off % 4 == 0
            assert int(ws.view(torch.int32)[off // 4].item()) == 0
    for name, a, bb, r, n in zip(("gw", "gb", "gs", "gx"), outs["tuned"], outs["plain"], want, noise):
        assert_close(a, r, n, f"tuned {name}")
        assert_close(bb, r, n, f"plain {name}")
    # the tuned path has no floating-point atomics (batch chunks of a block reduce on chip in a fixed
    # order), so two runs agree bit for bit
    for name, a, a2 in zip(("gw", "gb", "gs", "gx"), outs["tuned"], outs["tuned again"]):
        assert np.array_equal(a, a2), name
    # the same gradients, bit for bit, when the forward pass kept its intermediate results (no replay)
    y_plain = torch.empty_like(tx)
    assert lib.gn_step_forward_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), y_plain.data_ptr(),
                                   B, M, N, K, inner, block, 1e-5, 0, 2, stream) == 0
    nst = lib.gn_step_stash_bytes(B, M, N, K, inner, block)
    nws = lib.gn_step_backward_stash_workspace_bytes(B, M, N, K, inner, block)
    assert nst > 0 and 0 < nws < need
    stash = torch.empty(nst, dtype=torch.uint8, device="cuda")
    ws2 = torch.empty(nws, dtype=torch.uint8, device="cuda")
    y_stash = torch.empty_like(tx)
    assert lib.gn_step_forward_stash_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), y_stash.data_ptr(),
                                         B, M, N, K, inner, block, 2, stash.data_ptr(), stash.numel(), stream) == 0
    assert torch.equal(y_stash, y_plain)
    g = [torch.full_like(t, 3.0) for t in (tw, tb, ts, tx)]
    rc = lib.gn_step_backward_stash_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                        *(t.data_ptr() for t in g), B, M, N, K, inner, block, 2, stash.data_ptr(),
                                        stash.numel(), ws2.data_ptr(), ws2.numel(), stream)
    assert rc == 0, lib.gn_status_string(rc)
    off = lib.gn_step_backward_stash_error_flag_offset(B, M, N, K, inner)
    assert int(ws2.view(torch.int32)[off // 4].item()) == 0
    for name, a, t in zip(("gw", "gb", "gs", "gx"), outs["tuned"], g):
        assert np.array_equal(a, t.cpu().numpy()), name
    # too small a stash or workspace is refused, not overrun
    assert lib.gn_step_backward_stash_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                          *(t.data_ptr() for t in g), B, M, N, K, inner, block, 2, stash.data_ptr(),
                                          stash.numel() - 512, ws2.data_ptr(), ws2.numel(), stream) == -6
    # no tuned path: sides that are not multiples of 8, per-block normalisation at block 4, double precision
    assert lib.gn_step_stash_bytes(B, 12, N, K, inner, 4) == 0
    assert lib.gn_step_backward_workspace_bytes(B, 12, N, K, inner, 4, 0, 4) == 0
    assert lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, 4, 1, 4) == 0
    assert lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, block, 0, 8) == 0


@pytest.mark.parametrize("activation", ["silu", "tanh", "leaky_relu"])
def test_tuned_backward_with_per_block_normalisation(activation):
    """float32, normalize on, block 8: the four-kernel path (replay with tile statistics, reverse sweep with the
    two block sums, weight gradients on mean-free tiles, cross-block kernel with the halo terms) against the
    float64 oracle on a grid with interior, face, edge and corner blocks and an odd batch; bit-identical when
    repeated (no floating-point atomics); and against the one-kernel path, which scatters with atomics
    (gridnet/backend_torch.py:92-97, src/gridnet_cuda_kernels.cu:396-416)."""
    from gridnet_b200._lib import lib

    shape, B, inner = (24, 16, 32), 5, 3
    w, b, s, x = rng_inputs(51, B, shape, unit_scale=False)
    x = (x + 0.5).astype(np.float32)  # tiles with a mean
    b = (0.1 * np.random.default_rng(52).standard_normal(shape)).astype(np.float32)
    s = (1 + 0.1 * np.random.default_rng(53).standard_normal(shape)).astype(np.float32)
    gy = np.random.default_rng(54).standard_normal(x.shape).astype(np.float32)
    act = {"relu": 0, "leaky_relu": 1, "silu": 2, "tanh": 3}[activation]
    assert act == lib.gn_activation_from_name(activation.encode())
    want = orc.step_backward(*(a.astype(np.float64) for a in (w, b, s, x, gy)), inner, 8, 1e-5, True, activation)
    noise = orc.step_backward(w, b, s, x, gy, inner, 8, 1e-5, True, activation)
    tw, tb, ts, tx, tgy = (dev(a) for a in (w, b, s, x, gy))
    M, N, K = shape
    stream = torch.cuda.current_stream().cuda_stream
    outs = {}
    for tag in ("plain", "tuned", "tuned again"):
        g = [torch.full_like(t, 3.0) for t in (tw, tb, ts, tx)]
        if tag == "plain":
            rc = lib.gn_step_backward_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                          *(t.data_ptr() for t in g), B, M, N, K, inner, 8, 1e-5, 1, act, stream)
        else:
            need = lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, 8, 1, 4)
            assert need > lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, 8, 0, 4) > 0
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            rc = lib.gn_step_backward_ws_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                             *(t.data_ptr() for t in g), B, M, N, K, inner, 8, 1e-5, 1, act,
                                             ws.data_ptr(), ws.numel(), stream)
        assert rc == 0, lib.gn_status_string(rc)
        outs[tag] = [t.cpu().numpy() for t in g]
    for name, a, c in zip(("gw", "gb", "gs", "gx"), outs["tuned"], outs["tuned again"]):
        assert np.array_equal(a, c), f"{name}: the tuned path is not bit-reproducible"
    for tag in ("plain", "tuned"):
        for name, g, r, n in zip(("gw", "gb", "gs", "gx"), outs[tag], want, noise):
            assert_close(g, r, n, f"{tag} {name} {activation}, normalize on")
    assert lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, 4, 1, 4) == 0  # block 4 keeps the one-kernel path


@pytest.mark.parametrize("activation,inner", [("tanh", 3), ("silu", 2), ("relu", 1), ("leaky_relu", 4)])
def test_tuned_gated_backward(activation, inner):
    """float32 gated backward at block 8: the four-kernel path (with workspace) against the float64 oracle and
    the one-kernel path on a grid with interior, face, edge and corner blocks and an odd batch, through the C ABI;
    bit-identical when repeated (src/gridnet_cuda_kernels.cu:538-734, gridnet/backend_torch.py:145-267)."""
    from gridnet_b200._lib import lib

    shape, B = (24, 16, 32), 5
    w, b, x = rng_inputs(71, B, shape, gated=True, unit_scale=True)
    b = (0.3 * b).astype(np.float32)
    gy = np.random.default_rng(72).standard_normal(x.shape).astype(np.float32)
    act = lib.gn_activation_from_name(activation.encode())
    want = orc.gated_backward(*(a.astype(np.float64) for a in (w, b, x, gy)), inner, 8, activation)
    noise = orc.gated_backward(w, b, x, gy, inner, 8, activation)
    tw, tb, tx, tgy = (dev(a) for a in (w, b, x, gy))
    M, N, K = shape
    stream = torch.cuda.current_stream().cuda_stream
    outs = {}
    for tag in ("plain", "tuned", "tuned again"):
        g = [torch.full_like(t, 3.0) for t in (tw, tb, tx)]
        if tag == "plain":
            rc = lib.gn_gated_backward_f32(tw.data_ptr(), tb.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                           *(t.data_ptr() for t in g), B, M, N, K, inner, 8, act, stream)
        else:
            need = lib.gn_gated_backward_workspace_bytes(B, M, N, K, inner, 8, 4)
            assert need > 0
            ws = torch.empty(need, dtype=torch.uint8, device="cuda")
            rc = lib.gn_gated_backward_ws_f32(tw.data_ptr(), tb.data_ptr(), tx.data_ptr(), tgy.data_ptr(),
                                              *(t.data_ptr() for t in g), B, M, N, K, inner, 8, act, ws.data_ptr(),
                                              ws.numel(), stream)
            off = lib.gn_gated_backward_error_flag_offset(B, M, N, K, inner)
            assert int(ws.view(torch.int32)[off // 4].item()) == 0
        assert rc == 0, lib.gn_status_string(rc)
        outs[tag] = [t.cpu().numpy() for t in g]
    for name, a, c in zip(("gw", "gb", "gx"), outs["tuned"], outs["tuned again"]):
        assert np.array_equal(a, c), f"{name}: the tuned path is not bit-reproducible"
    for tag in ("plain", "tuned"):
        for name, g, r, n in zip(("gw", "gb", "gx"), outs[tag], want, noise):
            assert_close(g, r, n, f"{tag} gated {name} {activation} inner={inner}")
    # no tuned path: block 4, double precision, sides that are not multiples of 8; too small a workspace falls back
    assert lib.gn_gated_backward_workspace_bytes(B, M, N, K, inner, 4, 4) == 0
    assert lib.gn_gated_backward_workspace_bytes(B, M, N, K, inner, 8, 8) == 0
    assert lib.gn_gated_backward_workspace_bytes(B, 12, N, K, inner, 8, 4) == 0


@pytest.mark.parametrize("with_stash", [False, True])
def test_backward_on_a_raw_input_with_statistics(with_stash):
    """gn_step_backward_fused_in_f32 (the step backward inside the model loop: raw output of the step before, its
    statistics and the LayerNorm parameters instead of the normalised tensor) against normalising first and calling
    the ordinary workspace / stash entry points: same bits, with the inner iterations replayed and kept."""
    from gridnet_b200._lib import lib

    shape, B, inner = (24, 16, 32), 5, 3
    M, N, K = shape
    P = M * N * K
    w, b, s, xraw = rng_inputs(91, B, shape, unit_scale=True)
    r = np.random.default_rng(92)
    b = (0.1 * r.standard_normal(shape)).astype(np.float32)
    gamma = (1 + 0.1 * r.standard_normal(shape)).astype(np.float32)
    beta = (0.1 * r.standard_normal(shape)).astype(np.float32)
    xraw = (0.7 * xraw + 0.2).astype(np.float32)
    gy = r.standard_normal(xraw.shape).astype(np.float32)
    tw, tb, ts, tx, tgy, tga, tbe = (dev(a) for a in (w, b, s, xraw, gy, gamma, beta))
    st = torch.cuda.current_stream().cuda_stream
    # statistics and the normalised tensor through the library's own LayerNorm
    nws = torch.empty(int(lib.gn_norm_workspace_bytes(B, P)), dtype=torch.uint8, device="cuda")
    xn, mr = torch.empty_like(tx), torch.empty(B, 2, device="cuda")
    assert lib.gn_norm_forward_f32(tx.data_ptr(), tga.data_ptr(), tbe.data_ptr(), xn.data_ptr(), mr.data_ptr(), B, P, 1e-5,
                                   nws.data_ptr(), nws.numel(), st) == 0
    stash = None
    if with_stash:
        stash = torch.empty(int(lib.gn_step_stash_bytes(B, M, N, K, inner, 8)), dtype=torch.uint8, device="cuda")
        y = torch.empty_like(tx)
        assert lib.gn_step_forward_stash_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), xn.data_ptr(), y.data_ptr(), B, M, N,
                                             K, inner, 8, 2, stash.data_ptr(), stash.numel(), st) == 0
        need = int(lib.gn_step_backward_stash_workspace_bytes(B, M, N, K, inner, 8))
    else:
        need = int(lib.gn_step_backward_workspace_bytes(B, M, N, K, inner, 8, 0, 4))
    outs = {}
    for tag in ("normalised first", "raw input"):
        g = [torch.full_like(t, 3.0) for t in (tw, tb, ts, tx)]
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        if tag == "raw input":
            rc = lib.gn_step_backward_fused_in_f32(
                tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), mr.data_ptr(), tga.data_ptr(), tbe.data_ptr(),
                tgy.data_ptr(), *(t.data_ptr() for t in g), B, M, N, K, inner, 8, 2,
                None if stash is None else stash.data_ptr(), 0 if stash is None else stash.numel(), ws.data_ptr(),
                ws.numel(), st)
        elif with_stash:
            rc = lib.gn_step_backward_stash_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), xn.data_ptr(), tgy.data_ptr(),
                                                *(t.data_ptr() for t in g), B, M, N, K, inner, 8, 2, stash.data_ptr(),
                                                stash.numel(), ws.data_ptr(), ws.numel(), st)
        else:
            rc = lib.gn_step_backward_ws_f32(tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), xn.data_ptr(), tgy.data_ptr(),
                                             *(t.data_ptr() for t in g), B, M, N, K, inner, 8, 1e-5, 0, 2, ws.data_ptr(),
                                             ws.numel(), st)
        assert rc == 0, lib.gn_status_string(rc)
        outs[tag] = [t.cpu().numpy() for t in g]
    for name, a, c in zip(("gw", "gb", "gs", "gx"), outs["normalised first"], outs["raw input"]):
        assert np.array_equal(a, c), f"{name}: normalising while loading changed the bits"
    # block 4 has no such path
    assert lib.gn_step_backward_fused_in_f32(
        tw.data_ptr(), tb.data_ptr(), ts.data_ptr(), tx.data_ptr(), mr.data_ptr(), tga.data_ptr(), tbe.data_ptr(),
        tgy.data_ptr(), *(t.data_ptr() for t in g), B, M, N, K, inner, 4, 2, None, 0, ws.data_ptr(), ws.numel(), st) == -8
