"""Seeded random sweep over grid shapes, batch sizes, inner counts, block sizes and activations for the
plain op (forward and all four gradients) and the gated forward, against the float64 oracle: catches
index arithmetic that only breaks on unusual combinations (single-block sides, one sample, batches that
do not divide over the CTAs, sides that are multiples of 4 but not of 8)."""
import numpy as np
import pytest
import torch

from oracle import gridnet_oracle as orc

from util import assert_close, rng_inputs

pytestmark = pytest.mark.gpu

ACTS = ["relu", "leaky_relu", "silu", "tanh"]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _cases(seed, n):
    r = np.random.default_rng(seed)
    out = []
    for i in range(n):
        bs = int(r.choice([8, 4]))
        unit = int(r.choice([8, 8, 8, 4])) if bs == 4 else 8  # block 4: some sides not multiples of 8
        shape = tuple(int(unit * r.integers(1, 5)) for _ in range(3))
        out.append((i, shape, bs, int(r.integers(1, 10)), int(r.integers(1, 6)), ACTS[int(r.integers(0, 4))]))
    return out


@pytest.mark.parametrize("case,shape,bs,batch,inner,act", _cases(2024, 24))
def test_plain_forward_backward_random(case, shape, bs, batch, inner, act):
    import gridnet_b200 as gb

    w, b, s, x = rng_inputs(1000 + case, batch, shape, unit_scale=True)
    gy = np.random.default_rng(2000 + case).standard_normal(x.shape).astype(np.float32)
    a64 = [a.astype(np.float64) for a in (w, b, s, x)]
    ref_y = orc.step_forward(*a64, inner, bs, 1e-5, False, act)
    ref_y32 = orc.step_forward(w, b, s, x, inner, bs, 1e-5, False, act)
    tw, tb, ts, tx = (dev(a).requires_grad_(True) for a in (w, b, s, x))
    y = gb.GridnetCudaOp.apply(tw, tb, ts, tx, inner, bs, 1e-5, False, act)
    assert_close(y.detach().cpu().numpy(), ref_y, ref_y32, f"forward {shape} bs={bs} B={batch} inner={inner} {act}")
    grads = torch.autograd.grad(y, (tw, tb, ts, tx), dev(gy))
    ref_g = orc.step_backward(*a64, gy.astype(np.float64), inner, bs, 1e-5, False, act)
    ref_g32 = orc.step_backward(w, b, s, x, gy, inner, bs, 1e-5, False, act)
    for name, g, r, n32 in zip(("gw", "gb", "gs", "gx"), grads, ref_g, ref_g32):
        assert_close(g.cpu().numpy(), r, n32, f"{name} {shape} bs={bs} B={batch} inner={inner} {act}")


@pytest.mark.parametrize("case,shape,bs,batch,inner,act", _cases(2025, 12))
def test_gated_forward_random(case, shape, bs, batch, inner, act):
    import gridnet_b200 as gb

    w, b, x = rng_inputs(3000 + case, batch, shape, gated=True)
    w = (w / 3).astype(np.float32)
    ref = orc.gated_forward(*(a.astype(np.float64) for a in (w, b, x)), inner, bs, act)
    ref32 = orc.gated_forward(w, b, x, inner, bs, act)
    got = gb.GatedGridnetCudaOp.apply(dev(w), dev(b), dev(x), inner, bs, act).cpu().numpy()
    assert_close(got, ref, ref32, f"gated {shape} bs={bs} B={batch} inner={inner} {act}")
