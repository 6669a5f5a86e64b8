"""Generate the golden vectors in this directory from the reference's own CPU code.

Run once, in a container that has the reference checkout (it is NOT available
where the GPU tests run, which is why the outputs are committed):

    python tests/golden/make_golden.py /path/to/gridnet-checkout

It imports ``gridnet/backend_torch.py`` from that checkout unchanged, feeds it
seeded inputs, and stores inputs (float32, so they are exact in both precisions)
together with the reference's float32 and float64 outputs and its autograd
gradients (float64, like gridnet/backend_cuda_test.py:79-105).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from gridnet.backend_torch import gated_gridnet_step_pytorch, gridnet_step_pytorch

    torch.set_num_threads(4)
    g = torch.Generator().manual_seed(20240229)

    def rn(*shape):
        return torch.randn(*shape, generator=g, dtype=torch.float32)

    # ---- plain step, forward, all activations / both normalize values / both block sizes
    fwd = {}
    cases = [
        ("a", (16, 16, 16), 8, 2, True, "silu"),
        ("b", (8, 16, 24), 4, 2, True, "silu"),
        ("c", (16, 8, 8), 4, 3, False, "silu"),
        ("d", (16, 8, 8), 8, 2, False, "relu"),
        ("e", (8, 8, 16), 8, 1, False, "leaky_relu"),
        ("f", (8, 8, 8), 4, 2, True, "tanh"),
        ("g", (8, 8, 8), 8, 9, False, "silu"),
    ]
    for name, shape, bs, inner, norm, act in cases:
        x, w, b, s = rn(2, *shape), rn(27, *shape), rn(*shape), rn(*shape)
        if name == "g":
            w = w / 27 ** 0.5
            s = torch.ones_like(s)
        y32 = gridnet_step_pytorch(w, b, s, x, inner, bs, 1e-5, norm, act)
        y64 = gridnet_step_pytorch(w.double(), b.double(), s.double(), x.double(), inner, bs, 1e-5, norm, act)
        fwd[f"{name}_meta"] = np.array([bs, inner, int(norm)], dtype=np.int64)
        fwd[f"{name}_act"] = np.array(act)
        for k, v in dict(x=x, w=w, b=b, s=s, y32=y32, y64=y64).items():
            fwd[f"{name}_{k}"] = v.numpy()
    np.savez_compressed(os.path.join(HERE, "step_forward.npz"), **fwd)

    # ---- plain step, gradients by autograd in float64
    bwd = {}
    cases = [
        ("a", (8, 8, 16), 8, 2, True, "silu"),
        ("b", (8, 8, 8), 4, 2, True, "tanh"),
        ("c", (8, 16, 8), 4, 3, False, "silu"),
        ("d", (8, 8, 8), 8, 1, False, "leaky_relu"),
        ("e", (8, 8, 8), 8, 2, False, "relu"),
    ]
    for name, shape, bs, inner, norm, act in cases:
        x, w, b, s = (t.double().requires_grad_(True) for t in (rn(2, *shape), rn(27, *shape), rn(*shape), rn(*shape)))
        gy = rn(2, *shape).double()
        y = gridnet_step_pytorch(w, b, s, x, inner, bs, 1e-5, norm, act)
        gw, gb, gs, gx = torch.autograd.grad(y, (w, b, s, x), gy)
        bwd[f"{name}_meta"] = np.array([bs, inner, int(norm)], dtype=np.int64)
        bwd[f"{name}_act"] = np.array(act)
        for k, v in dict(x=x, w=w, b=b, s=s, gy=gy).items():
            bwd[f"{name}_{k}"] = v.detach().float().numpy()
        for k, v in dict(gw=gw, gb=gb, gs=gs, gx=gx).items():
            bwd[f"{name}_{k}"] = v.numpy()
    np.savez_compressed(os.path.join(HERE, "step_backward.npz"), **bwd)

    # ---- gated step, forward and gradients
    gat = {}
    cases = [
        ("a", (8, 8, 16), 8, 2, "tanh"),
        ("b", (8, 16, 8), 4, 2, "tanh"),
        ("c", (8, 8, 8), 4, 3, "silu"),
        ("d", (8, 8, 8), 8, 1, "relu"),
    ]
    for name, shape, bs, inner, act in cases:
        x32, w32, b32 = rn(2, *shape), rn(27, 2, *shape), rn(2, *shape)
        y32 = gated_gridnet_step_pytorch(w32, b32, x32, inner, bs, act)
        x, w, b = (t.double().requires_grad_(True) for t in (x32, w32, b32))
        gy = rn(2, *shape).double()
        y = gated_gridnet_step_pytorch(w, b, x, inner, bs, act)
        gw, gb, gx = torch.autograd.grad(y, (w, b, x), gy)
        gat[f"{name}_meta"] = np.array([bs, inner], dtype=np.int64)
        gat[f"{name}_act"] = np.array(act)
        for k, v in dict(x=x32, w=w32, b=b32, gy=gy.float(), y32=y32).items():
            gat[f"{name}_{k}"] = v.numpy()
        for k, v in dict(y64=y.detach(), gw=gw, gb=gb, gx=gx).items():
            gat[f"{name}_{k}"] = v.numpy()
    np.savez_compressed(os.path.join(HERE, "gated.npz"), **gat)

    # ---- the model loop: outer x (step, LayerNorm over the whole grid), and LayerNorm grads
    loop = {}
    shape, bs, inner, outer = (16, 16, 16), 8, 2, 4
    w = rn(27, *shape) / 27 ** 0.5
    b = 0.1 * rn(*shape)
    s = 1 + 0.1 * rn(*shape)
    gamma = 1 + 0.1 * rn(*shape)
    beta = 0.1 * rn(*shape)
    x = torch.zeros(3, *shape)
    x[..., 0] = rn(3, *shape[:2])
    outs = {}
    for dt, tag in ((torch.float32, "y32"), (torch.float64, "y64")):
        h = x.to(dt)
        ln = torch.nn.LayerNorm(shape, dtype=dt)
        with torch.no_grad():
            ln.weight.copy_(gamma.to(dt))
            ln.bias.copy_(beta.to(dt))
            for _ in range(outer):
                h = gridnet_step_pytorch(w.to(dt), b.to(dt), s.to(dt), h, inner, bs, 1e-5, False, "silu")
                h = ln(h)
        outs[tag] = h.numpy()
    loop["meta"] = np.array([bs, inner, outer], dtype=np.int64)
    for k, v in dict(x=x, w=w, b=b, s=s, gamma=gamma, beta=beta).items():
        loop[k] = v.numpy()
    loop.update(outs)
    # LayerNorm forward/backward on a random tensor, float64
    lx = rn(3, *shape).double().requires_grad_(True)
    lgam = gamma.double().requires_grad_(True)
    lbet = beta.double().requires_grad_(True)
    lgy = rn(3, *shape).double()
    ly = torch.nn.functional.layer_norm(lx, shape, lgam, lbet, 1e-5)
    lgx, lgg, lgb = torch.autograd.grad(ly, (lx, lgam, lbet), lgy)
    for k, v in dict(ln_x=lx.detach().float(), ln_gy=lgy.float()).items():
        loop[k] = v.numpy()
    # outputs recomputed from the float32-rounded inputs so that they are exact
    lx2 = lx.detach().float().double().requires_grad_(True)
    lgy2 = lgy.float().double()
    ly2 = torch.nn.functional.layer_norm(lx2, shape, lgam, lbet, 1e-5)
    lgx, lgg, lgb = torch.autograd.grad(ly2, (lx2, lgam, lbet), lgy2)
    for k, v in dict(ln_y=ly2.detach(), ln_gx=lgx, ln_gg=lgg, ln_gb=lgb).items():
        loop[k] = v.numpy()
    np.savez_compressed(os.path.join(HERE, "outer_loop.npz"), **loop)

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
