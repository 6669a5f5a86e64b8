"""A slab backend for CPU ranks that does the local arithmetic with the CPU oracle (test
infrastructure): it lets the orchestration in gridnet_b200/slab.py run under gloo without a GPU."""
import numpy as np
import torch

from oracle import gridnet_oracle as orc

from gridnet_b200.slab import GHOST


class OracleSlabBackend:
    def __init__(self, layout, weight, bias, scale, gamma, beta, inner, activation="silu", ln_eps=1e-5,
                 dtype=np.float64):
        self.layout, self.inner, self.act, self.ln_eps, self.dtype = layout, inner, activation, ln_eps, dtype
        n = lambda t: t.numpy().astype(dtype)
        self.w, self.b, self.s, self.gamma, self.beta = n(weight), n(bias), n(scale), n(gamma), n(beta)

    def step(self, x, y, in_stats):
        xin = x.numpy().astype(self.dtype)
        if in_stats is not None:
            st = in_stats.numpy().astype(self.dtype)
            xin = (xin - st[:, 0, None, None, None]) * st[:, 1, None, None, None] * self.gamma + self.beta
        out = orc.step_forward(self.w, self.b, self.s, xin, self.inner, 8, 1e-5, False, self.act)
        k = self.layout.k_loc
        real = out[..., GHOST:GHOST + k]
        y[..., GHOST:GHOST + k] = torch.from_numpy(real.astype(np.float32 if y.dtype == torch.float32 else np.float64))
        r64 = real.astype(np.float64).reshape(real.shape[0], -1)
        return torch.from_numpy(np.stack([r64.sum(1), (r64 * r64).sum(1)], 1))

    def finalize(self, sums, count):
        mean = sums[:, 0] / count
        var = (sums[:, 1] / count - mean * mean).clamp_min(0)
        return torch.stack([mean, 1.0 / torch.sqrt(var + self.ln_eps)], 1)

    def apply(self, x, stats, y):
        st = stats.numpy().astype(self.dtype)
        out = (x.numpy().astype(self.dtype) - st[:, 0, None, None, None]) * st[:, 1, None, None, None] * self.gamma + self.beta
        y.copy_(torch.from_numpy(out).to(y.dtype))
        return y

    # ---- training pieces (forward and backward on the padded slab), all through the oracle
    def _t(self, a, like):
        return torch.from_numpy(np.ascontiguousarray(a)).to(like.dtype)

    def train_step(self, xp):
        out = orc.step_forward(self.w, self.b, self.s, xp.numpy().astype(self.dtype), self.inner, 8, 1e-5, False, self.act)
        return self._t(out, xp)

    def train_step_backward(self, xp, gyp):
        gw, gb, gs, gx = orc.step_backward(self.w, self.b, self.s, xp.numpy().astype(self.dtype),
                                           gyp.numpy().astype(self.dtype), self.inner, 8, 1e-5, False, self.act)
        return tuple(self._t(a, xp) for a in (gw, gb, gs, gx))

    def ln_local_sums(self, sp):
        v = sp.numpy().astype(np.float64).reshape(sp.shape[0], -1)
        return torch.from_numpy(np.stack([v.sum(1), (v * v).sum(1)], 1))

    def ln_backward_sums(self, sp, gp, stats):
        st = stats.numpy().astype(np.float64)
        xh = (sp.numpy().astype(np.float64) - st[:, 0, None, None, None]) * st[:, 1, None, None, None]
        gg = gp.numpy().astype(np.float64) * self.gamma
        B = sp.shape[0]
        return torch.from_numpy(np.stack([gg.reshape(B, -1).sum(1), (gg * xh).reshape(B, -1).sum(1)], 1))

    def ln_backward_apply(self, sp, gp, stats, sums, count):
        st = stats.numpy().astype(np.float64)
        ac = sums.numpy().astype(np.float64) / count
        xh = (sp.numpy().astype(np.float64) - st[:, 0, None, None, None]) * st[:, 1, None, None, None]
        g = gp.numpy().astype(np.float64)
        gx = st[:, 1, None, None, None] * (g * self.gamma - ac[:, 0, None, None, None] - xh * ac[:, 1, None, None, None])
        return self._t(gx, sp), self._t((g * xh).sum(0), sp), self._t(g.sum(0), sp)
