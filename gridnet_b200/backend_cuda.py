"""Autograd ops with the reference's op surface (gridnet/backend_cuda.py:5-190).

``GridnetCudaOp.apply(weight, bias, residual_scale, init_activations, inner_iters,
block_size, eps, normalize, activation)`` and ``GatedGridnetCudaOp.apply(weight,
bias, init_activations, inner_iters, block_size, activation)`` take the same
arguments, make the same shape/dtype/device assertions (AssertionError), return a
clone for an empty batch and hand back the same gradient tuples as the reference
classes, so ``gridnet/__init__.py:14-18`` can import them in place of the originals.

Added on top of that surface, for the whole-grid normalisation the reference's
models run between steps (gridnet/scripts/train_mnist.py:54,62-64):
``GridNormOp`` (LayerNorm over [M,N,K] per sample, forward and backward) and
``outer_forward`` (the fused inference loop).
"""
from __future__ import annotations

import torch

from . import gridnet_cuda
from ._lib import activation_id, check, lib


def _assert_step_args(weight, bias, residual_scale, init_activations, block_size, gated):
    batch_size, m, n, k = init_activations.shape
    assert m % block_size == 0 and n % block_size == 0 and k % block_size == 0, (
        f"{block_size=} incompatible with {init_activations.shape=}")
    want = (27, 2, m, n, k) if gated else (27, m, n, k)
    assert tuple(weight.shape) == want, f"{weight.shape=} invalid for {init_activations.shape=}"
    assert bias.shape == weight.shape[1:], f"{bias.shape=} invalid for {weight.shape=}"
    others = [("bias", bias), ("init_activations", init_activations)]
    if not gated:
        assert bias.shape == residual_scale.shape, f"{bias.shape=} invalid for {residual_scale.shape=}"
        others.insert(1, ("residual_scale", residual_scale))
    for name, t in others:
        assert weight.dtype == t.dtype, f"mismatching dtypes: {weight.dtype=} {name}.dtype={t.dtype}"
    for name, t in others:
        assert weight.device == t.device, f"mismatching devices: {weight.device=} {name}.device={t.device}"
    return batch_size


_keep_forward_stash = None  # None: decide per call from the free device memory


def keep_forward_stash(enabled):
    """Trade memory for time in training: a :class:`GridnetCudaOp` forward that will be differentiated
    (float32, per-block normalisation off, tuned path) can also keep every inner iteration's pre-activations
    and intermediate activations, ``(2 * inner_iters - 1)`` extra activation tensors per call, so that its
    backward skips recomputing them (about a quarter of the backward time; same gradient bits). The reference
    always recomputes. ``True`` / ``False`` force the choice; ``None`` (the default) keeps them whenever they
    take at most a tenth of the device memory that is free at that moment, and recomputes otherwise, call by
    call; the fused training loop (:class:`FusedLoopTrainOp`) decides once per loop how many of its LAST outer
    steps keep them: as many as fit into 70 % of the free memory. Returns the previous setting."""
    global _keep_forward_stash
    previous, _keep_forward_stash = _keep_forward_stash, (None if enabled is None else bool(enabled))
    return previous


def _stash_wanted(weight, init_activations, inner_iters: int, block_size: int) -> bool:
    if _keep_forward_stash is not None:
        return _keep_forward_stash
    B, M, N, K = init_activations.shape
    need = int(lib.gn_step_stash_bytes(B, M, N, K, int(inner_iters), int(block_size)))
    if need <= 0:
        return False
    dev = weight.device
    free, _ = torch.cuda.mem_get_info(dev)
    # what torch's caching allocator holds but has not handed out counts as free too
    free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
    return need * 10 <= free


def _stash_steps(weight, x, inner_iters: int, block_size: int, steps: int) -> int:
    """How many of the ``steps`` outer steps of a fused training loop keep their inner iterations: all or none when
    :func:`keep_forward_stash` forces it; otherwise as many as fit into 70 % of the device memory that is free when
    the loop starts (a step costs its stash plus the raw output that is saved anyway). Asked once per loop: the
    driver's memory query is not free, and a loop should not change its mind half-way for a few megabytes."""
    if _keep_forward_stash is not None:
        return steps if _keep_forward_stash else 0
    B, M, N, K = x.shape
    need = int(lib.gn_step_stash_bytes(B, M, N, K, int(inner_iters), int(block_size)))
    if need <= 0 or steps <= 0:
        return 0
    dev = weight.device
    free, _ = torch.cuda.mem_get_info(dev)
    free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
    per_step = need + x.numel() * 4
    return max(0, min(steps, int(0.7 * free) // per_step))


class GridnetCudaOp(torch.autograd.Function):
    """One outer-loop step of the plain gridnet (gridnet/backend_cuda.py:5-108)."""

    @staticmethod
    def forward(ctx, weight, bias, residual_scale, init_activations, inner_iters: int, block_size: int,
                eps: float, normalize: bool, activation: str):
        batch_size = _assert_step_args(weight, bias, residual_scale, init_activations, block_size, False)
        if not batch_size:
            return init_activations.clone()
        ctx.save_for_backward(weight, bias, residual_scale, init_activations)
        ctx.cfg = (inner_iters, block_size, eps, normalize, activation)
        ctx.stash = None
        outputs = torch.empty_like(init_activations)
        if (not normalize and weight.dtype == torch.float32 and any(ctx.needs_input_grad[:4])
                and _stash_wanted(weight, init_activations, inner_iters, block_size)):
            ctx.stash = gridnet_cuda.forward_with_stash(weight, bias, residual_scale, init_activations, outputs,
                                                        inner_iters, block_size, activation)
            return outputs
        gridnet_cuda.forward(weight, bias, residual_scale, init_activations, outputs, inner_iters, block_size,
                             eps, normalize, activation)
        return outputs

    @staticmethod
    def backward(ctx, grad_output):
        weight, bias, residual_scale, init_activations = ctx.saved_tensors
        inner_iters, block_size, eps, normalize, activation = ctx.cfg
        # every gradient buffer is written in full by the library: no zero fill
        weight_grad = torch.empty_like(weight)
        bias_grad = torch.empty_like(bias)
        scale_grad = torch.empty_like(residual_scale)
        act_grad = torch.empty_like(init_activations)
        if ctx.stash is not None:
            stash, ctx.stash = ctx.stash, None
            gridnet_cuda.backward_with_stash(weight, bias, residual_scale, init_activations, grad_output.contiguous(),
                                             weight_grad, bias_grad, scale_grad, act_grad, inner_iters, block_size,
                                             activation, stash)
            return weight_grad, bias_grad, scale_grad, act_grad, None, None, None, None, None
        gridnet_cuda.backward(weight, bias, residual_scale, init_activations, grad_output.contiguous(),
                              weight_grad, bias_grad, scale_grad, act_grad, inner_iters, block_size, eps,
                              normalize, activation)
        return weight_grad, bias_grad, scale_grad, act_grad, None, None, None, None, None


class GatedGridnetCudaOp(torch.autograd.Function):
    """One outer-loop step of the gated gridnet (gridnet/backend_cuda.py:111-190)."""

    @staticmethod
    def forward(ctx, weight, bias, init_activations, inner_iters: int, block_size: int, activation: str):
        batch_size = _assert_step_args(weight, bias, None, init_activations, block_size, True)
        if not batch_size:
            return init_activations.clone()
        ctx.save_for_backward(weight, bias, init_activations)
        ctx.cfg = (inner_iters, block_size, activation)
        outputs = torch.empty_like(init_activations)
        gridnet_cuda.forward_gated(weight, bias, init_activations, outputs, inner_iters, block_size, activation)
        return outputs

    @staticmethod
    def backward(ctx, grad_output):
        weight, bias, init_activations = ctx.saved_tensors
        inner_iters, block_size, activation = ctx.cfg
        weight_grad = torch.empty_like(weight)
        bias_grad = torch.empty_like(bias)
        act_grad = torch.empty_like(init_activations)
        gridnet_cuda.backward_gated(weight, bias, init_activations, grad_output.contiguous(), weight_grad,
                                    bias_grad, act_grad, inner_iters, block_size, activation)
        return weight_grad, bias_grad, act_grad, None, None, None


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _require_f32_cuda(**tensors):
    for name, t in tensors.items():
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dtype != torch.float32:
            raise RuntimeError(f"{name} must be float32")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")


class GridNormOp(torch.autograd.Function):
    """``torch.nn.LayerNorm`` over the whole grid of each sample, float32.

    ``GridNormOp.apply(x, gamma, beta, eps)`` with x [B, M, N, K] and gamma, beta
    [M, N, K] equals ``F.layer_norm(x, x.shape[1:], gamma, beta, eps)``.
    """

    @staticmethod
    def forward(ctx, x, gamma, beta, eps: float = 1e-5):
        assert x.shape[1:] == gamma.shape == beta.shape, f"{gamma.shape=} {beta.shape=} invalid for {x.shape=}"
        if not x.shape[0]:
            return x.clone()
        _require_f32_cuda(x=x, gamma=gamma, beta=beta)
        B, P = x.shape[0], x[0].numel()
        y = torch.empty_like(x)
        ws = _workspace(lib.gn_norm_workspace_bytes(B, P), x.device)
        with torch.cuda.device(x.device):
            check(lib.gn_norm_forward_f32(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), None, B,
                                          P, float(eps), ws.data_ptr(), ws.numel(),
                                          torch.cuda.current_stream().cuda_stream))
        ctx.save_for_backward(x, gamma)
        ctx.eps = float(eps)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, gamma = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        B, P = x.shape[0], x[0].numel()
        gx, gg, gb = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
        ws = _workspace(lib.gn_norm_workspace_bytes(B, P), x.device)
        with torch.cuda.device(x.device):
            check(lib.gn_norm_backward_f32(x.data_ptr(), gamma.data_ptr(), grad_y.data_ptr(), gx.data_ptr(),
                                           gg.data_ptr(), gb.data_ptr(), B, P, ctx.eps, ws.data_ptr(), ws.numel(),
                                           torch.cuda.current_stream().cuda_stream))
        return gx, gg, gb, None


class FusedLoopTrainOp(torch.autograd.Function):
    """The model loop of the reference's scripts with gradients:

        h = x
        for _ in range(outer_iters):
            h = layer_norm(gridnet_step(weight, bias, residual_scale, h, ..., normalize=False), norm_weight, norm_bias)

    (gridnet/scripts/train_mnist.py:62-64) as ONE autograd node, float32, shared parameters. The forward pass is the
    fused loop of :func:`outer_forward`: every step kernel reduces the statistics of what it writes and normalises
    its input while loading it, so between steps only the RAW step outputs (and [B, 2] statistics) exist and are
    saved - half the activations that the step-by-step composition saves, and two passes over the grid fewer per
    outer step. The backward pass walks the steps in reverse with the library's LayerNorm backward (reusing the
    saved statistics) and the tuned step backward, whose normalised input is rebuilt from the saved raw tensor.
    With the memory-for-time setting (:func:`keep_forward_stash`) the step kernels also keep their inner
    iterations for the backward, as :class:`GridnetCudaOp` does.

    ``FusedLoopTrainOp.apply(weight, bias, residual_scale, norm_weight, norm_bias, x, inner_iters, outer_iters,
    block_size, activation, ln_eps)``."""

    @staticmethod
    def supported(weight, x, inner_iters: int, block_size: int) -> bool:
        if weight.dtype != torch.float32 or not weight.is_cuda or inner_iters < 1 or x.shape[0] == 0:
            return False
        B, M, N, K = x.shape
        # the tuned forward (needed for the fusion) and the tuned backward both want whole 8^3 regions
        return block_size in (4, 8) and M % 8 == 0 and N % 8 == 0 and K % 8 == 0 and \
            int(lib.gn_step_backward_workspace_bytes(B, M, N, K, int(inner_iters), int(block_size), 0, 4)) > 0

    @staticmethod
    def forward(ctx, weight, bias, residual_scale, norm_weight, norm_bias, x, inner_iters: int, outer_iters: int,
                block_size: int, activation: str, ln_eps: float):
        need_grad = any(ctx.needs_input_grad[:6])
        x = x.contiguous()
        y, raws, stats, stashes = _fused_loop_forward([(weight, bias, residual_scale)] * int(outer_iters), norm_weight,
                                                      norm_bias, x, int(inner_iters), int(block_size), activation,
                                                      float(ln_eps), need_grad)
        ctx.save_for_backward(weight, bias, residual_scale, norm_weight, norm_bias, x, *raws, *stats)
        ctx.stashes = stashes
        ctx.cfg = (int(inner_iters), int(outer_iters), int(block_size), activation, float(ln_eps))
        return y

    @staticmethod
    def backward(ctx, grad_y):
        inner, outer, block, activation, ln_eps = ctx.cfg
        saved = ctx.saved_tensors
        weight, bias, scale, gamma, beta, x = saved[:6]
        raws, stats = saved[6:6 + outer], saved[6 + outer:6 + 2 * outer]
        stashes, ctx.stashes = ctx.stashes, None
        total = []

        def add(k, grads):  # the steps share one parameter set: their gradients are summed as they appear
            if not total:
                total.extend(grads)
            else:
                for acc, g in zip(total, grads):
                    acc += g

        gg, gbt, g = _fused_loop_backward([(weight, bias, scale)] * outer, gamma, beta, x, raws, stats, stashes,
                                          grad_y, inner, block, activation, add)
        if outer == 0:
            z = torch.zeros_like
            return z(weight), z(bias), z(scale), z(gamma), z(beta), g, None, None, None, None, None
        return total[0], total[1], total[2], gg, gbt, g, None, None, None, None, None


class FusedLoopSeparateTrainOp(torch.autograd.Function):
    """:class:`FusedLoopTrainOp` for a loop in which every outer step has its own network
    (``separate_params`` of gridnet/scripts/train_imagenet.py:54-58,76-79): the same fused forward and the same
    reverse walk, each step's parameter gradients going to that step's parameters.

    ``FusedLoopSeparateTrainOp.apply(norm_weight, norm_bias, x, inner_iters, block_size, activation, ln_eps,
    weight_0, bias_0, residual_scale_0, weight_1, ...)``: three tensors per outer step."""

    @staticmethod
    def forward(ctx, norm_weight, norm_bias, x, inner_iters: int, block_size: int, activation: str, ln_eps: float,
                *step_params):
        assert len(step_params) % 3 == 0, "three tensors (weight, bias, residual_scale) per outer step"
        plist = [tuple(step_params[i:i + 3]) for i in range(0, len(step_params), 3)]
        need_grad = any(ctx.needs_input_grad)
        x = x.contiguous()
        y, raws, stats, stashes = _fused_loop_forward(plist, norm_weight, norm_bias, x, int(inner_iters),
                                                      int(block_size), activation, float(ln_eps), need_grad)
        ctx.save_for_backward(norm_weight, norm_bias, x, *step_params, *raws, *stats)
        ctx.stashes = stashes
        ctx.cfg = (int(inner_iters), len(plist), int(block_size), activation)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        inner, outer, block, activation = ctx.cfg
        saved = ctx.saved_tensors
        gamma, beta, x = saved[:3]
        flat = saved[3:3 + 3 * outer]
        plist = [tuple(flat[i:i + 3]) for i in range(0, 3 * outer, 3)]
        raws, stats = saved[3 + 3 * outer:3 + 4 * outer], saved[3 + 4 * outer:3 + 5 * outer]
        stashes, ctx.stashes = ctx.stashes, None
        per_step = [None] * outer

        def keep(k, grads):
            per_step[k] = grads

        gg, gbt, g = _fused_loop_backward(plist, gamma, beta, x, raws, stats, stashes, grad_y, inner, block, activation,
                                          keep)
        if outer == 0:
            return torch.zeros_like(gamma), torch.zeros_like(beta), g, None, None, None, None
        return (gg, gbt, g, None, None, None, None) + tuple(t for grads in per_step for t in grads)


class FusedLoopResidualTrainOp(torch.autograd.Function):
    """The residual form of the model loop with gradients (gridnet/scripts/train_imagenet.py:81-83):

        for net in nets:  n = layer_norm(h);  h = h + (net(n) - n)

    as one autograd node. Forward: the step kernel normalises h while loading it, one pass writes
    ``h + (y - layer_norm(h))`` and reduces the statistics of the result (``gn_norm_residual_combine_f32``); saved
    are the step inputs h_k and their statistics (and the inner iterations of the last steps, memory permitting).
    Backward, per step in reverse: the tuned step backward on the rebuilt ``n``, ``grad_n = grad_step - grad``,
    the library's LayerNorm backward with the saved statistics, ``grad = grad + grad_h``.

    ``FusedLoopResidualTrainOp.apply(norm_weight, norm_bias, x, inner_iters, block_size, activation, ln_eps,
    outer_iters, *params)`` with ``params`` either one (weight, bias, residual_scale) shared by all outer steps or
    ``outer_iters`` of them, one after the other."""

    @staticmethod
    def forward(ctx, norm_weight, norm_bias, x, inner_iters: int, block_size: int, activation: str, ln_eps: float,
                outer_iters: int, *params):
        outer = int(outer_iters)
        assert len(params) in (3, 3 * outer), "one (weight, bias, residual_scale), or one per outer step"
        shared = len(params) == 3 and outer != 1
        plist = [tuple(params[:3])] * outer if len(params) == 3 else [tuple(params[i:i + 3]) for i in range(0, 3 * outer, 3)]
        x = x.contiguous()
        B, M, N, K = x.shape
        P = M * N * K
        act = activation_id(activation)
        dev = x.device
        _require_f32_cuda(norm_weight=norm_weight, norm_bias=norm_bias, x=x)
        need_grad = any(ctx.needs_input_grad)
        inputs, stats, stashes = [], [], []
        with torch.cuda.device(dev):
            st = torch.cuda.current_stream().cuda_stream
            nws = _workspace(lib.gn_norm_workspace_bytes(B, P), dev)
            sums = torch.empty(B, 2, dtype=torch.float64, device=dev)
            mr = torch.empty(B, 2, dtype=torch.float32, device=dev)
            h = x
            if outer:
                check(lib.gn_norm_local_sums_f32(h.data_ptr(), sums.data_ptr(), B, P, nws.data_ptr(), nws.numel(), st))
                check(lib.gn_norm_finalize_f32(sums.data_ptr(), 1, mr.data_ptr(), B, P, float(ln_eps), st))
            keep = _stash_steps(plist[0][0], x, inner_iters, block_size, outer) if need_grad and outer else 0
            y = torch.empty_like(x)
            for k, (weight, bias, residual_scale) in enumerate(plist):
                _assert_step_args(weight, bias, residual_scale, x, block_size, False)
                _require_f32_cuda(weight=weight, bias=bias, residual_scale=residual_scale)
                stash = None
                if need_grad and k >= outer - keep:
                    stash = _staggered_bytes(int(lib.gn_step_stash_bytes(B, M, N, K, int(inner_iters), int(block_size))),
                                             dev, k + 3)
                check(lib.gn_step_forward_train_f32(
                    weight.data_ptr(), bias.data_ptr(), residual_scale.data_ptr(), h.data_ptr(), y.data_ptr(),
                    norm_weight.data_ptr(), norm_bias.data_ptr(), mr.data_ptr(), None, B, M, N, K, int(inner_iters),
                    int(block_size), act, None if stash is None else stash.data_ptr(),
                    0 if stash is None else stash.numel(), st))
                nxt = _staggered_like(x, k) if need_grad else torch.empty_like(x)
                mr_next = torch.empty(B, 2, dtype=torch.float32, device=dev)
                check(lib.gn_norm_residual_combine_f32(h.data_ptr(), y.data_ptr(), norm_weight.data_ptr(),
                                                       norm_bias.data_ptr(), mr.data_ptr(), nxt.data_ptr(),
                                                       mr_next.data_ptr(), B, P, float(ln_eps), nws.data_ptr(),
                                                       nws.numel(), st))
                if need_grad:
                    inputs.append(h)
                    stats.append(mr)
                    stashes.append(stash)
                h, mr = nxt, mr_next
            out = h if outer else x.clone()
        ctx.save_for_backward(norm_weight, norm_bias, *params, *inputs, *stats)
        ctx.stashes = stashes
        ctx.cfg = (int(inner_iters), outer, int(block_size), activation, len(params), shared)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        inner, outer, block, activation, nparams, shared = ctx.cfg
        saved = ctx.saved_tensors
        gamma, beta = saved[:2]
        params = saved[2:2 + nparams]
        plist = [tuple(params[:3])] * outer if nparams == 3 else [tuple(params[i:i + 3]) for i in range(0, 3 * outer, 3)]
        inputs, stats = saved[2 + nparams:2 + nparams + outer], saved[2 + nparams + outer:2 + nparams + 2 * outer]
        stashes, ctx.stashes = list(ctx.stashes), None
        g = grad_out.contiguous()
        if outer == 0:
            return (torch.zeros_like(gamma), torch.zeros_like(beta), g, None, None, None, None, None) + \
                tuple(torch.zeros_like(t) for t in params)
        B, M, N, K = g.shape
        P = M * N * K
        dev = g.device
        per_step = [None] * outer
        total = None
        gg = gbt = None
        with torch.cuda.device(dev):
            st = torch.cuda.current_stream().cuda_stream
            nws = _workspace(lib.gn_norm_workspace_bytes(B, P), dev)
            sums = torch.empty(B, 2, dtype=torch.float64, device=dev)
            for k in reversed(range(outer)):
                weight, bias, scale = plist[k]
                h, mr = inputs[k], stats[k]
                dw, db, ds, gn = (torch.empty_like(t) for t in (weight, bias, scale, h))
                # the step's input n = layer_norm(h): rebuilt by the backward kernels while they load h (block 8),
                # else by a pass here
                if _step_backward_fused_in(weight, bias, scale, h, mr, gamma, beta, g, dw, db, ds, gn, inner, block,
                                           activation, stashes[k]):
                    stashes[k] = None
                else:
                    n = torch.empty_like(h)
                    check(lib.gn_norm_apply_f32(h.data_ptr(), gamma.data_ptr(), beta.data_ptr(), mr.data_ptr(), n.data_ptr(),
                                                B, P, st))
                    if stashes[k] is not None:
                        gridnet_cuda.backward_with_stash(weight, bias, scale, n, g, dw, db, ds, gn, inner, block, activation,
                                                         stashes[k])
                        stashes[k] = None
                    else:
                        gridnet_cuda.backward(weight, bias, scale, n, g, dw, db, ds, gn, inner, block, 1e-5, False, activation)
                    del n
                gn -= g  # h' = h + net(n) - n: n also enters with a minus sign
                gh, dg, dbt = torch.empty_like(h), torch.empty_like(gamma), torch.empty_like(gamma)
                check(lib.gn_norm_backward_local_sums_f32(h.data_ptr(), gamma.data_ptr(), gn.data_ptr(), mr.data_ptr(),
                                                          sums.data_ptr(), B, P, nws.data_ptr(), nws.numel(), st))
                check(lib.gn_norm_backward_apply_f32(h.data_ptr(), gamma.data_ptr(), gn.data_ptr(), mr.data_ptr(),
                                                     sums.data_ptr(), P, gh.data_ptr(), dg.data_ptr(), dbt.data_ptr(), B, P,
                                                     nws.data_ptr(), nws.numel(), st))
                g = g + gh
                if nparams == 3:
                    if total is None:
                        total = [dw, db, ds]
                    else:
                        for acc, t in zip(total, (dw, db, ds)):
                            acc += t
                else:
                    per_step[k] = (dw, db, ds)
                if gg is None:
                    gg, gbt = dg, dbt
                else:
                    gg += dg
                    gbt += dbt
        pgrads = tuple(total) if nparams == 3 else tuple(t for grads in per_step for t in grads)
        return (gg, gbt, g, None, None, None, None, None) + pgrads


_STAGGER = 4352  # bytes: 17 x 256, keeps 16-byte alignment
_STAGGER_FROM = 1 << 30  # only tensors of a GiB and more: measured at 2 GiB (C3); at 128 MiB (C4) it cost 1 %


def _staggered_bytes(nbytes: int, device, k: int) -> torch.Tensor:
    """``nbytes`` of device memory starting ``(k % 7 + 1) * 4352`` bytes into its allocation. The tensors a training
    step streams side by side (input, output, kept iterations) are each an exact power of two in size at the
    benchmark's shapes, so fresh allocations start at the same offset inside every 2 MB page; depending on where
    the driver put the pages, the forward pass of C3 then took anything from 79 to 105 ms. Different offsets make
    the streams fall on different memory channels whatever the placement."""
    if nbytes < _STAGGER_FROM:
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    off = (k % 7 + 1) * _STAGGER
    return torch.empty(nbytes + 8 * _STAGGER, dtype=torch.uint8, device=device)[off:off + nbytes]


def _staggered_like(x: torch.Tensor, k: int) -> torch.Tensor:
    return _staggered_bytes(x.numel() * x.element_size(), x.device, k).view(x.dtype).view(x.shape)


def _fused_loop_forward(plist, norm_weight, norm_bias, x, inner_iters, block_size, activation, ln_eps, need_grad):
    """The fused forward of the model loop with one (weight, bias, residual_scale) per outer step: every step kernel
    normalises its input while loading it and reduces the statistics of what it writes. Returns the normalised
    final grid, the raw step outputs, their (mean, rstd) and the kept inner iterations (or None) per step."""
    B, M, N, K = x.shape
    P = M * N * K
    act = activation_id(activation)
    dev = x.device
    for weight, bias, residual_scale in plist:
        _assert_step_args(weight, bias, residual_scale, x, block_size, False)
        assert norm_weight.shape == bias.shape == norm_bias.shape, f"{norm_weight.shape=} invalid for {bias.shape=}"
        _require_f32_cuda(weight=weight, bias=bias, residual_scale=residual_scale)
    _require_f32_cuda(norm_weight=norm_weight, norm_bias=norm_bias, x=x)
    nparts = int(lib.gn_step_stats_partials(M, N, K, block_size))
    partials = torch.empty(B, nparts, 2, dtype=torch.float64, device=dev)
    raws, stats, stashes = [], [], []
    src, src_stats = x, None
    with torch.cuda.device(dev):
        st = torch.cuda.current_stream().cuda_stream
        # the LAST steps keep their inner iterations: their backward comes first, so their stash is freed first
        keep = _stash_steps(plist[0][0], x, inner_iters, block_size, len(plist)) if need_grad and plist else 0
        for k, (weight, bias, residual_scale) in enumerate(plist):
            dst = _staggered_like(x, k) if need_grad else torch.empty_like(x)
            stash = None
            if need_grad and k >= len(plist) - keep:
                stash = _staggered_bytes(int(lib.gn_step_stash_bytes(B, M, N, K, int(inner_iters), int(block_size))),
                                         dev, k + 3)
            check(lib.gn_step_forward_train_f32(
                weight.data_ptr(), bias.data_ptr(), residual_scale.data_ptr(), src.data_ptr(), dst.data_ptr(),
                norm_weight.data_ptr(), norm_bias.data_ptr(), None if src_stats is None else src_stats.data_ptr(),
                partials.data_ptr(), B, M, N, K, int(inner_iters), int(block_size), act,
                None if stash is None else stash.data_ptr(), 0 if stash is None else stash.numel(), st))
            mr = torch.empty(B, 2, dtype=torch.float32, device=dev)
            check(lib.gn_norm_finalize_f32(partials.data_ptr(), nparts, mr.data_ptr(), B, P, float(ln_eps), st))
            if need_grad:
                raws.append(dst)
                stats.append(mr)
                stashes.append(stash)
            src, src_stats = dst, mr
        y = torch.empty_like(x)
        if plist:
            check(lib.gn_norm_apply_f32(src.data_ptr(), norm_weight.data_ptr(), norm_bias.data_ptr(),
                                        src_stats.data_ptr(), y.data_ptr(), B, P, st))
        else:
            y.copy_(x)
    return y, raws, stats, stashes


def _step_backward_fused_in(weight, bias, scale, x_raw, mean_rstd, gamma, beta, gy, dw, db, ds, gx, inner, block,
                            activation, stash) -> bool:
    """The tuned step backward on an input given as (raw tensor, statistics, norm parameters); False where the
    library has no such path (the caller then normalises first)."""
    from ._lib import GN_ERR_UNSUPPORTED

    if int(block) != 8:
        return False
    B, M, N, K = x_raw.shape
    with torch.cuda.device(x_raw.device):
        if stash is not None:
            need = int(lib.gn_step_backward_stash_workspace_bytes(B, M, N, K, int(inner), int(block)))
        else:
            need = int(lib.gn_step_backward_workspace_bytes(B, M, N, K, int(inner), int(block), 0, 4))
        if need <= 0:
            return False
        ws = torch.empty(need, dtype=torch.uint8, device=x_raw.device)
        rc = lib.gn_step_backward_fused_in_f32(
            weight.data_ptr(), bias.data_ptr(), scale.data_ptr(), x_raw.data_ptr(), mean_rstd.data_ptr(), gamma.data_ptr(),
            beta.data_ptr(), gy.data_ptr(), dw.data_ptr(), db.data_ptr(), ds.data_ptr(), gx.data_ptr(), B, M, N, K,
            int(inner), int(block), activation_id(activation), None if stash is None else stash.data_ptr(),
            0 if stash is None else stash.numel(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    if rc == GN_ERR_UNSUPPORTED:
        return False
    check(rc)
    return True


def _fused_loop_backward(plist, gamma, beta, x, raws, stats, stashes, grad_y, inner, block, activation, sink):
    """The reverse walk over the steps of :func:`_fused_loop_forward`: the library's LayerNorm backward with the
    saved statistics, then the tuned step backward on the step's normalised input rebuilt from the saved raw
    tensor. ``sink(k, (dw, db, ds))`` receives step k's parameter gradients; returns the gradients of the norm
    weight and bias (summed over the steps) and of x."""
    outer = len(plist)
    B, M, N, K = x.shape
    P = M * N * K
    dev = x.device
    g = grad_y.contiguous()
    gg = gbt = None
    stashes = list(stashes)
    with torch.cuda.device(dev):
        st = torch.cuda.current_stream().cuda_stream
        nws = _workspace(lib.gn_norm_workspace_bytes(B, P), dev)
        sums = torch.empty(B, 2, dtype=torch.float64, device=dev)
        for k in reversed(range(outer)):
            weight, bias, scale = plist[k]
            # LayerNorm backward of step k with the statistics saved by the forward pass
            gs_k, dg, dbt = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
            check(lib.gn_norm_backward_local_sums_f32(raws[k].data_ptr(), gamma.data_ptr(), g.data_ptr(),
                                                      stats[k].data_ptr(), sums.data_ptr(), B, P, nws.data_ptr(),
                                                      nws.numel(), st))
            check(lib.gn_norm_backward_apply_f32(raws[k].data_ptr(), gamma.data_ptr(), g.data_ptr(), stats[k].data_ptr(),
                                                 sums.data_ptr(), P, gs_k.data_ptr(), dg.data_ptr(), dbt.data_ptr(), B, P,
                                                 nws.data_ptr(), nws.numel(), st))
            dw, db, ds, gx = (torch.empty_like(t) for t in (weight, bias, scale, x))
            # the step's input: x itself for the first step, else the normalised output of the step before - which
            # the backward kernels rebuild while loading the raw tensor where they can (block 8), else a pass here
            if k > 0 and _step_backward_fused_in(weight, bias, scale, raws[k - 1], stats[k - 1], gamma, beta, gs_k, dw, db,
                                                 ds, gx, inner, block, activation, stashes[k]):
                stashes[k] = None
                sink(k, (dw, db, ds))
                if gg is None:
                    gg, gbt = dg, dbt
                else:
                    gg += dg
                    gbt += dbt
                g = gx
                continue
            if k == 0:
                xin = x
            else:
                xin = torch.empty_like(x)
                check(lib.gn_norm_apply_f32(raws[k - 1].data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                            stats[k - 1].data_ptr(), xin.data_ptr(), B, P, st))
            if stashes[k] is not None:
                gridnet_cuda.backward_with_stash(weight, bias, scale, xin, gs_k, dw, db, ds, gx, inner, block, activation,
                                                 stashes[k])
                stashes[k] = None
            else:
                gridnet_cuda.backward(weight, bias, scale, xin, gs_k, dw, db, ds, gx, inner, block, 1e-5, False,
                                      activation)
            sink(k, (dw, db, ds))
            if gg is None:
                gg, gbt = dg, dbt
            else:
                gg += dg
                gbt += dbt
            g = gx
    return gg, gbt, g


def fused_loop_forward(step_params, norm_weight, norm_bias, x, inner_iters: int, block_size: int,
                       activation: str = "silu", ln_eps: float = 1e-5, outer_residual: bool = False) -> torch.Tensor:
    """The model loop of gridnet/scripts/train_imagenet.py:76-86 without gradients, for the variants that
    :func:`outer_forward` does not take: ``step_params`` is one ``(weight, bias, residual_scale)`` per outer step
    (``separate_params``; repeat one tuple for shared parameters), and with ``outer_residual`` a step is
    ``n = norm(h); h = h + (net(n) - n)`` instead of ``h = norm(net(h))``. Float32, tuned step kernel
    (whole 8^3 regions, block 4 or 8). The normalised tensor is never stored: the step kernel normalises while it
    loads, and either it (plain form) or the combining pass (residual form) reduces the next statistics."""
    x = x.contiguous()
    if not outer_residual:
        with torch.no_grad():
            return _fused_loop_forward(list(step_params), norm_weight, norm_bias, x, int(inner_iters), int(block_size),
                                       activation, float(ln_eps), False)[0]
    B, M, N, K = x.shape
    P = M * N * K
    act = activation_id(activation)
    dev = x.device
    _require_f32_cuda(norm_weight=norm_weight, norm_bias=norm_bias, x=x)
    with torch.cuda.device(dev), torch.no_grad():
        st = torch.cuda.current_stream().cuda_stream
        nws = _workspace(lib.gn_norm_workspace_bytes(B, P), dev)
        sums = torch.empty(B, 2, dtype=torch.float64, device=dev)
        mr = [torch.empty(B, 2, dtype=torch.float32, device=dev) for _ in range(2)]
        h, y = x, torch.empty_like(x)
        out = torch.empty_like(x)
        check(lib.gn_norm_local_sums_f32(h.data_ptr(), sums.data_ptr(), B, P, nws.data_ptr(), nws.numel(), st))
        check(lib.gn_norm_finalize_f32(sums.data_ptr(), 1, mr[0].data_ptr(), B, P, float(ln_eps), st))
        for k, (weight, bias, residual_scale) in enumerate(step_params):
            _assert_step_args(weight, bias, residual_scale, x, block_size, False)
            _require_f32_cuda(weight=weight, bias=bias, residual_scale=residual_scale)
            cur, nxt = mr[k & 1], mr[(k + 1) & 1]
            check(lib.gn_step_forward_train_f32(
                weight.data_ptr(), bias.data_ptr(), residual_scale.data_ptr(), h.data_ptr(), y.data_ptr(),
                norm_weight.data_ptr(), norm_bias.data_ptr(), cur.data_ptr(), None, B, M, N, K, int(inner_iters),
                int(block_size), act, None, 0, st))
            check(lib.gn_norm_residual_combine_f32(h.data_ptr(), y.data_ptr(), norm_weight.data_ptr(),
                                                   norm_bias.data_ptr(), cur.data_ptr(), out.data_ptr(), nxt.data_ptr(),
                                                   B, P, float(ln_eps), nws.data_ptr(), nws.numel(), st))
            h = out  # the combining pass may write over its own h
        return h.clone() if h is x else h


def device_status(clear: bool = True, device=None) -> bool:
    """True if, since the last clear, a kernel on ``device`` gave up a bounded wait on a bulk tile copy and had
    no workspace flag to report it in (the results of that call are invalid). Synchronises the device."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        torch.cuda.synchronize(dev)
        rc = int(lib.gn_device_status(1 if clear else 0))
    if rc < 0:
        check(rc)
    return rc == 1


def outer_forward_failed(workspace: torch.Tensor, batch: int, shape, block_size: int) -> bool:
    """True if the last :func:`outer_forward` that used ``workspace`` recorded a device-side failure
    (a bounded wait on a bulk tile copy that gave up). Synchronises the device."""
    m, n, k = shape
    off = int(lib.gn_outer_forward_error_flag_offset(batch, m, n, k, block_size))
    torch.cuda.synchronize(workspace.device)
    return bool(workspace[off:off + 4].view(torch.int32).item())


def outer_forward_workspace(batch: int, shape, block_size: int, device) -> torch.Tensor:
    """Scratch buffer for :func:`outer_forward`; reusable across calls of the same size."""
    m, n, k = shape
    return _workspace(lib.gn_outer_forward_workspace_bytes(batch, m, n, k, block_size), device)


@torch.no_grad()
def outer_forward(weight, bias, residual_scale, norm_weight, norm_bias, init_activations, inner_iters: int,
                  outer_iters: int, block_size: int, activation: str = "silu", ln_eps: float = 1e-5,
                  out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Inference loop of the reference's models, fused:

        h = init_activations
        for _ in range(outer_iters):
            h = gridnet_step(weight, bias, residual_scale, h, inner_iters, block_size, normalize=False, ...)
            h = layer_norm(h, (M, N, K), norm_weight, norm_bias, ln_eps)

    (gridnet/scripts/train_mnist.py:62-64). float32, no autograd.
    """
    batch_size = _assert_step_args(weight, bias, residual_scale, init_activations, block_size, False)
    assert norm_weight.shape == bias.shape == norm_bias.shape, f"{norm_weight.shape=} invalid for {bias.shape=}"
    if not batch_size:
        return init_activations.clone()
    _require_f32_cuda(weight=weight, bias=bias, residual_scale=residual_scale, norm_weight=norm_weight,
                      norm_bias=norm_bias, init_activations=init_activations)
    B, M, N, K = init_activations.shape
    y = torch.empty_like(init_activations) if out is None else out
    need = lib.gn_outer_forward_workspace_bytes(B, M, N, K, block_size)
    ws = workspace if workspace is not None else _workspace(need, weight.device)
    # A caller-owned workspace keeps the parameters re-ordered for the large-batch kernel between calls. They are
    # rebuilt unless this very workspace tensor was used by the previous call with the same parameter tensors and
    # neither they nor the workspace have been written to through torch since (torch counts in-place writes).
    params = (weight, bias, residual_scale, norm_weight, norm_bias)
    key = (tuple((t.data_ptr(), t._version) for t in params), (B, M, N, K, int(block_size)))
    flags = 0
    if workspace is not None and getattr(ws, "_gn_packed_for", None) == (key, ws._version):
        flags = 1  # GN_OUTER_PARAMS_UNCHANGED
    with torch.cuda.device(weight.device):
        check(lib.gn_outer_forward_flags_f32(weight.data_ptr(), bias.data_ptr(), residual_scale.data_ptr(),
                                             norm_weight.data_ptr(), norm_bias.data_ptr(),
                                             init_activations.data_ptr(), y.data_ptr(), B, M, N, K, int(inner_iters),
                                             int(outer_iters), int(block_size), float(ln_eps),
                                             activation_id(activation), ws.data_ptr(), ws.numel(), flags,
                                             torch.cuda.current_stream().cuda_stream))
    if workspace is not None:
        ws._gn_packed_for = (key, ws._version)
    return y


def step_stats_partials(shape, block_size: int) -> int:
    """Number of (sum, sum of squares) pairs per sample that :func:`fused_step` writes."""
    m, n, k = shape
    return int(lib.gn_step_stats_partials(m, n, k, block_size))


@torch.no_grad()
def fused_step(weight, bias, residual_scale, x, out, inner_iters: int, block_size: int, activation: str = "silu",
               norm_weight=None, norm_bias=None, in_mean_rstd=None, out_partials=None) -> torch.Tensor:
    """One step of the fused loop (``gn_step_forward_fused_f32``): ``x`` may be the raw
    output of the previous step, normalised on load with ``in_mean_rstd`` [B, 2] and
    ``norm_weight`` / ``norm_bias``; ``out_partials`` [B, nparts, 2] float64 receives the
    statistics partials of ``out``. Block size 8, float32."""
    _require_f32_cuda(weight=weight, bias=bias, residual_scale=residual_scale, x=x, out=out)
    B, M, N, K = x.shape
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(weight.device):
        check(lib.gn_step_forward_fused_f32(weight.data_ptr(), bias.data_ptr(), residual_scale.data_ptr(),
                                            x.data_ptr(), out.data_ptr(), ptr(norm_weight), ptr(norm_bias),
                                            ptr(in_mean_rstd), ptr(out_partials), B, M, N, K, int(inner_iters),
                                            int(block_size), activation_id(activation),
                                            torch.cuda.current_stream().cuda_stream))
    return out


@torch.no_grad()
def norm_finalize(partials, mean_rstd, P: int, eps: float = 1e-5) -> torch.Tensor:
    """[B, nparts, 2] float64 partial sums -> [B, 2] float32 (mean, 1/sqrt(var + eps))."""
    B, nparts = partials.shape[0], partials.shape[1]
    with torch.cuda.device(partials.device):
        check(lib.gn_norm_finalize_f32(partials.data_ptr(), nparts, mean_rstd.data_ptr(), B, int(P), float(eps),
                                       torch.cuda.current_stream().cuda_stream))
    return mean_rstd


@torch.no_grad()
def norm_apply(x, norm_weight, norm_bias, mean_rstd, out) -> torch.Tensor:
    """out = (x - mean) * rstd * norm_weight + norm_bias per sample."""
    _require_f32_cuda(x=x, norm_weight=norm_weight, norm_bias=norm_bias, out=out)
    B, P = x.shape[0], x[0].numel()
    with torch.cuda.device(x.device):
        check(lib.gn_norm_apply_f32(x.data_ptr(), norm_weight.data_ptr(), norm_bias.data_ptr(),
                                    mean_rstd.data_ptr(), out.data_ptr(), B, P,
                                    torch.cuda.current_stream().cuda_stream))
    return out


# ---- building blocks of the large-batch step kernel (gn_pair64_* in include/gridnet_b200.h) ----------------
def _il64_groups(batch: int) -> int:
    return (int(batch) + 63) // 64


@torch.no_grad()
def pair64_pack_weights(weight, bias, residual_scale, norm_weight=None, norm_bias=None) -> torch.Tensor:
    """weight [27,M,N,K], bias, residual_scale [M,N,K] (float32, M, N, K multiples of 8) and, if steps are to
    normalise their input on load, the whole-grid norm's weight and bias [M,N,K] -> the parameters in the order
    the large-batch step kernel reads them (one flat float32 tensor)."""
    _require_f32_cuda(weight=weight, bias=bias, residual_scale=residual_scale)
    ptr = lambda t: None if t is None else t.data_ptr()
    M, N, K = bias.shape
    nbytes = int(lib.gn_pair64_packed_weight_bytes(M, N, K))
    if nbytes == 0:
        raise RuntimeError(f"grid {tuple(bias.shape)} is not a multiple of 8 in every dimension")
    packed = torch.empty(nbytes // 4, dtype=torch.float32, device=weight.device)
    with torch.cuda.device(weight.device):
        check(lib.gn_pair64_pack_weights_f32(weight.data_ptr(), bias.data_ptr(), residual_scale.data_ptr(),
                                             ptr(norm_weight), ptr(norm_bias), packed.data_ptr(), M, N, K,
                                             torch.cuda.current_stream().cuda_stream))
    return packed


@torch.no_grad()
def pair64_interleave(x, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [B,M,N,K] -> the same activations interleaved by groups of 64 samples, [ceil(B/64), M, N, K, 64]
    (samples beyond B are zero)."""
    _require_f32_cuda(x=x)
    B, M, N, K = x.shape
    if out is None:
        out = torch.empty(_il64_groups(B), M, N, K, 64, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.gn_pair64_interleave_f32(x.data_ptr(), out.data_ptr(), B, M, N, K,
                                           torch.cuda.current_stream().cuda_stream))
    return out


@torch.no_grad()
def pair64_deinterleave(x_il64, batch: int, shape, mean_rstd=None, norm_weight=None, norm_bias=None,
                        out: torch.Tensor | None = None) -> torch.Tensor:
    """Inverse of :func:`pair64_interleave`; with ``mean_rstd`` the whole-grid normalisation is applied on the
    way: ``(v - mean) * rstd * norm_weight + norm_bias``."""
    _require_f32_cuda(x_il64=x_il64)
    M, N, K = shape
    if out is None:
        out = torch.empty(batch, M, N, K, dtype=torch.float32, device=x_il64.device)
    ptr = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(x_il64.device):
        check(lib.gn_pair64_deinterleave_f32(x_il64.data_ptr(), ptr(mean_rstd), ptr(norm_weight), ptr(norm_bias),
                                             out.data_ptr(), int(batch), M, N, K,
                                             torch.cuda.current_stream().cuda_stream))
    return out


@torch.no_grad()
def pair64_step(packed, x_il64, y_il64, batch: int, shape, inner_iters: int, activation: str = "silu",
                in_mean_rstd=None, out_partials=None, error_flag=None) -> torch.Tensor:
    """One step of the large-batch kernel on interleaved activations (``gn_step_forward_pair64_f32``); the
    optional arguments have the meaning they have in :func:`fused_step`, with ``64 * ceil(B/64)`` rows (the
    norm's weight and bias that ``in_mean_rstd`` goes with are the ones given to :func:`pair64_pack_weights`)."""
    M, N, K = shape
    ptr = lambda t: None if t is None else t.data_ptr()
    nparts = 0 if out_partials is None else int(out_partials.shape[1])
    with torch.cuda.device(x_il64.device):
        check(lib.gn_step_forward_pair64_f32(packed.data_ptr(), x_il64.data_ptr(), y_il64.data_ptr(),
                                             ptr(in_mean_rstd), ptr(out_partials), nparts, int(batch),
                                             M, N, K, int(inner_iters), activation_id(activation), ptr(error_flag),
                                             torch.cuda.current_stream().cuda_stream))
    return y_il64


class HostPipelinedForward:
    """The fused inference loop for batches that live in (pinned) HOST memory.

    ``submit(host_x, host_y)`` queues host->device copy, :func:`outer_forward` and device->host
    copy of one batch on three streams with ``depth`` device buffer sets, so the copies of one
    batch overlap the compute of its neighbours; ``synchronize()`` waits for everything queued.
    A buffer set is busy for copy-in + compute + copy-out, so three sets (the default) are what
    keeps all three stages running at once; with two, a step takes half of that sum.
    ``host_x`` / ``host_y`` are ``[B, M, N, K]`` float32 CPU tensors (pinned for real overlap).
    """

    def __init__(self, weight, bias, residual_scale, norm_weight, norm_bias, batch: int, inner_iters: int,
                 outer_iters: int, block_size: int, activation: str = "silu", ln_eps: float = 1e-5, depth: int = 3):
        self.params = (weight, bias, residual_scale, norm_weight, norm_bias)
        self.cfg = (int(inner_iters), int(outer_iters), int(block_size), activation, float(ln_eps))
        dev = weight.device
        shape = tuple(bias.shape)
        self.device = dev
        self.depth = depth
        self.dx = [torch.empty(batch, *shape, device=dev) for _ in range(depth)]
        self.dy = [torch.empty(batch, *shape, device=dev) for _ in range(depth)]
        self.ws = outer_forward_workspace(batch, shape, block_size, dev)
        self.s_in, self.s_compute, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]
        self.ev_compute = [torch.cuda.Event() for _ in range(depth)]
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.count = 0
        torch.cuda.synchronize(dev)

    def submit(self, host_x: torch.Tensor, host_y: torch.Tensor) -> None:
        j = self.count % self.depth
        reuse = self.count >= self.depth
        self.count += 1
        inner, outer, block, act, eps = self.cfg
        if reuse:  # buffer set j is free once its previous result has left the device
            self.s_in.wait_event(self.ev_out[j])
            self.s_compute.wait_event(self.ev_out[j])
        with torch.cuda.stream(self.s_in):
            self.dx[j].copy_(host_x, non_blocking=True)
            self.ev_in[j].record(self.s_in)
        self.s_compute.wait_event(self.ev_in[j])
        with torch.cuda.stream(self.s_compute):
            outer_forward(*self.params, self.dx[j], inner, outer, block, act, eps, out=self.dy[j], workspace=self.ws)
            self.ev_compute[j].record(self.s_compute)
        self.s_out.wait_event(self.ev_compute[j])
        with torch.cuda.stream(self.s_out):
            host_y.copy_(self.dy[j], non_blocking=True)
            self.ev_out[j].record(self.s_out)

    def join(self, stream=None) -> None:
        """Make ``stream`` (default: the current stream) wait for everything queued so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for ev in self.ev_out[: min(self.count, self.depth)]:
            stream.wait_event(ev)

    def synchronize(self) -> None:
        for s in (self.s_in, self.s_compute, self.s_out):
            s.synchronize()
