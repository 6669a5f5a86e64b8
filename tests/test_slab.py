"""Slab sharding along K (gridnet_b200/slab.py): R ranks must reproduce the single-device
model loop. CPU: the orchestration under gloo (world size 2) and emulated (world 4) with the
oracle doing the local arithmetic. GPU: the CUDA backend, ranks emulated on one device."""
import os
import tempfile

import numpy as np
import pytest
import torch

from oracle import gridnet_oracle as orc

from gridnet_b200.slab import (SlabLayout, SlabRunner, SlabTrainer, run_distributed, run_emulated, train_distributed,
                               train_emulated)
from slab_checker_backend import OracleSlabBackend


def problem(seed, B, shape):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    w = rn(27, *shape) / 27 ** 0.5
    b = 0.1 * rn(*shape)
    s = 1 + 0.1 * rn(*shape)
    gamma = 1 + 0.1 * rn(*shape)
    beta = 0.1 * rn(*shape)
    x = torch.zeros(B, *shape, dtype=torch.float64)
    x[..., 0] = rn(B, *shape[:2])
    x[..., shape[2] // 2] = 0.5 * rn(B, *shape[:2])  # something on an interior slab boundary too
    return w, b, s, gamma, beta, x


def oracle_runner(layout, prob, inner):
    w, b, s, gamma, beta, x = prob
    sh = layout.shard
    be = OracleSlabBackend(layout, sh(w, False), sh(b, False), sh(s, False), sh(gamma, True), sh(beta, True), inner)
    return SlabRunner(layout, be, sh(x, True), b.numel())


def test_layout_shard_and_faces():
    full = torch.arange(2 * 3 * 32, dtype=torch.float32).reshape(2, 3, 32)
    for world in (1, 2, 4):
        parts = []
        for r in range(world):
            lay = SlabLayout(32, world, r)
            p = lay.shard(full)
            assert p.shape[-1] == lay.k_loc + 16
            parts.append(lay.real(p))
            if lay.left is not None:
                assert torch.equal(p[..., 7], full[..., lay.k0 - 1])
            else:
                assert (p[..., :8] == 0).all()
            if lay.right is not None:
                assert torch.equal(p[..., 8 + lay.k_loc], full[..., lay.k0 + lay.k_loc])
            assert torch.equal(lay.face_to_left(p), full[..., lay.k0])
            assert torch.equal(lay.face_to_right(p), full[..., lay.k0 + lay.k_loc - 1])
        assert torch.equal(torch.cat(parts, -1), full)
    with pytest.raises(AssertionError):
        SlabLayout(24, 2, 0)  # slabs must be whole blocks


@pytest.mark.parametrize("world", [1, 2, 4])
def test_emulated_ranks_match_single_grid_oracle(world):
    shape, B, inner, outer = (8, 8, 32), 2, 2, 3
    prob = problem(30, B, shape)
    want = orc.outer_forward(*(t.numpy() for t in prob), inner, outer, 8)
    runners = [oracle_runner(SlabLayout(shape[2], world, r), prob, inner) for r in range(world)]
    got = torch.cat(run_emulated(runners, outer), -1).numpy()
    assert np.abs(got - want).max() < 1e-10 * (1 + np.abs(want).max())


def _gloo_worker(rank, world, port, tmpdir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shape, B, inner, outer = (8, 8, 32), 2, 2, 3
        runner = oracle_runner(SlabLayout(shape[2], world, rank), problem(31, B, shape), inner)
        out = run_distributed(runner, outer)
        np.save(os.path.join(tmpdir, f"out{rank}.npy"), out.numpy())
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_single_grid_oracle():
    import torch.multiprocessing as mp

    world = 2
    port = 29600 + os.getpid() % 300
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_gloo_worker, args=(world, port, tmp), nprocs=world, join=True)
        got = np.concatenate([np.load(os.path.join(tmp, f"out{r}.npy")) for r in range(world)], -1)
    shape, B, inner, outer = (8, 8, 32), 2, 2, 3
    want = orc.outer_forward(*(t.numpy() for t in problem(31, B, shape)), inner, outer, 8)
    assert np.abs(got - want).max() < 1e-10 * (1 + np.abs(want).max())


# ---- training: forward + backward with the reverse face exchange --------------------------------------------------
def oracle_trainer(layout, prob, inner):
    w, b, s, gamma, beta, x = prob
    sh = lambda t: layout.shard(t, False)
    be = OracleSlabBackend(layout, sh(w), sh(b), sh(s), sh(gamma), sh(beta), inner)
    return SlabTrainer(layout, be, sh(x), b.numel())


def upstream(seed, B, shape):
    return torch.randn(B, *shape, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)


def check_training_result(world, shape, outs, results, prob, gy, inner, outer, tol):
    """R-rank output and gradients (concatenated along K) against the single-grid oracle chain."""
    want_y = orc.outer_forward(*(t.numpy() for t in prob), inner, outer, 8)
    want = orc.outer_backward(*(t.numpy() for t in prob), gy.numpy(), inner, outer, 8)
    got_y = np.concatenate([np.asarray(o, dtype=np.float64) for o in outs], -1)
    assert np.abs(got_y - want_y).max() <= tol * (1 + np.abs(want_y).max())
    for i, name in enumerate(("weight", "bias", "scale", "gamma", "beta", "input")):
        got = np.concatenate([np.asarray(r[i], dtype=np.float64) for r in results], -1)
        assert got.shape == want[i].shape, name
        assert np.abs(got - want[i]).max() <= tol * (1 + np.abs(want[i]).max()), (name, np.abs(got - want[i]).max())


@pytest.mark.parametrize("world", [1, 2, 4])
def test_emulated_training_ranks_match_single_grid_oracle(world):
    shape, B, inner, outer = (8, 8, 32), 2, 2, 3
    prob = problem(40, B, shape)
    gy = upstream(41, B, shape)
    lays = [SlabLayout(shape[2], world, r) for r in range(world)]
    trainers = [oracle_trainer(l, prob, inner) for l in lays]
    outs, results = train_emulated(trainers, outer, lambda r, out: gy[..., lays[r].k0:lays[r].k0 + lays[r].k_loc])
    check_training_result(world, shape, [o.numpy() for o in outs], [[t.numpy() for t in r] for r in results], prob, gy,
                          inner, outer, 1e-10)


def _gloo_train_worker(rank, world, port, tmpdir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shape, B, inner, outer = (8, 8, 32), 2, 2, 3
        lay = SlabLayout(shape[2], world, rank)
        gy = upstream(43, B, shape)
        out, res = train_distributed(oracle_trainer(lay, problem(42, B, shape), inner), outer,
                                     lambda o: gy[..., lay.k0:lay.k0 + lay.k_loc])
        np.savez(os.path.join(tmpdir, f"train{rank}.npz"), out=out.numpy(), **{f"g{i}": t.numpy() for i, t in enumerate(res)})
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_train_like_the_single_grid_oracle():
    import torch.multiprocessing as mp

    world = 2
    port = 29900 + os.getpid() % 90
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_gloo_train_worker, args=(world, port, tmp), nprocs=world, join=True)
        zs = [np.load(os.path.join(tmp, f"train{r}.npz")) for r in range(world)]
        outs = [z["out"] for z in zs]
        results = [[z[f"g{i}"] for i in range(6)] for z in zs]
    shape, B, inner, outer = (8, 8, 32), 2, 2, 3
    check_training_result(world, shape, outs, results, problem(42, B, shape), upstream(43, B, shape), inner, outer, 1e-10)


@pytest.mark.gpu
@pytest.mark.parametrize("world,shape", [(2, (16, 16, 32)), (4, (8, 16, 64)), (1, (16, 8, 16))])
def test_cuda_slab_training_matches_single_device(world, shape):
    """The CUDA backend, ranks emulated on one device: output and all six gradients against the float64 oracle
    chain (1e-4 relative / 1e-5 absolute, with the float32 oracle's own noise as the allowance) and against the
    single-device autograd ops of the package."""
    import gridnet_b200 as gb
    from gridnet_b200.slab import make_cuda_trainer
    from util import assert_close

    B, inner, outer = 3, 2, 3
    prob = [t.float() for t in problem(44, B, shape)]
    gy = upstream(45, B, shape).float()
    lays = [SlabLayout(shape[2], world, r) for r in range(world)]
    trainers = [make_cuda_trainer(l, *prob, inner) for l in lays]
    outs, results = train_emulated(trainers, outer, lambda r, out: gy[..., lays[r].k0:lays[r].k0 + lays[r].k_loc].cuda())
    got_y = torch.cat(outs, -1)
    got = [torch.cat([r[i] for r in results], -1) for i in range(6)]
    # single device, autograd through the package's ops
    w, b, s, gamma, beta, x = (t.cuda().requires_grad_(True) for t in prob)
    h = x
    for _ in range(outer):
        h = gb.GridNormOp.apply(gb.GridnetCudaOp.apply(w, b, s, h, inner, 8, 1e-5, False, "silu"), gamma, beta, 1e-5)
    single = torch.autograd.grad(h, (w, b, s, gamma, beta, x), gy.cuda())
    assert torch.allclose(got_y, h.detach(), rtol=1e-5, atol=1e-6)
    for name, a, c in zip(("weight", "bias", "scale", "gamma", "beta", "input"), got, single):
        assert torch.allclose(a, c, rtol=1e-3, atol=1e-4 * (1 + c.abs().max().item())), (name, (a - c).abs().max().item())
    args64 = [t.double().numpy() for t in prob] + [gy.double().numpy()]
    want64 = orc.outer_backward(*args64, inner, outer, 8)
    want32 = orc.outer_backward(*(a.astype(np.float32) for a in args64), inner, outer, 8)
    for name, a, r64, r32 in zip(("weight", "bias", "scale", "gamma", "beta", "input"), got, want64, want32):
        assert_close(a.cpu().numpy(), r64, r32, f"slab training, world {world}: gradient of {name}")


@pytest.mark.gpu
@pytest.mark.parametrize("world,shape", [(2, (16, 16, 32)), (4, (8, 16, 64)), (1, (16, 8, 16))])
def test_cuda_slabs_match_single_device(world, shape):
    import gridnet_b200 as gb
    from gridnet_b200.slab import make_cuda_runner

    B, inner, outer = 3, 2, 4
    prob = [t.float() for t in problem(32, B, shape)]
    w, b, s, gamma, beta, x = prob
    runners = [make_cuda_runner(SlabLayout(shape[2], world, r), w, b, s, gamma, beta, x, inner) for r in range(world)]
    got = torch.cat(run_emulated(runners, outer), -1)
    # the boundary-first / interior-later order of the overlapped driver gives the same bits
    runners2 = [make_cuda_runner(SlabLayout(shape[2], world, r), w, b, s, gamma, beta, x, inner) for r in range(world)]
    assert torch.equal(torch.cat(run_emulated(runners2, outer, split=True), -1), got)
    # faces stored by the step kernel itself into the neighbours' packed buffers, then unpacked: same bits
    from gridnet_b200.slab import run_emulated_direct

    runners3 = [make_cuda_runner(SlabLayout(shape[2], world, r), w, b, s, gamma, beta, x, inner) for r in range(world)]
    assert torch.equal(torch.cat(run_emulated_direct(runners3, outer), -1), got)
    # ... and with the statistics travelling through mailboxes instead of an all-reduce: same bits again
    from gridnet_b200.slab import run_emulated_mailboxes

    runners4 = [make_cuda_runner(SlabLayout(shape[2], world, r), w, b, s, gamma, beta, x, inner) for r in range(world)]
    assert torch.equal(torch.cat(run_emulated_mailboxes(runners4, outer), -1), got)
    # ... and with the faces stored straight into the neighbours' ghost columns (no packed buffers, no unpacking)
    from gridnet_b200.slab import run_emulated_in_place

    runners5 = [make_cuda_runner(SlabLayout(shape[2], world, r), w, b, s, gamma, beta, x, inner) for r in range(world)]
    assert torch.equal(torch.cat(run_emulated_in_place(runners5, outer), -1), got)
    single = gb.outer_forward(*(t.cuda() for t in prob), inner, outer, 8)
    assert torch.allclose(got, single, rtol=1e-5, atol=1e-6), (got - single).abs().max().item()
    want = orc.outer_forward(*(t.double().numpy() for t in prob), inner, outer, 8)
    err = np.abs(got.cpu().numpy() - want)
    assert (err <= 1e-5 + 1e-4 * np.abs(want)).all(), err.max()


@pytest.mark.gpu
def test_publish_finalize_in_one_launch_equals_the_two_kernels():
    """gn_slab_publish_finalize_f32 (publish this rank's sums, wait for all flags, finish the statistics in one
    launch) against gn_slab_publish_sums_f32 + gn_slab_finalize_unpack_f32, with a world of one rank (the only
    world whose waits a single GPU can satisfy from inside one kernel), over several steps of both parities."""
    from gridnet_b200._lib import lib
    from gridnet_b200.slab import make_cuda_runner

    shape, B, inner = (16, 8, 16), 3, 2
    prob = [t.float() for t in problem(41, B, shape)]
    w, b, s, gamma, beta, x = prob
    lay = SlabLayout(shape[2], 1, 0)
    stats = {}
    for tag in ("two kernels", "one kernel"):
        r = make_cuda_runner(lay, w, b, s, gamma, beta, x, inner)
        box = torch.zeros((int(lib.gn_slab_mailbox_bytes(1, B)) + 7) // 8, dtype=torch.int64, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = []
        for step in (1, 2, 3):
            r.compute_direct_no_sums(0, 0)
            if tag == "one kernel":
                r.stats = r.backend.publish_finalize([box.data_ptr()], 0, 1, step, r.grid_size, r.bufs[r.cur], flag)
            else:
                r.backend.publish_sums([box.data_ptr()], 0, 1, step)
                r.stats = r.backend.finalize_unpack(box, 1, step, r.grid_size, None, None, r.bufs[r.cur], flag)
            got.append(r.stats.clone())
        assert not bool(flag.item())
        stats[tag] = (got, r.result())
    for a, c in zip(stats["two kernels"][0], stats["one kernel"][0]):
        assert torch.equal(a, c)
    assert torch.equal(stats["two kernels"][1], stats["one kernel"][1])
