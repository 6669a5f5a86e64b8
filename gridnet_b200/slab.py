"""Slab-sharded inference loop: one grid split along K (the last, information-flow axis)
across ranks, one rank per GPU.

The reference is single-GPU; this is the multi-GPU form of its model loop
(gridnet/scripts/train_mnist.py:62-64) for grids too large or too slow for one device.
Every rank owns ``K / world`` consecutive K-columns of the activations and of every
parameter. Per outer step there is exactly one exchange:

* each rank's boundary faces ``[B, M, N]`` go to its two neighbours (send/recv), landing in
  the receiver's OWN memory as ghost columns that the step kernel reads like any halo cell;
* the per-sample (sum, sum of squares) of the step's raw output are all-reduced, because the
  LayerNorm between steps spans the whole grid.

Training (:class:`SlabTrainer`) adds the two exchanges of the backward pass: the all-reduce of the
LayerNorm backward's per-sample sums, and the reverse face exchange in which the gradient found in a
rank's ghost columns goes back to the neighbour that owns those columns.

Local layout: ``[..., 8 + K_loc + 8]`` — one ghost block of 8 columns on each side keeps
block alignment; only ghost column 7 (left) and ``8 + K_loc`` (right) are ever read.

There are two ways to move the faces. :func:`run_distributed` packs them with torch indexing and
sends them with grouped NCCL send/recv. :func:`run_direct` needs neither: the step kernel of a
boundary K-block stores its face straight into a packed buffer in the NEIGHBOUR's memory (mapped
into this process through torch's symmetric memory, :class:`PeerFaceBuffers`), so the transfer rides
inside the compute kernel over NVLink; the all-reduce of the statistics that every step needs anyway
is also the point after which a rank knows its neighbours' kernels - and with them their face
stores - have finished.

The arithmetic is delegated to a backend object so that the orchestration can be exercised
on CPU ranks (gloo) with a checker backend in the tests; :class:`CudaSlabBackend` is the
product backend and calls the C ABI (``gn_step_forward_slab_f32`` and friends).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

GHOST = 8


@dataclass(frozen=True)
class SlabLayout:
    K: int
    world: int
    rank: int

    def __post_init__(self):
        assert self.world >= 1 and 0 <= self.rank < self.world
        assert self.K % (8 * self.world) == 0, f"K={self.K} must be a multiple of 8 * world={8 * self.world}"

    @property
    def k_loc(self) -> int:
        return self.K // self.world

    @property
    def k0(self) -> int:
        return self.rank * self.k_loc

    @property
    def k_pad(self) -> int:
        return self.k_loc + 2 * GHOST

    @property
    def left(self):
        return self.rank - 1 if self.rank > 0 else None

    @property
    def right(self):
        return self.rank + 1 if self.rank + 1 < self.world else None

    def shard(self, full: torch.Tensor, with_ghost_faces: bool = True) -> torch.Tensor:
        """``[..., K]`` -> this rank's padded slab ``[..., k_pad]`` (ghost columns zero, or the
        neighbours' adjacent columns when ``with_ghost_faces``)."""
        out = full.new_zeros(*full.shape[:-1], self.k_pad)
        out[..., GHOST:GHOST + self.k_loc] = full[..., self.k0:self.k0 + self.k_loc]
        if with_ghost_faces:
            if self.k0 > 0:
                out[..., GHOST - 1] = full[..., self.k0 - 1]
            if self.k0 + self.k_loc < self.K:
                out[..., GHOST + self.k_loc] = full[..., self.k0 + self.k_loc]
        return out.contiguous()

    def real(self, padded: torch.Tensor) -> torch.Tensor:
        return padded[..., GHOST:GHOST + self.k_loc]

    # boundary faces of a padded slab (contiguous copies, ready to send)
    def face_to_left(self, padded):
        return padded[..., GHOST].contiguous()

    def face_to_right(self, padded):
        return padded[..., GHOST + self.k_loc - 1].contiguous()

    def put_from_left(self, padded, face):
        padded[..., GHOST - 1] = face

    def put_from_right(self, padded, face):
        padded[..., GHOST + self.k_loc] = face

    def zero_ghosts(self, padded):
        """Clears both ghost blocks in place (the real columns are untouched)."""
        padded[..., :GHOST] = 0
        padded[..., GHOST + self.k_loc:] = 0
        return padded


class CudaSlabBackend:
    """Runs the local arithmetic of one rank through the C ABI (float32, block 8, normalize off)."""

    def __init__(self, layout: SlabLayout, weight, bias, scale, gamma, beta, inner: int, activation: str = "silu",
                 ln_eps: float = 1e-5):
        from ._lib import activation_id, check, lib

        self.lib, self.check = lib, check
        self.layout = layout
        for t in (weight, bias, scale, gamma, beta):
            assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.shape[-1] == layout.k_pad
        self.w, self.b, self.s, self.gamma, self.beta = weight, bias, scale, gamma, beta
        self.inner, self.act, self.ln_eps = int(inner), activation_id(activation), float(ln_eps)
        self._act_name = activation
        self.M, self.N = bias.shape[0], bias.shape[1]
        self.nparts = 4 * (self.M // 8) * (self.N // 8) * (layout.k_loc // 8)
        self._partials = None

    def _stream(self):
        return torch.cuda.current_stream().cuda_stream

    def _launch(self, x, y, in_stats, kb_first: int, kb_count: int, pair_offset: int):
        B = x.shape[0]
        if self._partials is None or self._partials.shape[0] != B:
            self._partials = torch.empty(B, self.nparts, 2, dtype=torch.float64, device=x.device)
        self.check(self.lib.gn_step_forward_slab_f32(
            self.w.data_ptr(), self.b.data_ptr(), self.s.data_ptr(), x.data_ptr(), y.data_ptr(),
            self.gamma.data_ptr(), self.beta.data_ptr(), None if in_stats is None else in_stats.data_ptr(),
            self._partials.data_ptr() + 16 * pair_offset, self.nparts, B, self.M, self.N, self.layout.k_pad,
            kb_first, kb_count, self.inner, self.act, self._stream()))

    @property
    def _pairs_per_kblock(self) -> int:
        return 4 * (self.M // 8) * (self.N // 8)

    def step(self, x, y, in_stats):
        """y[real blocks] = step(x) with x normalised on load when ``in_stats`` is given; returns the
        local per-sample (sum, sum of squares) of what was written, ``[B, 2]`` float64."""
        self._launch(x, y, in_stats, 1, self.layout.k_loc // 8, 0)
        return self.sums()

    def step_with_faces(self, x, y, in_stats, face_to_left: int, face_to_right: int, reduce: bool = True,
                        face_stride: int = 1):
        """:meth:`step` whose boundary K-blocks also store their faces to the two device addresses (0 = no
        neighbour on that side; normally peer memory): packed ``[B, M, N]``, or with ``face_stride`` = the
        neighbour's padded K straight into the ghost column of the buffer it reads next."""
        B = x.shape[0]
        if self._partials is None or self._partials.shape[0] != B:
            self._partials = torch.empty(B, self.nparts, 2, dtype=torch.float64, device=x.device)
        self.check(self.lib.gn_step_forward_slab_faces_strided_f32(
            self.w.data_ptr(), self.b.data_ptr(), self.s.data_ptr(), x.data_ptr(), y.data_ptr(),
            self.gamma.data_ptr(), self.beta.data_ptr(), None if in_stats is None else in_stats.data_ptr(),
            self._partials.data_ptr(), self.nparts, B, self.M, self.N, self.layout.k_pad,
            1, self.layout.k_loc // 8, self.inner, self.act, face_to_left or None, face_to_right or None,
            int(face_stride), self._stream()))
        return self.sums() if reduce else None

    def unpack_faces(self, from_left, from_right, x):
        """Packed faces ``[B, M, N]`` (or None) -> the two ghost columns of the padded slab ``x``."""
        B = x.shape[0]
        self.check(self.lib.gn_slab_unpack_faces_f32(
            None if from_left is None else from_left.data_ptr(), None if from_right is None else from_right.data_ptr(),
            x.data_ptr(), B, self.M, self.N, self.layout.k_pad, GHOST - 1, GHOST + self.layout.k_loc, self._stream()))

    def publish_sums(self, mailbox_ptrs, rank: int, world: int, step: int):
        """Adds up the partials of the last step per sample and stores them, then the step number, into every
        rank's mailbox (``gn_slab_publish_sums_f32``)."""
        import ctypes

        B = self._partials.shape[0]
        arr = (ctypes.c_void_p * world)(*mailbox_ptrs)
        self.check(self.lib.gn_slab_publish_sums_f32(self._partials.data_ptr(), self.nparts, B, rank, world, arr, step & 1,
                                                     step, self._stream()))

    def publish_finalize(self, mailbox_ptrs, rank: int, world: int, step: int, count: int, like, error_flag=None):
        """:meth:`publish_sums` and the statistics half of :meth:`finalize_unpack` in one launch
        (``gn_slab_publish_finalize_f32``): for exchanges with nothing to unpack, on one rank per GPU. Returns
        ``[B, 2]`` (mean, rstd)."""
        import ctypes

        B = self._partials.shape[0]
        arr = (ctypes.c_void_p * world)(*mailbox_ptrs)
        stats = torch.empty(B, 2, dtype=torch.float32, device=like.device)
        self.check(self.lib.gn_slab_publish_finalize_f32(
            self._partials.data_ptr(), self.nparts, B, rank, world, arr, step & 1, step, int(count), self.ln_eps,
            stats.data_ptr(), None if error_flag is None else error_flag.data_ptr(), self._stream()))
        return stats

    def finalize_unpack(self, mailbox, world: int, step: int, count: int, from_left, from_right, x, error_flag=None):
        """Waits (bounded) for the step's sums of all ranks, finishes the statistics and moves the faces into the
        ghost columns of ``x`` (``gn_slab_finalize_unpack_f32``); returns ``[B, 2]`` (mean, rstd)."""
        B = x.shape[0]
        stats = torch.empty(B, 2, dtype=torch.float32, device=x.device)
        ptr = lambda t: None if t is None else t.data_ptr()
        self.check(self.lib.gn_slab_finalize_unpack_f32(
            mailbox.data_ptr(), world, B, step & 1, step, int(count), self.ln_eps, stats.data_ptr(), ptr(from_left),
            ptr(from_right), x.data_ptr(), self.M, self.N, self.layout.k_pad, GHOST - 1, GHOST + self.layout.k_loc,
            ptr(error_flag), self._stream()))
        return stats

    # The same step in two parts, so that the faces can travel while the interior computes:
    # the K-blocks that touch a neighbour slab first, the rest afterwards.
    def step_boundary(self, x, y, in_stats):
        n = self.layout.k_loc // 8
        self._launch(x, y, in_stats, 1, 1, 0)
        if n > 1:
            self._launch(x, y, in_stats, n, 1, self._pairs_per_kblock)

    def step_interior(self, x, y, in_stats):
        n = self.layout.k_loc // 8
        if n > 2:
            self._launch(x, y, in_stats, 2, n - 2, 2 * self._pairs_per_kblock)

    def sums(self):
        return self._partials.sum(1)

    def finalize(self, sums, count: int):
        """Global ``[B, 2]`` float64 sums over ``count`` values per sample -> ``[B, 2]`` (mean, rstd)."""
        B = sums.shape[0]
        stats = torch.empty(B, 2, dtype=torch.float32, device=sums.device)
        sums = sums.contiguous()
        self.check(self.lib.gn_norm_finalize_f32(sums.data_ptr(), 1, stats.data_ptr(), B, int(count), self.ln_eps,
                                                 self._stream()))
        return stats

    def apply(self, x, stats, y):
        B, P = x.shape[0], x[0].numel()
        self.check(self.lib.gn_norm_apply_f32(x.data_ptr(), self.gamma.data_ptr(), self.beta.data_ptr(),
                                              stats.data_ptr(), y.data_ptr(), B, P, self._stream()))
        return y


    # ---- training: the step op and the whole-grid norm on the padded slab, forward and backward ----------------
    def _norm_ws(self, B, P):
        n = max(int(self.lib.gn_norm_workspace_bytes(B, P)), 256)
        return torch.empty(n, dtype=torch.uint8, device=self.w.device)

    def train_step(self, xp):
        """One step of the op on the whole padded slab (``gn_step_forward_f32``). The ghost blocks are computed
        too and mean nothing: their weights are zero, and the caller clears them."""
        from . import gridnet_cuda

        yp = torch.empty_like(xp)
        gridnet_cuda.forward(self.w, self.b, self.s, xp, yp, self.inner, 8, 1e-5, False, self._act_name)
        return yp

    def train_step_backward(self, xp, gyp):
        """Backward of :meth:`train_step` for an upstream gradient that is zero in the ghost blocks: parameter
        gradients (zero in the ghost blocks) and the gradient of the padded input, whose two ghost columns next
        to the real ones carry what belongs to the neighbours."""
        from . import gridnet_cuda

        gw, gb, gs, gxp = (torch.empty_like(t) for t in (self.w, self.b, self.s, xp))
        gridnet_cuda.backward(self.w, self.b, self.s, xp, gyp.contiguous(), gw, gb, gs, gxp, self.inner, 8, 1e-5, False,
                              self._act_name)
        return gw, gb, gs, gxp

    def ln_local_sums(self, sp):
        B, P = sp.shape[0], sp[0].numel()
        sums = torch.empty(B, 2, dtype=torch.float64, device=sp.device)
        ws = self._norm_ws(B, P)
        self.check(self.lib.gn_norm_local_sums_f32(sp.data_ptr(), sums.data_ptr(), B, P, ws.data_ptr(), ws.numel(),
                                                   self._stream()))
        return sums

    def ln_backward_sums(self, sp, gp, stats):
        B, P = sp.shape[0], sp[0].numel()
        sums = torch.empty(B, 2, dtype=torch.float64, device=sp.device)
        ws = self._norm_ws(B, P)
        self.check(self.lib.gn_norm_backward_local_sums_f32(sp.data_ptr(), self.gamma.data_ptr(), gp.data_ptr(),
                                                            stats.data_ptr(), sums.data_ptr(), B, P, ws.data_ptr(),
                                                            ws.numel(), self._stream()))
        return sums

    def ln_backward_apply(self, sp, gp, stats, sums, count: int):
        B, P = sp.shape[0], sp[0].numel()
        gsp, gg, gbt = torch.empty_like(sp), torch.empty_like(self.gamma), torch.empty_like(self.gamma)
        ws = self._norm_ws(B, P)
        sums = sums.contiguous()
        self.check(self.lib.gn_norm_backward_apply_f32(sp.data_ptr(), self.gamma.data_ptr(), gp.data_ptr(),
                                                       stats.data_ptr(), sums.data_ptr(), int(count), gsp.data_ptr(),
                                                       gg.data_ptr(), gbt.data_ptr(), B, P, ws.data_ptr(), ws.numel(),
                                                       self._stream()))
        return gsp, gg, gbt


class SlabRunner:
    """State machine of one rank; the communication between its calls is done by a driver
    (:func:`run_distributed` over torch.distributed, or an in-process emulation in tests)."""

    def __init__(self, layout: SlabLayout, backend, x_padded: torch.Tensor, grid_size: int, work_buffers=None):
        self.layout, self.backend = layout, backend
        self.grid_size = int(grid_size)  # M * N * K of the WHOLE grid
        # the two buffers the steps alternate between: the caller's (e.g. peer-mapped, ghost blocks zero), or fresh
        b1, b2 = work_buffers if work_buffers is not None else (torch.zeros_like(x_padded), torch.zeros_like(x_padded))
        self.bufs = [x_padded, b1, b2]
        self.cur = 0          # index of the buffer holding the current (raw) activations
        self.stats = None     # (mean, rstd) of the current buffer when it is a raw step output

    def compute(self):
        """One step on the current buffer; returns the local sums to be all-reduced."""
        nxt = 1 if self.cur != 1 else 2
        sums = self.backend.step(self.bufs[self.cur], self.bufs[nxt], self.stats)
        self.cur = nxt
        return sums

    def compute_direct(self, face_to_left: int, face_to_right: int):
        """One step whose faces the kernel delivers itself; returns the local sums."""
        nxt = 1 if self.cur != 1 else 2
        sums = self.backend.step_with_faces(self.bufs[self.cur], self.bufs[nxt], self.stats, face_to_left, face_to_right)
        self.cur = nxt
        return sums

    def unpack(self, from_left, from_right):
        self.backend.unpack_faces(from_left, from_right, self.bufs[self.cur])

    def next_index(self) -> int:
        """Index (1 or 2) of the buffer the next step writes."""
        return 1 if self.cur != 1 else 2

    def compute_direct_no_sums(self, face_to_left: int, face_to_right: int, face_stride: int = 1):
        """:meth:`compute_direct` that leaves the partials in the backend (for :class:`PeerStatsMailboxes`)."""
        nxt = self.next_index()
        self.backend.step_with_faces(self.bufs[self.cur], self.bufs[nxt], self.stats, face_to_left, face_to_right,
                                     reduce=False, face_stride=face_stride)
        self.cur = nxt

    def can_split(self) -> bool:
        return hasattr(self.backend, "step_boundary")

    def compute_boundary(self):
        """First half of a step: only the K-blocks whose faces the neighbours need."""
        self._nxt = 1 if self.cur != 1 else 2
        self.backend.step_boundary(self.bufs[self.cur], self.bufs[self._nxt], self.stats)

    def compute_interior(self):
        """Second half; returns the local sums of the whole step."""
        self.backend.step_interior(self.bufs[self.cur], self.bufs[self._nxt], self.stats)
        self.cur = self._nxt
        return self.backend.sums()

    def faces_out(self, buf=None):
        b = self.bufs[self.cur if buf is None else buf]
        return self.layout.face_to_left(b), self.layout.face_to_right(b)

    def faces_in(self, from_left, from_right, buf=None):
        b = self.bufs[self.cur if buf is None else buf]
        if from_left is not None:
            self.layout.put_from_left(b, from_left)
        if from_right is not None:
            self.layout.put_from_right(b, from_right)

    def set_global_sums(self, sums):
        self.stats = self.backend.finalize(sums, self.grid_size)

    def result(self):
        """Normalised output of the last step, ``[B, M, N, K_loc]`` (real columns only)."""
        src = self.bufs[self.cur]
        out = torch.empty_like(src)
        self.backend.apply(src, self.stats, out)
        return self.layout.real(out).contiguous()


def _exchange(runner: SlabRunner, group, buf=None):
    """Grouped send/recv of the two boundary faces of ``buf`` into its ghost columns."""
    import torch.distributed as dist

    lay = runner.layout
    to_left, to_right = runner.faces_out(buf)
    from_left = torch.empty_like(to_left) if lay.left is not None else None
    from_right = torch.empty_like(to_right) if lay.right is not None else None
    ops = []
    if lay.left is not None:
        ops += [dist.P2POp(dist.isend, to_left, lay.left, group), dist.P2POp(dist.irecv, from_left, lay.left, group)]
    if lay.right is not None:
        ops += [dist.P2POp(dist.isend, to_right, lay.right, group), dist.P2POp(dist.irecv, from_right, lay.right, group)]
    for r in (dist.batch_isend_irecv(ops) if ops else []):
        r.wait()
    runner.faces_in(from_left, from_right, buf)


def run_distributed(runner: SlabRunner, outer: int, group=None, overlap: bool = False) -> torch.Tensor:
    """Drive one rank's :class:`SlabRunner` for ``outer`` steps over torch.distributed (NCCL on
    GPUs, gloo on CPU): grouped send/recv of the two faces, all-reduce of the sums.

    With ``overlap`` on a CUDA backend that can split a step, the K-blocks next to the neighbours
    are computed first and their faces are packed, exchanged and unpacked on a second stream while
    the interior blocks compute; only the tiny all-reduce of the statistics stays on the critical path.
    It is off by default: with slabs as thin as 256^3 / 8 GPUs the loop is bound by host-side launch
    and torch.distributed call overhead, and the extra launches made it slower (1.05 ms against
    0.78 ms per outer step at that slab size on two B200s)."""
    import torch.distributed as dist

    on_gpu = runner.bufs[0].is_cuda
    if not (overlap and on_gpu and runner.can_split()):
        for _ in range(outer):
            sums = runner.compute()
            _exchange(runner, group)
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
            runner.set_global_sums(sums)
        return runner.result()

    main = torch.cuda.current_stream()
    comm = getattr(runner, "_comm_stream", None)
    if comm is None:
        comm = runner._comm_stream = torch.cuda.Stream()
    for _ in range(outer):
        runner.compute_boundary()
        nxt = runner._nxt
        boundary_done = torch.cuda.Event()
        boundary_done.record(main)
        with torch.cuda.stream(comm):
            comm.wait_event(boundary_done)
            _exchange(runner, group, nxt)
            faces_done = torch.cuda.Event()
            faces_done.record(comm)
        sums = runner.compute_interior()
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        main.wait_event(faces_done)
        runner.set_global_sums(sums)
    return runner.result()


class PeerFaceBuffers:
    """Receive buffers for the faces, two step parities deep, allocated in torch's symmetric memory so that
    the neighbours' kernels can store into them: ``recv[parity][side]`` is ``[B, M, N]`` float32, side 0 =
    the face arriving from the left neighbour, 1 = from the right one. ``target(parity)`` gives the two
    device addresses THIS rank's step kernel stores to: the left neighbour's from-the-right buffer and the
    right neighbour's from-the-left buffer (0 where there is no neighbour).

    Two parities are needed because a neighbour may start its next step (and store the next face) before
    this rank has unpacked the current one; it cannot get two steps ahead, because every step ends with an
    all-reduce that needs this rank's contribution.

    NVLink multicast is switched off for the mapping (plain peer stores only)."""

    def __init__(self, layout: SlabLayout, B: int, M: int, N: int, device, group=None):
        import os

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.layout = layout
        group = group if group is not None else dist.group.WORLD
        self.buf = symm.empty(2, 2, B, M, N, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        face_bytes = B * M * N * 4
        ptrs = self.handle.buffer_ptrs

        def addr(rank, parity, side):
            return int(ptrs[rank]) + (parity * 2 + side) * face_bytes

        self._targets = [
            (addr(layout.left, q, 1) if layout.left is not None else 0,
             addr(layout.right, q, 0) if layout.right is not None else 0)
            for q in (0, 1)
        ]
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def target(self, parity: int):
        return self._targets[parity]

    def received(self, parity: int):
        lay = self.layout
        return (self.buf[parity, 0] if lay.left is not None else None,
                self.buf[parity, 1] if lay.right is not None else None)


class PeerSlabBuffers:
    """The two work buffers of a rank's :class:`SlabRunner` in torch's symmetric memory, so that the neighbours'
    step kernels can store their boundary faces straight into the ghost columns the rank reads in its next step
    (plain peer stores, one float per entry; NVLink multicast switched off). Nothing is unpacked afterwards.
    ``work_buffers()`` goes to the runner; ``targets(nxt)`` are the two addresses for a step that writes buffer
    ``nxt`` (1 or 2), ``stride`` the distance between face entries."""

    def __init__(self, layout: SlabLayout, B: int, M: int, N: int, device, group=None):
        import os

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.layout = layout
        group = group if group is not None else dist.group.WORLD
        self.buf = symm.empty(2, B, M, N, layout.k_pad, dtype=torch.float32, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        self.stride = layout.k_pad
        buf_bytes = B * M * N * layout.k_pad * 4
        ptrs = self.handle.buffer_ptrs

        def addr(rank, nxt, col):
            return int(ptrs[rank]) + (nxt - 1) * buf_bytes + col * 4

        # my first column is the left neighbour's right ghost column, my last one the right neighbour's left one
        self._targets = {
            nxt: (addr(layout.left, nxt, GHOST + layout.k_loc) if layout.left is not None else 0,
                  addr(layout.right, nxt, GHOST - 1) if layout.right is not None else 0)
            for nxt in (1, 2)
        }
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def work_buffers(self):
        return self.buf[0], self.buf[1]

    def targets(self, nxt: int):
        return self._targets[nxt]


class PeerStatsMailboxes:
    """One mailbox per rank for the per-sample statistics of a step, allocated in torch's symmetric memory so that
    every rank can store into every other rank's (plain peer stores; NVLink multicast switched off). With them a
    step of the slab loop needs no collective call at all: see :func:`run_direct`."""

    def __init__(self, layout: SlabLayout, B: int, device, group=None):
        import os

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from ._lib import lib

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = layout.world, layout.rank
        nbytes = int(lib.gn_slab_mailbox_bytes(self.world, B))
        assert nbytes > 0, "at most 16 ranks"
        self.buf = symm.empty((nbytes + 7) // 8, dtype=torch.int64, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0  # outer steps published so far over the life of the mailboxes (flags only ever grow)
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def failed(self) -> bool:
        """True if a wait for the other ranks' sums has run out since the mailboxes were made. Synchronises."""
        return bool(self.error_flag.item())


def run_in_place(runner: SlabRunner, outer: int, slabs: "PeerSlabBuffers", mailboxes: "PeerStatsMailboxes",
                 probe=None) -> torch.Tensor:
    """Drive one rank for ``outer`` steps with the faces stored by the step kernel straight into the neighbours'
    ghost columns (:class:`PeerSlabBuffers`; the runner must have been built on ``slabs.work_buffers()``) and the
    sums exchanged through :class:`PeerStatsMailboxes`: per step the step kernel and one kernel that publishes the
    sums, waits for the other ranks' and finishes the statistics - no unpacking pass, no collective call. A neighbour
    writes a ghost column of the buffer this rank reads NEXT while this rank still writes that buffer's real
    columns; it cannot write again before this rank has published its next sums, i.e. finished reading.
    ``probe(k, i)`` (optional) is called before the two launches of step k (i = 0, 1) and after them (2), e.g. to
    record CUDA events."""
    be, lay = runner.backend, runner.layout
    mark = probe if probe is not None else (lambda k, i: None)
    for k in range(outer):
        mailboxes.step += 1
        step = mailboxes.step
        mark(k, 0)
        runner.compute_direct_no_sums(*slabs.targets(runner.next_index()), face_stride=slabs.stride)
        mark(k, 1)
        runner.stats = be.publish_finalize(mailboxes.ptrs, lay.rank, lay.world, step, runner.grid_size,
                                           runner.bufs[runner.cur], mailboxes.error_flag)
        mark(k, 2)
    return runner.result()


def run_direct(runner: SlabRunner, outer: int, peers: PeerFaceBuffers, group=None,
               mailboxes: "PeerStatsMailboxes | None" = None) -> torch.Tensor:
    """Drive one rank for ``outer`` steps with the faces delivered by the step kernel itself
    (:class:`PeerFaceBuffers`): per step one kernel, the all-reduce of the sums, the finalisation of the
    statistics and the unpacking of the received faces - no pack kernels, no send/recv calls.

    With ``mailboxes`` the all-reduce goes too: the sums travel by peer stores and flags
    (:class:`PeerStatsMailboxes`), so a step is three launches and no collective call; the flag that says "this
    rank's sums have landed" also says "its face stores have landed", since both come from the same stream."""
    import torch.distributed as dist

    if mailboxes is not None:
        be, lay = runner.backend, runner.layout
        for k in range(outer):
            mailboxes.step += 1
            step = mailboxes.step
            q = step & 1
            runner.compute_direct_no_sums(*peers.target(q))
            be.publish_sums(mailboxes.ptrs, lay.rank, lay.world, step)
            from_left, from_right = peers.received(q)
            runner.stats = be.finalize_unpack(mailboxes.buf, lay.world, step, runner.grid_size, from_left, from_right,
                                              runner.bufs[runner.cur], mailboxes.error_flag)
        return runner.result()

    for k in range(outer):
        q = k & 1
        sums = runner.compute_direct(*peers.target(q))
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)  # also: every neighbour's step k has finished
        runner.set_global_sums(sums)
        runner.unpack(*peers.received(q))
    return runner.result()


def run_emulated_direct(runners, outer: int):
    """:func:`run_direct` with all ranks in one process on one GPU: the "peer" buffers are ordinary tensors
    of the other runners, everything else (kernel-side face stores, parity, unpacking) is the same."""
    world = len(runners)
    first = runners[0].bufs[0]
    B, M, N = first.shape[0], first.shape[1], first.shape[2]
    recv = [torch.zeros(2, 2, B, M, N, dtype=torch.float32, device=first.device) for _ in range(world)]
    for k in range(outer):
        q = k & 1
        sums = []
        for i, r in enumerate(runners):
            to_left = recv[i - 1][q, 1].data_ptr() if i > 0 else 0
            to_right = recv[i + 1][q, 0].data_ptr() if i + 1 < world else 0
            sums.append(r.compute_direct(to_left, to_right))
        total = torch.stack(sums).sum(0)
        for i, r in enumerate(runners):
            r.set_global_sums(total.clone())
            r.unpack(recv[i][q, 0] if i > 0 else None, recv[i][q, 1] if i + 1 < world else None)
    return [r.result() for r in runners]


def run_emulated_in_place(runners, outer: int):
    """:func:`run_in_place` with all ranks in one process on one GPU: the neighbours' work buffers are ordinary
    tensors of the other runners; every rank's step and publish kernels are launched before any rank's finalize
    kernel, so the waits find their flags already set."""
    from ._lib import lib

    world = len(runners)
    first = runners[0].bufs[0]
    B, dev = first.shape[0], first.device
    nbytes = int(lib.gn_slab_mailbox_bytes(world, B))
    boxes = [torch.zeros((nbytes + 7) // 8, dtype=torch.int64, device=dev) for _ in range(world)]
    ptrs = [b.data_ptr() for b in boxes]
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    for k in range(outer):
        step = k + 1
        for i, r in enumerate(runners):
            nxt, lay = r.next_index(), r.layout
            to_left = runners[i - 1].bufs[nxt][0, 0, 0, GHOST + lay.k_loc:].data_ptr() if i > 0 else 0
            to_right = runners[i + 1].bufs[nxt][0, 0, 0, GHOST - 1:].data_ptr() if i + 1 < world else 0
            r.compute_direct_no_sums(to_left, to_right, face_stride=lay.k_pad)
            r.backend.publish_sums(ptrs, i, world, step)
        for i, r in enumerate(runners):
            r.stats = r.backend.finalize_unpack(boxes[i], world, step, r.grid_size, None, None, r.bufs[r.cur], flag)
    assert not bool(flag.item()), "a wait for the ranks' sums ran out"
    return [r.result() for r in runners]


def run_emulated_mailboxes(runners, outer: int):
    """:func:`run_direct` with mailboxes, all ranks in one process on one GPU: every rank's step and publish
    kernels are launched before any rank's finalize kernel, so the waits find their flags already set."""
    from ._lib import lib

    world = len(runners)
    first = runners[0].bufs[0]
    B, M, N = first.shape[0], first.shape[1], first.shape[2]
    dev = first.device
    recv = [torch.zeros(2, 2, B, M, N, dtype=torch.float32, device=dev) for _ in range(world)]
    nbytes = int(lib.gn_slab_mailbox_bytes(world, B))
    boxes = [torch.zeros((nbytes + 7) // 8, dtype=torch.int64, device=dev) for _ in range(world)]
    ptrs = [b.data_ptr() for b in boxes]
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    for k in range(outer):
        step = k + 1
        q = step & 1
        for i, r in enumerate(runners):
            to_left = recv[i - 1][q, 1].data_ptr() if i > 0 else 0
            to_right = recv[i + 1][q, 0].data_ptr() if i + 1 < world else 0
            r.compute_direct_no_sums(to_left, to_right)
            r.backend.publish_sums(ptrs, i, world, step)
        for i, r in enumerate(runners):
            r.stats = r.backend.finalize_unpack(boxes[i], world, step, r.grid_size, recv[i][q, 0] if i > 0 else None,
                                                recv[i][q, 1] if i + 1 < world else None, r.bufs[r.cur], flag)
    assert not bool(flag.item()), "a wait for the ranks' sums ran out"
    return [r.result() for r in runners]


def run_emulated(runners, outer: int, split: bool = False):
    """All ranks in one process, taking turns (for single-GPU tests): same data movement as
    :func:`run_distributed`, with tensor copies in place of the collectives. ``split`` uses the
    boundary-first / interior-later order of the overlapped driver."""
    world = len(runners)
    for _ in range(outer):
        if split:
            for r in runners:
                r.compute_boundary()
            faces = [r.faces_out(r._nxt) for r in runners]
            sums = [r.compute_interior() for r in runners]
        else:
            sums = [r.compute() for r in runners]
            faces = [r.faces_out() for r in runners]
        total = torch.stack(sums).sum(0)
        for i, r in enumerate(runners):
            from_left = faces[i - 1][1] if i > 0 else None
            from_right = faces[i + 1][0] if i + 1 < world else None
            r.faces_in(from_left, from_right)
            r.set_global_sums(total.clone())
    return [r.result() for r in runners]


def make_cuda_runner(layout: SlabLayout, weight, bias, scale, gamma, beta, x, inner: int, activation: str = "silu",
                     ln_eps: float = 1e-5, device=None, work_buffers=None) -> SlabRunner:
    """Shard FULL tensors (any device) for this rank and build its runner on ``device``."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    sh = lambda t, ghost: layout.shard(t, ghost).to(device)
    backend = CudaSlabBackend(layout, sh(weight, False), sh(bias, False), sh(scale, False), sh(gamma, True),
                              sh(beta, True), inner, activation, ln_eps)
    M, N, K = bias.shape
    return SlabRunner(layout, backend, sh(x, True), M * N * K, work_buffers=work_buffers)


class SlabTrainer:
    """One rank's part of a TRAINING step of the model loop on a slab-sharded grid: the forward pass of
    ``outer`` x (step, whole-grid LayerNorm) keeping what the backward pass needs, then the backward pass.

    What crosses rank boundaries, per outer step (gridnet/scripts/train_mnist.py:62-64 on one device; the
    single-device semantics of the halo gradient are the tile-gradient scatter of
    src/gridnet_cuda_kernels.cu:424-435):

    * forward: the two boundary faces of the step's input (into the neighbours' ghost columns) and the
      per-sample (sum, sum of squares) of the step's output (all-reduce), as in inference;
    * backward: the all-reduce of the LayerNorm backward's two per-sample sums, and the REVERSE face
      exchange: the gradient that a rank's boundary blocks leave in its ghost columns belongs to the
      neighbour's boundary column, which adds it to its own gradient.

    Parameters and their gradients are local to a rank (no weight all-reduce). Like :class:`SlabRunner` this
    is a state machine; :func:`train_distributed` and :func:`train_emulated` drive it."""

    def __init__(self, layout: SlabLayout, backend, x_padded: torch.Tensor, grid_size: int):
        self.layout, self.backend, self.grid_size = layout, backend, int(grid_size)
        self.h = layout.zero_ghosts(x_padded.clone())   # current activations, padded, ghosts clear until faces arrive
        self.saved = []                                 # per outer step: (step input with faces, step output, stats)
        self._pending = None
        self.grads = None                               # (gw, gb, gs, ggamma, gbeta), padded, summed over the steps
        self.g = None                                   # gradient w.r.t. the current activations, padded, ghosts clear

    # ---- forward
    def faces_out(self):
        return self.layout.face_to_left(self.h), self.layout.face_to_right(self.h)

    def faces_in(self, from_left, from_right):
        if from_left is not None:
            self.layout.put_from_left(self.h, from_left)
        if from_right is not None:
            self.layout.put_from_right(self.h, from_right)

    def forward_step(self):
        """The step on the padded slab; returns the local (sum, sum of squares) of its real output."""
        s = self.layout.zero_ghosts(self.backend.train_step(self.h))
        self._pending = (self.h, s)
        return self.backend.ln_local_sums(s)

    def forward_norm(self, global_sums):
        xin, s = self._pending
        stats = self.backend.finalize(global_sums, self.grid_size)
        self.saved.append((xin, s, stats))
        self.h = self.layout.zero_ghosts(self.backend.apply(s, stats, torch.empty_like(s)))

    def output(self):
        return self.layout.real(self.h).contiguous()

    # ---- backward
    def backward_begin(self, grad_output_real):
        self.g = torch.zeros_like(self.h)
        self.layout.real(self.g).copy_(grad_output_real)
        self.grads = None

    def backward_norm_sums(self):
        _, s, stats = self.saved[-1]
        return self.backend.ln_backward_sums(s, self.g, stats)

    def backward_step(self, global_sums):
        """LayerNorm backward with the global sums, then the step's backward; returns the gradients that landed in
        the two ghost columns (for the left and the right neighbour)."""
        xin, s, stats = self.saved.pop()
        gs_, gg, gbt = self.backend.ln_backward_apply(s, self.g, stats, global_sums, self.grid_size)
        self.layout.zero_ghosts(gs_)
        gw, gb, gsc, gx = self.backend.train_step_backward(xin, gs_)
        new = (gw, gb, gsc, gg, gbt)
        self.grads = new if self.grads is None else tuple(a + b for a, b in zip(self.grads, new))
        lay = self.layout
        to_left = gx[..., GHOST - 1].contiguous() if lay.left is not None else None
        to_right = gx[..., GHOST + lay.k_loc].contiguous() if lay.right is not None else None
        self.g = lay.zero_ghosts(gx)
        return to_left, to_right

    def backward_faces_in(self, from_left, from_right):
        """Adds what the neighbours found in their ghost copies of this rank's boundary columns."""
        lay = self.layout
        if from_left is not None:
            self.g[..., GHOST] += from_left
        if from_right is not None:
            self.g[..., GHOST + lay.k_loc - 1] += from_right

    def result(self):
        """(grad_weight, grad_bias, grad_scale, grad_gamma, grad_beta, grad_input) of the real columns."""
        lay = self.layout
        return tuple(lay.real(t).contiguous() for t in self.grads) + (lay.real(self.g).contiguous(),)


def _swap_with_neighbours(layout: SlabLayout, to_left, to_right, like, group=None):
    """Grouped send/recv: ``to_left`` / ``to_right`` go to the neighbours, returns what they sent this way."""
    import torch.distributed as dist

    from_left = torch.empty_like(like) if layout.left is not None else None
    from_right = torch.empty_like(like) if layout.right is not None else None
    ops = []
    if layout.left is not None:
        ops += [dist.P2POp(dist.isend, to_left, layout.left, group), dist.P2POp(dist.irecv, from_left, layout.left, group)]
    if layout.right is not None:
        ops += [dist.P2POp(dist.isend, to_right, layout.right, group), dist.P2POp(dist.irecv, from_right, layout.right, group)]
    for r in (dist.batch_isend_irecv(ops) if ops else []):
        r.wait()
    return from_left, from_right


def train_distributed(trainer: SlabTrainer, outer: int, grad_output_fn, group=None):
    """Forward and backward of the model loop for one rank over torch.distributed (NCCL on GPUs, gloo on CPU).
    ``grad_output_fn(output_real)`` gives the upstream gradient of this rank's part of the final activations.
    Returns ``(output_real, gradients)`` with the gradients as in :meth:`SlabTrainer.result`."""
    import torch.distributed as dist

    lay = trainer.layout
    for _ in range(outer):
        to_left, to_right = trainer.faces_out()
        trainer.faces_in(*_swap_with_neighbours(lay, to_left, to_right, to_left, group))
        sums = trainer.forward_step()
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        trainer.forward_norm(sums)
    out = trainer.output()
    trainer.backward_begin(grad_output_fn(out))
    for _ in range(outer):
        sums = trainer.backward_norm_sums()
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        to_left, to_right = trainer.backward_step(sums)
        like = to_left if to_left is not None else to_right
        if like is not None:
            trainer.backward_faces_in(*_swap_with_neighbours(lay, to_left, to_right, like, group))
    return out, trainer.result()


def train_emulated(trainers, outer: int, grad_output_fn):
    """:func:`train_distributed` with all ranks in one process, taking turns (tests on one device).
    ``grad_output_fn(rank, output_real)`` gives each rank's upstream gradient."""
    world = len(trainers)
    for _ in range(outer):
        faces = [t.faces_out() for t in trainers]
        for i, t in enumerate(trainers):
            t.faces_in(faces[i - 1][1] if i > 0 else None, faces[i + 1][0] if i + 1 < world else None)
        total = torch.stack([t.forward_step() for t in trainers]).sum(0)
        for t in trainers:
            t.forward_norm(total.clone())
    outs = [t.output() for t in trainers]
    for i, t in enumerate(trainers):
        t.backward_begin(grad_output_fn(i, outs[i]))
    for _ in range(outer):
        total = torch.stack([t.backward_norm_sums() for t in trainers]).sum(0)
        ghost = [t.backward_step(total.clone()) for t in trainers]
        for i, t in enumerate(trainers):
            t.backward_faces_in(ghost[i - 1][1] if i > 0 else None, ghost[i + 1][0] if i + 1 < world else None)
    return outs, [t.result() for t in trainers]


def make_cuda_trainer(layout: SlabLayout, weight, bias, scale, gamma, beta, x, inner: int, activation: str = "silu",
                      ln_eps: float = 1e-5, device=None) -> SlabTrainer:
    """Shard FULL tensors (any device) for this rank and build its trainer on ``device``."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    sh = lambda t: layout.shard(t, False).to(device)
    backend = CudaSlabBackend(layout, sh(weight), sh(bias), sh(scale), sh(gamma), sh(beta), inner, activation, ln_eps)
    M, N, K = bias.shape
    return SlabTrainer(layout, backend, sh(x), M * N * K)
