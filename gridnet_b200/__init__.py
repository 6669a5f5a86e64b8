"""gridnet_b200 — B200-native kernels for gridnet's block-local recurrent grid
update, behind the reference's own op surface.

``GridnetCudaOp`` / ``GatedGridnetCudaOp`` are drop-ins for the classes of the same
name in the reference's ``gridnet/backend_cuda.py``; ``gridnet_cuda`` mirrors its
native extension module. Everything runs through ``libgridnet_b200.so`` (C ABI in
``include/gridnet_b200.h``); there is no CPU or PyTorch fallback.
"""
from . import gridnet_cuda
from ._lib import LIB_PATH, GridnetB200Error
from .backend_cuda import (FusedLoopResidualTrainOp, FusedLoopSeparateTrainOp, FusedLoopTrainOp, fused_loop_forward, GatedGridnetCudaOp, GridnetCudaOp, GridNormOp, HostPipelinedForward, device_status, fused_step,
                           keep_forward_stash, norm_apply,
                           norm_finalize, outer_forward, outer_forward_failed, outer_forward_workspace,
                           step_stats_partials)

from .modules import (GatedGridnet, Gridnet, GridnetModel, GridNorm, Readout, gated_gridnet_step,
                      gridnet_step)
from .script_models import ImageNetModel, MnistModel
from .web_checkpoint import read_web_checkpoint, write_web_checkpoint

__all__ = [
    "Gridnet",
    "GatedGridnet",
    "GridNorm",
    "Readout",
    "GridnetModel",
    "MnistModel",
    "ImageNetModel",
    "gridnet_step",
    "gated_gridnet_step",
    "GridnetCudaOp",
    "GatedGridnetCudaOp",
    "GridNormOp",
    "FusedLoopResidualTrainOp",
    "FusedLoopSeparateTrainOp",
    "FusedLoopTrainOp",
    "fused_loop_forward",
    "outer_forward",
    "keep_forward_stash",
    "HostPipelinedForward",
    "outer_forward_workspace",
    "outer_forward_failed",
    "device_status",
    "fused_step",
    "norm_finalize",
    "norm_apply",
    "step_stats_partials",
    "gridnet_cuda",
    "write_web_checkpoint",
    "read_web_checkpoint",
    "GridnetB200Error",
    "LIB_PATH",
]
