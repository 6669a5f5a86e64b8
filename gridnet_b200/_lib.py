"""Loader for the C-ABI library ``libgridnet_b200.so`` (see include/gridnet_b200.h).

There is no fallback: if the shared object is missing or does not load, importing
this module raises ImportError, and every op of the package fails with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_float, c_int, c_longlong, c_size_t, c_ulonglong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgridnet_b200.so")

# name -> (restype, argtypes); must list every symbol include/gridnet_b200.h declares
_P = c_void_p
_geom = [c_int] * 4  # B, M, N, K
SIGNATURES = {
    "gn_status_string": (c_char_p, [c_int]),
    "gn_last_cuda_error": (c_char_p, []),
    "gn_activation_from_name": (c_int, [c_char_p]),
    "gn_version": (c_int, []),
    "gn_config_set": (c_int, [c_char_p, c_int]),
    "gn_step_forward_f32": (c_int, [_P] * 5 + _geom + [c_int, c_int, c_float, c_int, c_int, _P]),
    "gn_step_forward_f64": (c_int, [_P] * 5 + _geom + [c_int, c_int, c_double, c_int, c_int, _P]),
    "gn_step_backward_f32": (c_int, [_P] * 9 + _geom + [c_int, c_int, c_float, c_int, c_int, _P]),
    "gn_step_backward_f64": (c_int, [_P] * 9 + _geom + [c_int, c_int, c_double, c_int, c_int, _P]),
    "gn_step_backward_max_inner": (c_int, [c_int, c_int]),
    "gn_step_backward_workspace_bytes": (c_size_t, [c_int] * 8),
    "gn_step_backward_error_flag_offset": (c_size_t, [c_int] * 5),
    "gn_step_stash_bytes": (c_size_t, [c_int] * 6),
    "gn_step_backward_stash_workspace_bytes": (c_size_t, [c_int] * 6),
    "gn_step_backward_stash_error_flag_offset": (c_size_t, [c_int] * 5),
    "gn_step_forward_stash_f32": (c_int, [_P] * 5 + _geom + [c_int, c_int, c_int, _P, c_size_t, _P]),
    "gn_step_backward_stash_f32": (c_int, [_P] * 9 + _geom + [c_int, c_int, c_int, _P, c_size_t, _P, c_size_t, _P]),
    "gn_step_backward_fused_in_f32": (c_int, [_P] * 12 + _geom + [c_int, c_int, c_int, _P, c_size_t, _P, c_size_t, _P]),
    "gn_step_backward_ws_f32": (c_int, [_P] * 9 + _geom + [c_int, c_int, c_float, c_int, c_int, _P, c_size_t, _P]),
    "gn_gated_forward_f32": (c_int, [_P] * 4 + _geom + [c_int, c_int, c_int, _P]),
    "gn_gated_forward_f64": (c_int, [_P] * 4 + _geom + [c_int, c_int, c_int, _P]),
    "gn_gated_backward_f32": (c_int, [_P] * 7 + _geom + [c_int, c_int, c_int, _P]),
    "gn_gated_backward_f64": (c_int, [_P] * 7 + _geom + [c_int, c_int, c_int, _P]),
    "gn_gated_backward_workspace_bytes": (c_size_t, [c_int] * 7),
    "gn_gated_backward_error_flag_offset": (c_size_t, [c_int] * 5),
    "gn_gated_backward_ws_f32": (c_int, [_P] * 7 + _geom + [c_int, c_int, c_int, _P, c_size_t, _P]),
    "gn_norm_workspace_bytes": (c_size_t, [c_int, c_longlong]),
    "gn_norm_forward_f32": (c_int, [_P] * 5 + [c_int, c_longlong, c_float, _P, c_size_t, _P]),
    "gn_norm_backward_f32": (c_int, [_P] * 6 + [c_int, c_longlong, c_float, _P, c_size_t, _P]),
    "gn_norm_residual_combine_f32": (c_int, [_P] * 7 + [c_int, c_longlong, c_float, _P, c_size_t, _P]),
    "gn_norm_local_sums_f32": (c_int, [_P, _P, c_int, c_longlong, _P, c_size_t, _P]),
    "gn_norm_backward_local_sums_f32": (c_int, [_P] * 5 + [c_int, c_longlong, _P, c_size_t, _P]),
    "gn_norm_backward_apply_f32": (c_int, [_P] * 5 + [c_longlong] + [_P] * 3 + [c_int, c_longlong, _P, c_size_t, _P]),
    "gn_norm_static_max_batch": (c_int, []),
    "gn_norm_forward_static_f32": (c_int, [_P] * 4 + [c_int, c_longlong, c_float, _P]),
    "gn_step_stats_partials": (c_int, [c_int] * 4),
    "gn_step_forward_fused_f32": (c_int, [_P] * 9 + _geom + [c_int, c_int, c_int, _P]),
    "gn_device_status": (c_int, [c_int]),
    "gn_device_status_set": (c_int, [c_int]),
    "gn_probe_fp32_fma": (c_int, [_P, c_int, _P, _P]),
    "gn_pair64_supported": (c_int, [c_int] * 5),
    "gn_pair64_stats_partials": (c_int, [c_int] * 3),
    "gn_pair64_packed_weight_bytes": (c_size_t, [c_int] * 3),
    "gn_pair64_pack_weights_f32": (c_int, [_P] * 6 + [c_int] * 3 + [_P]),
    "gn_pair64_interleave_f32": (c_int, [_P] * 2 + _geom + [_P]),
    "gn_pair64_deinterleave_f32": (c_int, [_P] * 5 + _geom + [_P]),
    "gn_step_forward_pair64_f32": (c_int, [_P] * 5 + [c_int] + _geom + [c_int, c_int, _P, _P]),
    "gn_step_forward_train_f32": (c_int, [_P] * 9 + _geom + [c_int, c_int, c_int, _P, c_size_t, _P]),
    "gn_step_forward_slab_f32": (c_int, [_P] * 9 + [c_int] + _geom + [c_int, c_int, c_int, c_int, _P]),
    "gn_step_forward_slab_faces_f32": (c_int, [_P] * 9 + [c_int] + _geom + [c_int, c_int, c_int, c_int, _P, _P, _P]),
    "gn_step_forward_slab_faces_strided_f32": (c_int, [_P] * 9 + [c_int] + _geom + [c_int, c_int, c_int, c_int, _P, _P,
                                                                                   c_longlong, _P]),
    "gn_slab_unpack_faces_f32": (c_int, [_P] * 3 + _geom + [c_int, c_int, _P]),
    "gn_slab_mailbox_bytes": (c_size_t, [c_int, c_int]),
    "gn_slab_publish_sums_f32": (c_int, [_P, c_int, c_int, c_int, c_int, _P, c_int, c_ulonglong, _P]),
    "gn_slab_publish_finalize_f32": (c_int, [_P, c_int, c_int, c_int, c_int, _P, c_int, c_ulonglong, c_longlong, c_float, _P, _P, _P]),
    "gn_slab_finalize_unpack_f32": (c_int, [_P, c_int, c_int, c_int, c_ulonglong, c_longlong, c_float, _P, _P, _P, _P,
                                            c_int, c_int, c_int, c_int, c_int, _P, _P]),
    "gn_norm_finalize_f32": (c_int, [_P, c_int, _P, c_int, c_longlong, c_float, _P]),
    "gn_norm_apply_f32": (c_int, [_P] * 5 + [c_int, c_longlong, _P]),
    "gn_outer_forward_plan": (c_int, [c_int] * 7),
    "gn_outer_forward_workspace_bytes": (c_size_t, [c_int] * 5),
    "gn_outer_forward_error_flag_offset": (c_size_t, [c_int] * 5),
    "gn_outer_forward_f32": (c_int, [_P] * 7 + _geom + [c_int, c_int, c_int, c_float, c_int, _P, c_size_t, _P]),
    "gn_outer_forward_flags_f32": (c_int, [_P] * 7 + _geom + [c_int, c_int, c_int, c_float, c_int, _P, c_size_t, c_int, _P]),
}


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `make -C gridnet_b200/csrc` "
            "(or `python -c 'import __graft_entry__ as g; g.build()'`). "
            "gridnet_b200 has no CPU or PyTorch fallback."
        )
    try:
        lib = ctypes.CDLL(LIB_PATH)
    except OSError as e:  # pragma: no cover - depends on the machine
        raise ImportError(f"could not load {LIB_PATH}: {e}") from e
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class GridnetB200Error(RuntimeError):
    pass


# gn_status values the Python layer looks at (include/gridnet_b200.h)
GN_ERR_CUDA = -7
GN_ERR_UNSUPPORTED = -8


def check(status: int) -> None:
    """Turn a non-zero gn_status into a RuntimeError, like the reference's C++
    exceptions surface in Python (src/gridnet_cuda.cpp:6-10)."""
    if status != 0:
        msg = lib.gn_status_string(status).decode()
        if status == GN_ERR_CUDA:
            msg += ": " + lib.gn_last_cuda_error().decode()
        raise GridnetB200Error(msg)


def activation_id(name: str) -> int:
    aid = lib.gn_activation_from_name(str(name).encode())
    if aid < 0:
        # same wording as src/activations.h:15-16
        raise GridnetB200Error(f"unknown activation function: {name}")
    return aid
