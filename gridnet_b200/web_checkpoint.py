"""The checkpoint format of the reference's browser demo: writer and reader.

Layout (gridnet/scripts/convert_to_web.py:33-71, read back by web/ts/checkpoint.ts:28-99): a little-endian
``uint32`` with the length of a JSON header, the header ``{"params": [[name, shape], ...], "precision": 32 | 16,
"config": {"activation", "innerIters", "outerIters", "outerResidual"}}``, then every parameter's values flattened in
header order, as little-endian float32 or as the reference's own 16-bit encoding: sign, five exponent bits with bias
15 and the top ten fraction bits of the float32 value, truncated (no rounding); exponents below -15 are clamped to
-15, which turns small values into small denormal-looking codes exactly as the reference's writer does.

This sits beside the hot path (checkpoint interop); it involves no GPU work.
"""
from __future__ import annotations

import json
import struct
from collections import OrderedDict

import numpy as np


def _to_f32_array(v) -> np.ndarray:
    if hasattr(v, "detach"):
        v = v.detach().cpu().float().numpy()
    return np.ascontiguousarray(np.asarray(v, dtype=np.float32)).reshape(-1)


def _encode_f16_truncated(values: np.ndarray) -> np.ndarray:
    bits = values.astype("<f4").view("<u4").astype(np.int64)
    sign = (bits >> 31) & 1
    exp = ((bits >> 23) & 0xFF) - 127
    frac = bits & ((1 << 23) - 1)
    exp = np.where(exp < -15, -15, exp)
    return ((sign << 15) | (((exp + 15) & 0x1F) << 10) | (frac >> 13)).astype("<u2")


def write_web_checkpoint(state_dict, path: str, *, activation: str = "leaky_relu", inner_iters: int = 8,
                         outer_iters: int = 12, outer_residual: bool = False, precision: int = 32) -> None:
    """Writes ``state_dict`` (name -> tensor / array, in iteration order) in the browser demo's format."""
    if precision not in (16, 32):
        raise ValueError("precision must be 16 or 32")
    params = [(k, list(getattr(v, "shape", np.shape(v)))) for k, v in state_dict.items()]
    header = dict(params=params, precision=precision,
                  config={"activation": activation, "innerIters": inner_iters, "outerIters": outer_iters,
                          "outerResidual": outer_residual})
    blob = json.dumps(header).encode("utf-8")
    with open(path, "wb") as f:
        f.write(struct.pack("<I", len(blob)))
        f.write(blob)
        for v in state_dict.values():
            flat = _to_f32_array(v)
            f.write(flat.astype("<f4").tobytes() if precision == 32 else _encode_f16_truncated(flat).tobytes())


def read_web_checkpoint(path: str):
    """Reads a file written by :func:`write_web_checkpoint` or by the reference's converter; returns
    ``(params, config, precision)`` with ``params`` an ordered name -> float32 array mapping (16-bit values are
    widened the way web/ts/checkpoint.ts:76-99 does: exponent re-biased, fraction shifted back)."""
    with open(path, "rb") as f:
        data = f.read()
    (n,) = struct.unpack_from("<I", data, 0)
    header = json.loads(data[4:4 + n].decode("utf-8"))
    precision = int(header.get("precision", 32))
    body = data[4 + n:]
    if precision == 32:
        flat = np.frombuffer(body, dtype="<f4")
    else:
        half = np.frombuffer(body, dtype="<u2").astype(np.int64)
        sign, exp, frac = (half >> 15) & 1, ((half >> 10) & 0x1F) - 15, half & 0x3FF
        flat = ((sign << 31) | ((exp + 127) << 23) | (frac << 13)).astype("<u4").view("<f4")
    params, pos = OrderedDict(), 0
    for name, shape in header["params"]:
        count = int(np.prod(shape)) if len(shape) else 1
        params[name] = np.array(flat[pos:pos + count], dtype=np.float32).reshape(shape)
        pos += count
    if pos != flat.size:
        raise ValueError(f"{path}: {flat.size - pos} values left over after the listed parameters")
    return params, header["config"], precision
