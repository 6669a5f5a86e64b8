"""Generates tests/golden/web_checkpoint.npz: a small state dict and the bytes the REFERENCE's converter
(gridnet/scripts/convert_to_web.py, imported unchanged from the reference tree) writes for it, at 32 and 16 bits.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_web_checkpoint_fixture.py [/root/reference]
"""
import os
import sys
import tempfile
from collections import OrderedDict

import numpy as np
import torch

REFERENCE = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    sys.dont_write_bytecode = True
    sys.path.insert(0, REFERENCE)
    from gridnet.scripts import convert_to_web

    r = np.random.default_rng(7)
    state = OrderedDict()
    state["network.weight"] = torch.from_numpy((r.standard_normal((27, 4, 4, 4)) / 5).astype(np.float32))
    state["network.bias"] = torch.from_numpy((0.1 * r.standard_normal((4, 4, 4))).astype(np.float32))
    # values across the exponent range, including ones below the 16-bit format's smallest exponent and exact zeros
    edge = np.array([0.0, -0.0, 1.0, -1.0, 1e-3, -3e-5, 2e-6, 6.1e-5, 1024.5, -0.333333, 65504.0, 1e-8], np.float32)
    state["norm.weight"] = torch.from_numpy(edge.reshape(3, 4))
    state["readout.bias"] = torch.from_numpy(r.standard_normal(5).astype(np.float32))
    out = {"names": np.array(list(state)), **{"p_" + k: v.numpy() for k, v in state.items()}}
    with tempfile.TemporaryDirectory() as tmp:
        ckpt = os.path.join(tmp, "in.pt")
        torch.save({"model": state, "step": 3}, ckpt)
        for precision in (32, 16):
            dst = os.path.join(tmp, f"out{precision}.bin")
            sys.argv = ["convert_to_web", "--input_path", ckpt, "--output_path", dst, "--activation", "silu",
                        "--inner_iters", "2", "--outer_iters", "3", "--outer_residual", "--precision", str(precision)]
            convert_to_web.main()
            out[f"bytes{precision}"] = np.frombuffer(open(dst, "rb").read(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "web_checkpoint.npz"), **out)
    print("wrote", os.path.join(HERE, "web_checkpoint.npz"))


if __name__ == "__main__":
    main()
