"""The browser demo's checkpoint format (gridnet/scripts/convert_to_web.py:33-71): the writer must produce the bytes
the reference's converter produced for the same state dict (tests/golden/web_checkpoint.npz, made by
tests/golden/make_web_checkpoint_fixture.py), at both precisions, and the reader must take them back."""
import os
from collections import OrderedDict

import numpy as np
import pytest

from conftest import GOLDEN
from gridnet_b200.web_checkpoint import read_web_checkpoint, write_web_checkpoint


def golden():
    z = np.load(os.path.join(GOLDEN, "web_checkpoint.npz"))
    state = OrderedDict((str(k), z["p_" + str(k)]) for k in z["names"])
    return z, state


@pytest.mark.parametrize("precision", [32, 16])
def test_writer_reproduces_the_reference_bytes(tmp_path, precision):
    z, state = golden()
    path = str(tmp_path / "out.bin")
    write_web_checkpoint(state, path, activation="silu", inner_iters=2, outer_iters=3, outer_residual=True,
                         precision=precision)
    assert open(path, "rb").read() == z[f"bytes{precision}"].tobytes()


@pytest.mark.parametrize("precision", [32, 16])
def test_reader_takes_the_reference_file_back(tmp_path, precision):
    z, state = golden()
    path = str(tmp_path / "ref.bin")
    with open(path, "wb") as f:
        f.write(z[f"bytes{precision}"].tobytes())
    params, config, got_precision = read_web_checkpoint(path)
    assert got_precision == precision and list(params) == list(state)
    assert config == {"activation": "silu", "innerIters": 2, "outerIters": 3, "outerResidual": True}
    for k, v in state.items():
        assert params[k].shape == v.shape
        if precision == 32:
            assert np.array_equal(params[k], v)
        else:
            # ten fraction bits, truncated: relative error below 2^-10 for values the format can hold
            big = np.abs(v) >= 2.0 ** -14
            assert np.all(np.abs(params[k][big] - v[big]) <= np.abs(v[big]) * 2.0 ** -10)


def test_torch_state_dict_and_bad_precision(tmp_path):
    import torch

    sd = OrderedDict(a=torch.arange(6, dtype=torch.float64).reshape(2, 3), b=torch.tensor(2.5))
    path = str(tmp_path / "t.bin")
    write_web_checkpoint(sd, path)
    params, config, precision = read_web_checkpoint(path)
    assert precision == 32 and config["activation"] == "leaky_relu" and config["outerResidual"] is False
    assert np.array_equal(params["a"], np.arange(6, dtype=np.float32).reshape(2, 3)) and params["b"].shape == ()
    with pytest.raises(ValueError):
        write_web_checkpoint(sd, path, precision=8)
