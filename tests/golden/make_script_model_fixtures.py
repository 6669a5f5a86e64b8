"""Generates tests/golden/script_models.json from the reference's own model classes
(gridnet/scripts/train_mnist.py, train_imagenet.py) running on CPU through gridnet/backend_torch.py.

    PYTHONPATH=<reference checkout> python tests/golden/make_script_model_fixtures.py

For every configuration the fixture holds the state-dict layout (names and shapes) and the logits for
seeded parameters and inputs; tests/util.py:fill_state_dict and script_model_inputs regenerate both
from the seed, so neither parameters nor images are stored."""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from util import SCRIPT_MODEL_CONFIGS, fill_state_dict, script_model_inputs  # noqa: E402

from gridnet.scripts.train_imagenet import Model as ImageNetModel  # noqa: E402
from gridnet.scripts.train_mnist import Model as MnistModel  # noqa: E402


def main():
    out = {}
    for name, (kind, kwargs) in SCRIPT_MODEL_CONFIGS.items():
        cls = MnistModel if kind == "mnist" else ImageNetModel
        model = cls(device=torch.device("cpu"), **kwargs)
        fill_state_dict(model, seed=7)
        x = script_model_inputs(kind, seed=8)
        with torch.no_grad():
            logits = model(x)
        out[name] = {
            "state_dict": {k: list(v.shape) for k, v in model.state_dict().items()},
            "logits": logits.double().numpy().tolist(),
        }
        print(name, tuple(logits.shape), float(logits.abs().max()))
    with open(os.path.join(HERE, "script_models.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    main()
