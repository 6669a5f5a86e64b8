"""The model classes of the reference's training scripts, rebuilt on this package's modules: their
state-dict layout must equal the reference's (so its checkpoints load unchanged), and their logits must
match the reference's own CPU run (tests/golden/script_models.json, made by
tests/golden/make_script_model_fixtures.py) for the same seeded parameters and inputs."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import ROOT
from util import SCRIPT_MODEL_CONFIGS, fill_state_dict, script_model_inputs

with open(os.path.join(ROOT, "tests", "golden", "script_models.json")) as f:
    GOLDEN = json.load(f)


def build(name, device):
    from gridnet_b200.script_models import ImageNetModel, MnistModel

    kind, kwargs = SCRIPT_MODEL_CONFIGS[name]
    return kind, (MnistModel if kind == "mnist" else ImageNetModel)(device=torch.device(device), **kwargs)


@pytest.mark.parametrize("name", sorted(SCRIPT_MODEL_CONFIGS))
def test_state_dict_layout_equals_the_reference(name):
    _, model = build(name, "cpu")
    ours = {k: list(v.shape) for k, v in model.state_dict().items()}
    assert ours == GOLDEN[name]["state_dict"]
    # a checkpoint written by the reference therefore loads strictly
    fake = {k: torch.zeros(shape) for k, shape in GOLDEN[name]["state_dict"].items()}
    model.load_state_dict(fake, strict=True)


def test_no_silent_cpu_path():
    _, model = build("mnist", "cpu")
    with pytest.raises(RuntimeError, match="only runs on CUDA"):
        model(script_model_inputs("mnist", 8))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SCRIPT_MODEL_CONFIGS))
def test_logits_match_the_reference_run(name):
    kind, model = build(name, "cuda")
    fill_state_dict(model, seed=7)
    x = script_model_inputs(kind, seed=8).cuda()
    want = np.asarray(GOLDEN[name]["logits"])
    with torch.no_grad():
        got = model(x).double().cpu().numpy()  # fused loop where the variant allows it
    tol = 2e-4 * np.abs(want).max() + 1e-4
    assert np.abs(got - want).max() < tol, (np.abs(got - want).max(), tol)
    # the autograd path gives the same logits and finite gradients for every parameter
    out = model(x)
    assert np.abs(out.detach().double().cpu().numpy() - want).max() < tol
    grads = torch.autograd.grad(out.square().mean(), list(model.parameters()))
    assert all(bool(torch.isfinite(g).all()) for g in grads)
    assert any(float(g.abs().max()) > 0 for g in grads)
