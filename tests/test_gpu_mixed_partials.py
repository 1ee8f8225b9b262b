"""Mixed partial derivatives on the device: the rewritten losses of tests/test_mixed_partials_cpu.py
against the CPU oracle, on whichever engine the plan picks and on the layer-wise engine."""

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted
from quabla_b200._transforms import CompiledLoss

from _util import TOLERANCE, relative_error
from test_mixed_partials_cpu import CASES, problem

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("engine", ["default", "layerwise"])
@pytest.mark.parametrize("dtype,width", [(np.float64, 16), (np.float32, 64)])
@pytest.mark.parametrize("make_loss", CASES)
def test_mixed_partials_match_the_oracle(cuda_device, monkeypatch, make_loss, dtype, width, engine):
    if engine == "layerwise":
        monkeypatch.setenv("QB200_ENGINE", "layerwise")
    params, p = problem(dtype, points=700, width=width)
    args = (params, p)
    compiled = CompiledLoss(make_loss(qb), args, (0,), 0, build_plan=False)
    expected_value, expected_grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args))
    value, grads = qb.jit(qb.value_and_grad(make_loss(qb)), device="cuda:0")(*args)
    tol = TOLERANCE[np.dtype(dtype)]
    assert relative_error(value, expected_value) <= tol
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (name, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert relative_error(got[name].reshape(expected.shape), expected) <= tol, name
