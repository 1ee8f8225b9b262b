"""Device plans built from the reference's program text alone (no Python loss is traced): value and gradients
against the CPU oracle."""

import numpy as np
import pytest

from oracle import contracted
from quabla_b200._plan import Plan
from quabla_b200._plantext import plan_spec_from_text

from _util import TOLERANCE, relative_error
from test_plan_text_cpu import loss_text

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,points", [("poisson1d", 128), ("poisson2d", 64), ("burgers", 32), ("heat3d", 16),
                                         ("beam", 48)])
def test_a_plan_from_text_matches_the_oracle(cuda_device, name, points):
    text, constants, parameter_names, inputs, value, grads, w = loss_text(name, points)
    spec, parameters, data = plan_spec_from_text(text, parameter_names, constants=constants)
    expected_value, expected_grads = contracted.value_and_grad(spec, inputs)
    plan = Plan(spec, 0)
    for key, array in inputs.items():
        plan.bind(key, array)
    plan.execute()
    outputs = plan.outputs()
    tolerance = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(outputs[0], expected_value) <= tolerance
    assert relative_error(outputs[0], value) <= max(tolerance, 3e-6 if w.dtype == np.float32 else 0.0)
    for got, expected, (pname, _, _) in zip(outputs[1:], expected_grads, spec.parameters):
        assert relative_error(got.reshape(expected.shape), expected) <= tolerance, pname
    plan.close()
