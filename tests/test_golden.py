"""Golden vectors (tests/golden, made by the literal oracle) against the
contracted oracle on the CPU and against the device through the C ABI."""

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted
from quabla_b200 import workloads
from quabla_b200._transforms import CompiledLoss

from _util import check_against_golden, load_golden

# float32 fixtures carry the reference's per-node float32 rounding (about 2e-7
# away from exact arithmetic); 1e-5 is the float32 gate of the path.
TOLERANCE = {np.dtype(np.float64): 1e-12, np.dtype(np.float32): 1e-5}


@pytest.mark.parametrize("name", workloads.ORDER)
def test_contracted_oracle_reproduces_the_golden_vectors(name):
    w, fixture = load_golden(name)
    args = (w.params, *w.data)
    compiled = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    loss, grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args))
    named = {p[0]: g for p, g in zip(compiled.spec.parameters, grads)}
    check_against_golden(fixture, loss, named, TOLERANCE[np.dtype(w.dtype)])


@pytest.mark.gpu
@pytest.mark.parametrize("name", workloads.ORDER)
def test_device_reproduces_the_golden_vectors(cuda_device, name):
    w, fixture = load_golden(name)
    value, grads = qb.jit(qb.value_and_grad(w.loss), device="cuda:0")(w.params, *w.data)
    named = {}
    for layer, tree in enumerate(grads):
        named[f"params/{layer}/w"], named[f"params/{layer}/b"] = tree["w"], tree["b"]
    tolerance = 1e-10 if np.dtype(w.dtype) == np.float64 else 1e-5
    check_against_golden(fixture, value, named, tolerance)
