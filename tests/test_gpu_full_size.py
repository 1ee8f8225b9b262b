"""The five benchmark configurations at their full sizes.

Where the CPU oracle finishes in seconds on all host threads (2-D Poisson, beam, Burgers) the
device result is compared with it directly; the 3-D heat step (12 TFLOP per pass) is checked
through size-independent properties instead: bitwise repeatability, exact linearity in the loss
cotangent (a power of two scales every gradient bit for bit), and additivity over point shards.
"""

import numpy as np
import pytest

from oracle import contracted
from quabla_b200 import workloads
from quabla_b200._plan import COTANGENT_NAME, Plan
from quabla_b200._transforms import CompiledLoss

from _util import TOLERANCE, relative_error, traced

pytestmark = pytest.mark.gpu


def _run(spec, inputs, cotangent=None):
    plan = Plan(spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    if cotangent is not None:
        plan.bind(COTANGENT_NAME, np.asarray(cotangent, dtype=spec.dtype))
    plan.execute()
    outputs = plan.outputs()
    plan.execute()
    again = plan.outputs()
    plan.close()
    for a, b in zip(outputs, again):
        assert a.tobytes() == b.tobytes(), "two executes of one plan differ"
    return outputs


@pytest.mark.parametrize("name", ["poisson2d", "beam", "burgers"])
def test_full_size_step_matches_the_oracle(cuda_device, name):
    w, compiled, inputs = traced(name, None)
    outputs = _run(compiled.spec, inputs)
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs, threads=contracted.max_threads())
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(outputs[0], expected_loss) <= tol
    for got, expected, (pname, _, _) in zip(outputs[1:], expected_grads, compiled.spec.parameters):
        assert relative_error(got.reshape(expected.shape), expected) <= tol, pname


def test_full_size_heat_step_properties(cuda_device):
    w, compiled, inputs = traced("heat3d", None)
    base = _run(compiled.spec, inputs)
    assert np.isfinite(base[0]) and all(np.all(np.isfinite(g)) for g in base[1:])

    # Linearity in the cotangent: a power of two scales every gradient exactly.
    doubled = _run(compiled.spec, inputs, cotangent=2.0)
    for a, b in zip(base[1:], doubled[1:]):
        assert (2.0 * a).tobytes() == b.tobytes()

    # Additivity over shards: the mean over all points is the mean of the two half-batch means.
    points = w.data[0]
    half = points.shape[0] // 2
    parts = []
    for lo in (0, half):
        wh = workloads.make("heat3d", half)
        args = (w.params, np.ascontiguousarray(points[lo:lo + half]))
        ch = CompiledLoss(wh.loss, args, (0,), 0, build_plan=False)
        parts.append(_run(ch.spec, ch.named_inputs(args)))
    tol = TOLERANCE[np.dtype(np.float32)]
    assert relative_error(0.5 * (np.float64(parts[0][0]) + np.float64(parts[1][0])), np.float64(base[0])) <= tol
    for full, a, b in zip(base[1:], parts[0][1:], parts[1][1:]):
        assert relative_error(0.5 * (a.astype(np.float64) + b.astype(np.float64)), full.astype(np.float64)) <= tol

    # A 1/64 sample of the points against the oracle (the same network, the same kernels and tiling).
    sample = points.shape[0] // 64
    ws = workloads.make("heat3d", sample)
    args = (w.params, np.ascontiguousarray(points[:sample]))
    cs = CompiledLoss(ws.loss, args, (0,), 0, build_plan=False)
    named = cs.named_inputs(args)
    got = _run(cs.spec, named)
    expected_loss, expected_grads = contracted.value_and_grad(cs.spec, named, threads=contracted.max_threads())
    assert relative_error(got[0], expected_loss) <= tol
    for g, e, (pname, _, _) in zip(got[1:], expected_grads, cs.spec.parameters):
        assert relative_error(g.reshape(e.shape), e) <= tol, pname
