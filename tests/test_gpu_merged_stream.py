"""The merged second-order stream on the device: every engine and both jet-kernel families against the
CPU oracle (which evaluates one second-order stream per direction), and against the device's own
unmerged path."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted
from quabla_b200 import _lib, workloads
from quabla_b200._plan import Plan
from quabla_b200._transforms import CompiledLoss

from _util import TOLERANCE, relative_error, traced

pytestmark = pytest.mark.gpu


def _custom(sizes, dtype, points, residual, seed=11):
    """A loss mean(residual(u, point)^2) over `points` random points of the unit cube."""
    u = workloads.make_u(qb)
    params = workloads.init_mlp(qb.random.key(seed), sizes, dtype)
    p = np.stack([qb.random.uniform(qb.random.fold_in(qb.random.key(seed), j), (points,), dtype, 0.0, 1.0)
                  for j in range(sizes[0])], axis=1)

    def loss(params, p):
        return qb.mean(qb.vmap(lambda q: residual(lambda s: u(params, s), q))(p) ** 2)

    return loss, params, p


def _check(loss, params, data, engine=None):
    args = (params, data)
    compiled = CompiledLoss(loss, args, (0,), 0, build_plan=False)
    inputs = compiled.named_inputs(args)
    assert any(s.merge_weights is not None for s in compiled.spec.sets)
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    if engine is not None:
        assert plan.query(_lib.Q_ENGINE) in engine
    outputs = plan.outputs()
    plan.close()
    tol = TOLERANCE[np.dtype(compiled.spec.dtype)]
    assert relative_error(outputs[0], expected_loss) <= tol
    for got, expected, (pname, _, _) in zip(outputs[1:], expected_grads, compiled.spec.parameters):
        assert relative_error(got.reshape(expected.shape), expected) <= tol, pname


@pytest.mark.parametrize("dtype,width,engine", [(np.float32, 16, (1,)), (np.float32, 32, (1,)), (np.float32, 64, (2,)),
                                                (np.float64, 16, (0,)), (np.float64, 128, (0,)), (np.float32, 128, (3,))])
def test_weighted_laplacian_on_every_engine(cuda_device, dtype, width, engine):
    # 3 u_xx + 3 u_yy - u: two first-order directions plus the merged stream (fused engines where they
    # exist for the width, the layer-wise signature kernels otherwise).
    def residual(f, q):
        h = qb.hessian(f)(q)
        return 3.0 * (h[0, 0] + h[1, 1]) - f(q) + qb.sin(math.pi * q[0])

    _check(*_custom([2, width, width, 1], dtype, 777, residual), engine=engine)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_three_dimensional_laplacian_with_unequal_weights(cuda_device, dtype):
    # Width 48 has no fused kernel; 1001 points x 48 units is odd for 16-byte vectors in float64 only.
    def residual(f, q):
        h = qb.hessian(f)(q)
        return h[0, 0] + 2.0 * h[1, 1] + 0.5 * h[2, 2] + q[2]

    _check(*_custom([3, 48, 48, 48, 1], dtype, 1001, residual), engine=(0,))


def test_generic_jet_kernels_carry_the_merged_stream(cuda_device):
    # 37 units x 101 points: planes that are not a multiple of 16 bytes go through the generic jet kernels.
    def residual(f, q):
        h = qb.hessian(f)(q)
        return h[0, 0] + h[1, 1] - qb.grad(f)(q)[0]

    _check(*_custom([2, 37, 37, 1], np.float32, 101, residual), engine=(0,))


def _worker(name, points, **env):
    here = os.path.dirname(os.path.abspath(__file__))
    full = dict(os.environ)
    full.update(env)
    out = subprocess.run([sys.executable, os.path.join(here, "_engine_worker.py"), name, str(points)],
                         env=full, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("name,points", [("poisson2d", 5000), ("heat3d", 700)])
def test_merged_and_unmerged_paths_agree(cuda_device, name, points):
    merged = _worker(name, points)
    plain = _worker(name, points, QB200_MERGE="0")
    assert merged["streams"] < plain["streams"]
    tol = TOLERANCE[np.dtype(np.float32)]
    assert merged["max_error"] <= tol and plain["max_error"] <= tol
    assert relative_error(merged["loss"], plain["loss"]) <= tol
