"""Network shapes around the layer-wise engine's special cases, against the CPU oracle: one to three hidden
layers (with one hidden layer the first layer is also the last hidden layer), widths that take the tensor-core
GEMMs, the FP64 MMA GEMMs or the plain kernels, widths whose rows do not fill whole warps or whole blocks of the
jet kernels, and three inputs."""

import math

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted
from quabla_b200 import workloads
from quabla_b200._transforms import CompiledLoss

from _util import TOLERANCE, relative_error

pytestmark = pytest.mark.gpu


def _problem(sizes, dtype, points, seed=5):
    params = workloads.init_mlp(qb.random.key(seed), sizes, dtype)
    p = np.stack([qb.random.uniform(qb.random.fold_in(qb.random.key(seed), j), (points,), dtype, -1.0, 1.0)
                  for j in range(sizes[0])], axis=1)
    return params, p


def _loss(api):
    u = workloads.make_u(api)

    def loss(params, p):
        laplacian = api.vmap(lambda q: api.trace(api.hessian(lambda s: u(params, s))(q)))(p)
        value = api.vmap(lambda q: u(params, q))(p)
        return api.mean((laplacian + math.pi * value) ** 2)

    return loss


@pytest.mark.parametrize("sizes,dtype", [
    ([2, 256, 1], np.float32), ([2, 256, 256, 1], np.float32), ([3, 128, 256, 128, 1], np.float32),
    ([2, 128, 1], np.float64), ([2, 128, 128, 1], np.float64), ([3, 128, 128, 128, 1], np.float64),
    ([2, 48, 48, 1], np.float64), ([2, 96, 96, 1], np.float32), ([4, 192, 192, 1], np.float32),
], ids=lambda v: "-".join(map(str, v)) if isinstance(v, list) else np.dtype(v).name)
def test_value_and_gradients_match_the_oracle(cuda_device, monkeypatch, sizes, dtype):
    monkeypatch.setenv("QB200_ENGINE", "layerwise")
    params, p = _problem(sizes, dtype, points=900)
    args = (params, p)
    compiled = CompiledLoss(_loss(qb), args, (0,), 0, build_plan=False)
    expected_value, expected_grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args))
    value, grads = qb.jit(qb.value_and_grad(_loss(qb)), device="cuda:0")(*args)
    tol = TOLERANCE[np.dtype(dtype)]
    assert relative_error(value, expected_value) <= tol
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (name, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert relative_error(got[name].reshape(expected.shape), expected) <= tol, name


def test_smallest_launches_that_take_the_bfloat16_scheme(cuda_device, monkeypatch):
    # 13,200 points x 5 streams = 66,000 rows per GEMM, just over the 65,536 rows from which the forward and
    # data-gradient GEMMs run their correction products as bfloat16 instructions: the case with the fewest points
    # to average that scheme's random rounding errors out of the bias gradients.
    monkeypatch.setenv("QB200_ENGINE", "layerwise")
    sizes, dtype = [3, 128, 256, 128, 1], np.float32
    params, p = _problem(sizes, dtype, points=13200)
    args = (params, p)
    compiled = CompiledLoss(_loss(qb), args, (0,), 0, build_plan=False)
    expected_value, expected_grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args),
                                                               threads=contracted.max_threads())
    value, grads = qb.jit(qb.value_and_grad(_loss(qb)), device="cuda:0")(*args)
    tol = TOLERANCE[np.dtype(dtype)]
    assert relative_error(value, expected_value) <= tol
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (name, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert relative_error(got[name].reshape(expected.shape), expected) <= 0.5 * tol, name
