"""Mixed partial derivatives of the network (off-diagonal Hessian entries, third-order mixed terms): the
tracer rewrites them as pure derivatives along sums of directions; value and gradients must equal the
literal oracle's, which builds the reference's full Hessian (python/quabla/_transforms.py:1812-2036,
2173-2179) and reads the entry."""

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted, literal
from quabla_b200 import workloads
from quabla_b200._transforms import CompiledLoss

from _util import relative_error


def cross_only(api):
    """Residual with u_xy alone: no pure second derivative, so both polarisation directions are new."""
    u = workloads.make_u(api)

    def loss(params, p):
        def residual(q):
            h = api.hessian(lambda s: u(params, s))(q)
            return h[0, 1] - 0.3 * u(params, q)

        return api.mean(api.vmap(residual)(p) ** 2)

    return loss


def full_hessian(api):
    """A Monge-Ampere-like residual u_xx u_yy - u_xy u_yx: every Hessian entry, the mixed one twice."""
    u = workloads.make_u(api)

    def loss(params, p):
        def residual(q):
            h = api.hessian(lambda s: u(params, s))(q)
            return h[0, 0] * h[1, 1] - h[0, 1] * h[1, 0] + api.sin(q[0])

        return api.mean(api.vmap(residual)(p) ** 2)

    return loss


def third_order_mixed(api):
    """u_xxy through grad of a Hessian entry."""
    u = workloads.make_u(api)

    def loss(params, p):
        def residual(q):
            u_xx = lambda s: api.hessian(lambda r: u(params, r))(s)[0, 0]  # noqa: E731
            return api.grad(u_xx)(q)[1]

        return api.mean(api.vmap(residual)(p) ** 2)

    return loss


CASES = [cross_only, full_hessian, third_order_mixed]


def problem(dtype=np.float64, points=10, seed=9, width=12):
    params = workloads.init_mlp(qb.random.key(seed), [2, width, width, 1], dtype)
    p = np.stack([qb.random.uniform(qb.random.fold_in(qb.random.key(seed), j), (points,), dtype, -1.0, 1.0)
                  for j in range(2)], axis=1)
    return params, p


@pytest.mark.parametrize("make_loss", CASES)
def test_mixed_partials_equal_the_reference_hessian(make_loss):
    params, p = problem()
    expected_value, expected_grads = literal.value_and_grad(make_loss(literal))(params, p)
    args = (params, p)
    compiled = CompiledLoss(make_loss(qb), args, (0,), 0, build_plan=False)
    value, grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args))
    assert relative_error(value, expected_value) <= 1e-12
    want = {}
    for layer, tree in enumerate(expected_grads):
        want[f"params/{layer}/w"], want[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (name, _, _), got in zip(compiled.spec.parameters, grads):
        assert relative_error(got, np.asarray(want[name]).reshape(got.shape)) <= 1e-11, name


def test_streams_of_the_rewritten_mixed_partials(monkeypatch):
    params, p = problem()
    # u_xy = (D^2_{x+y} - D^2_{x-y}) / 4: two new directions and no unit direction; the two second derivatives
    # enter through one weighted sum, so they ride the merged stream (1 + 2 + 1 streams) ...
    spec = CompiledLoss(cross_only(qb), (params, p), (0,), 0, build_plan=False).spec
    assert spec.sets[0].directions == [((1.0, 1.0), 1), ((1.0, -1.0), 1)]
    assert spec.sets[0].merge_weights == [0.25, -0.25] and spec.sets[0].streams == 4
    # ... or two second-order directions when merging is off.
    monkeypatch.setenv("QB200_MERGE", "0")
    spec = CompiledLoss(cross_only(qb), (params, p), (0,), 0, build_plan=False).spec
    assert sorted(spec.sets[0].directions) == [((1.0, -1.0), 2), ((1.0, 1.0), 2)]
    monkeypatch.delenv("QB200_MERGE")
    # x and y are carried to second order anyway: u_xy = (D^2_{x+y} - u_xx - u_yy) / 2 adds one direction.
    spec = CompiledLoss(full_hessian(qb), (params, p), (0,), 0, build_plan=False).spec
    assert sorted(spec.sets[0].directions) == [((0.0, 1.0), 2), ((1.0, 0.0), 2), ((1.0, 1.0), 2)]
    # u_xxy = (D^3_{2x+y} - D^3_{2x-y} - 2 D^3_y) / 24.
    spec = CompiledLoss(third_order_mixed(qb), (params, p), (0,), 0, build_plan=False).spec
    assert sorted(spec.sets[0].directions) == [((0.0, 1.0), 3), ((2.0, -1.0), 3), ((2.0, 1.0), 3)]
