"""`jvp` inside a per-point residual: the tracer's forward-mode rule against the literal
oracle, which builds the reference's forward-mode graph (`graph._symbolic_jvp`,
python/quabla/_transforms.py:1321-1361; crates/quabla-core/src/tensor_ir/op/jvp.rs) and
splices it under `vmap`."""

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted, literal
from quabla_b200 import workloads
from quabla_b200._transforms import CompiledLoss

from _util import relative_error


def transport_loss(api, velocity=0.7, decay=0.5):
    """mean((u_t + velocity * u_x + decay * u)^2): the directional derivative along
    (velocity, 1) and the value come out of ONE jvp call."""
    u = workloads.make_u(api)

    def loss(params, p):
        def residual(q):
            value, tangent = api.jvp(lambda s: u(params, s), (q,), (np.array([velocity, 1.0]),))
            return tangent + decay * value

        return api.mean(api.vmap(residual)(p) ** 2)

    return loss


def nested_loss(api):
    """A second derivative as a jvp of a gradient: d/dx (du/dx) + u * du/dt."""
    u = workloads.make_u(api)

    def loss(params, p):
        def residual(q):
            f = lambda s: u(params, s)  # noqa: E731
            g, dg = api.jvp(api.grad(f), (q,), (np.array([1.0, 0.0]),))
            return dg[0] + f(q) * g[1]

        return api.mean(api.vmap(residual)(p) ** 2)

    return loss


def problem(dtype, sizes=(2, 16, 16, 1), points=12, seed=5):
    params = workloads.init_mlp(qb.random.key(seed), list(sizes), dtype)
    p = np.stack([qb.random.uniform(qb.random.fold_in(qb.random.key(seed), j), (points,), dtype, -1.0, 1.0)
                  for j in range(2)], axis=1)
    return params, p


@pytest.mark.parametrize("make_loss", [transport_loss, nested_loss])
def test_traced_jvp_equals_the_reference_forward_mode_graph(make_loss):
    params, p = problem(np.float64)
    expected_value, expected_grads = literal.value_and_grad(make_loss(literal))(params, p)
    args = (params, p)
    compiled = CompiledLoss(make_loss(qb), args, (0,), 0, build_plan=False)
    value, grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args))
    assert relative_error(value, expected_value) <= 1e-13
    want = {}
    for layer, tree in enumerate(expected_grads):
        want[f"params/{layer}/w"], want[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (name, _, _), got in zip(compiled.spec.parameters, grads):
        assert relative_error(got, np.asarray(want[name]).reshape(got.shape)) <= 1e-12, name


def test_jvp_outside_a_trace_is_refused():
    from quabla_b200._errors import UnsupportedOperationError

    with pytest.raises(UnsupportedOperationError):
        qb.jvp(lambda x: x * x, (np.ones(2),), (np.ones(2),))
