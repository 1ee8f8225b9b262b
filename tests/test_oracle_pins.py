"""Pins of the CPU oracle against the reference's own known answers.

The reference (Rust) cannot be built or imported here, so its golden vectors
are its closed-form tests, restated: tests/python/test_api.py:2112-2155,
2689-2766 (PINN loss and gradient by hand, graph size, Adam -> pi, vector
parameters vs finite differences), tests/python/test_optim_api.py:18-111 (Adam
and SGD analytic values), crates/quabla-core/tests/tensor_ir.rs:5296-5334 (a
data-parallel mean equals the single-device result).
"""

import math

import numpy as np
import pytest

from oracle import adam as host
from oracle import contracted, literal, rng
from quabla_b200 import random as qrandom
from quabla_b200 import workloads

from _util import relative_error, traced

PINN_POINTS = 8


def pinn_u(x, w):
    return literal.sin(x * w)


def pinn_loss_reference(w, xs):
    value = gradient = 0.0
    for x in xs:
        r = -(w**2) * math.sin(x * w) + math.pi**2 * math.sin(math.pi * x)
        dr = -2.0 * w * math.sin(x * w) - w**2 * x * math.cos(x * w)
        value += r * r / len(xs)
        gradient += 2.0 * r * dr / len(xs)
    return value, gradient


def vmapped_pinn_loss(w, x):
    u_xx = literal.vmap(literal.grad(literal.grad(pinn_u)), in_axes=(0, None))
    return literal.mean((u_xx(x, w) + math.pi**2 * literal.sin(math.pi * x)) ** 2)


def test_pinn_in_the_canonical_vmap_form_matches_the_hand_derivation():
    x, w = np.linspace(0.05, 0.95, PINN_POINTS), np.array(2.5)
    step = literal.value_and_grad(vmapped_pinn_loss)
    value, grad_w = step(w, x)
    expected_value, expected_grad = pinn_loss_reference(2.5, x.tolist())
    assert abs(float(value) - expected_value) <= 1e-12 * abs(expected_value)
    assert abs(float(grad_w) - expected_grad) <= 1e-12 * abs(expected_grad)
    h = 1e-6
    fd = (float(step(w + h, x)[0]) - float(step(w - h, x)[0])) / (2.0 * h)
    assert abs(float(grad_w) - fd) <= 1e-7 * abs(fd)


def test_vmapped_pinn_graph_has_the_reference_node_count_for_any_point_count():
    # "Graph / plan nodes on this build: 92 / 42 for any number of points"
    # (tests/python/test_api.py:2718-2736); the staged graph is what this pins.
    counts = []
    for points in (1, 8, 64):
        step = literal.value_and_grad(vmapped_pinn_loss)
        step(np.array(2.5), np.linspace(0.05, 0.95, points))
        counts.append(len(step.last_graph.nodes))
    assert counts == [92, 92, 92]


def test_adam_drives_the_pinn_parameter_to_pi():
    x, w = np.linspace(0.05, 0.95, PINN_POINTS), np.array(2.5)
    step = literal.value_and_grad(vmapped_pinn_loss)
    m = v = np.zeros(())
    for t in range(1, 301):
        value, grad_w = step(w, x)
        w, m, v = host.adam_update(w, grad_w, m, v, t, 0.05, 0.9, 0.999, 1e-8, 0.0, np.float64)
    assert f"{float(w):.6f}" == "3.141593"
    assert float(value) < 1e-10


def test_vector_parameter_pinn_matches_finite_differences():
    def u(x, p):
        return p["a"] * literal.tanh(p["b"] * x) + p["c"] * x**3

    def loss(p, x):
        u_xx = literal.vmap(literal.grad(literal.grad(u)), in_axes=(0, None))
        return literal.mean((u_xx(x, p) - literal.sin(x)) ** 2)

    params = {"a": np.array(0.7), "b": np.array(-1.3), "c": np.array(0.2)}
    x = np.linspace(-1.0, 1.0, 6)
    value, grads = literal.value_and_grad(loss)(params, x)
    for name in "abc":
        h = 1e-6
        plus = dict(params, **{name: params[name] + h})
        minus = dict(params, **{name: params[name] - h})
        fd = (float(literal.value_and_grad(loss)(plus, x)[0]) - float(literal.value_and_grad(loss)(minus, x)[0])) / (2 * h)
        assert abs(float(grads[name]) - fd) <= 1e-6 * max(1.0, abs(fd))


def test_adam_analytic_updates():
    # Adam(0.1, b1=0.5, b2=0.75, eps=0.01), p=3, g=2 (test_optim_api.py:18-37).
    p, m, v = np.array([3.0]), np.zeros(1), np.zeros(1)
    p1, m1, v1 = host.adam_update(p, np.array([2.0]), m, v, 1, 0.1, 0.5, 0.75, 0.01, 0.0, np.float64)
    assert math.isclose(p1[0], 3 - 0.1 * 2 / 2.01)
    assert m1[0] == 1
    p2, _, _ = host.adam_update(p1, np.array([2.0]), m1, v1, 2, 0.1, 0.5, 0.75, 0.01, 0.0, np.float64)
    assert math.isclose(p2[0], 3 - 0.2 * 2 / 2.01)


def test_adam_matches_the_textbook_trajectory():
    lr, b1, b2, eps = 0.03, 0.7, 0.95, 0.001  # test_optim_api.py:86-108
    p = np.array([1.0, -2.0])
    m, v = np.zeros(2), np.zeros(2)
    reference, rm, rv = p.tolist(), [0.0, 0.0], [0.0, 0.0]
    for step, values in enumerate(([2.0, -4.0], [-1.0, 0.0], [0.5, 1.0], [0.0, -3.0]), start=1):
        p, m, v = host.adam_update(p, np.array(values), m, v, step, lr, b1, b2, eps, 0.0, np.float64)
        for i, g in enumerate(values):
            rm[i] = b1 * rm[i] + (1 - b1) * g
            rv[i] = b2 * rv[i] + (1 - b2) * g * g
            reference[i] -= lr * (rm[i] / (1 - b1**step)) / (math.sqrt(rv[i] / (1 - b2**step)) + eps)
        assert np.allclose(p, reference, atol=1e-14, rtol=0)


def test_sgd_analytic_update():
    updated = host.sgd_update(np.array([2.0, -1.0]), np.array([4.0, -2.0]), 0.25, np.float64)
    assert updated.tolist() == [1.0, -0.5]


def test_vectorised_random_streams_equal_the_scalar_restatement():
    key = 0x1234ABCD
    assert [k.value for k in qrandom.split(qrandom.key(key), 5)] == rng.split_key(key, 5)
    assert qrandom.fold_in(qrandom.key(key), 1003).value == rng.fold_in_key(key, 1003)
    for dtype in (np.float32, np.float64):
        a = qrandom.uniform(qrandom.key(key), (257,), dtype, -1.0, 1.0)
        b = rng.random_uniform((257,), key, -1.0, 1.0, dtype)
        assert a.dtype == dtype and a.tobytes() == b.tobytes()
        assert a.min() >= -1.0 and a.max() < 1.0
    g = qrandom.glorot_normal(qrandom.key(key), (7, 5))
    assert np.allclose(g, rng.glorot_normal((7, 5), key), rtol=0, atol=1e-15)
    assert qrandom.glorot_normal(qrandom.key(key), (7, 5), np.float32).tobytes() == \
        rng.glorot_normal((7, 5), key).astype(np.float32).tobytes()


@pytest.mark.parametrize("name,points,activation", [
    ("poisson1d", 16, "tanh"), ("poisson2d", 16, "tanh"), ("burgers", 8, "tanh"), ("heat3d", 4, "tanh"),
    ("beam", 8, "tanh"), ("poisson1d", 16, "sin"), ("burgers", 8, "sin"), ("beam", 8, "sin"),
    # The reference's composite activations (where / exp / log1p graphs, composite.rs:160-209, _ops.py:475-505)
    # against closed-form derivative polynomials, to fourth order on the beam:
    ("poisson1d", 16, "sigmoid"), ("beam", 6, "sigmoid"), ("burgers", 8, "softplus"), ("beam", 6, "softplus"),
    ("poisson2d", 8, "silu"), ("beam", 6, "silu"), ("burgers", 8, "gelu"), ("beam", 6, "gelu")])
def test_contracted_oracle_equals_the_literal_oracle(name, points, activation):
    # Literal: the reference's graph transforms and per-node rounding.  Contracted:
    # jets forward, one reverse sweep, float64.  Equal up to rounding.
    w, compiled, inputs = traced(name, points, activation)
    assert compiled.spec.activation == activation
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    wl = workloads.make(name, points, api=literal, activation=activation)
    value, grads = literal.value_and_grad(wl.loss)(wl.params, *wl.data)
    tolerance = 1e-13 if np.dtype(w.dtype) == np.float64 else 2e-6
    assert value.dtype == np.dtype(w.dtype)
    assert relative_error(value, expected_loss) <= tolerance
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (pname, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert relative_error(np.asarray(got[pname]).reshape(expected.shape), expected) <= tolerance, pname


def test_data_parallel_mean_equals_the_single_device_result():
    wl = workloads.make("poisson1d", 16, api=literal)
    x, xb = wl.data
    loss = lambda params, x: literal.mean((literal.vmap(lambda t: workloads.make_u(literal)(params, t))(x)) ** 2)  # noqa: E731
    single_value, single_grads = literal.value_and_grad(loss)(wl.params, x)
    value, grads = literal.value_and_grad_data_parallel(loss, wl.params, [(x[:8],), (x[8:],)], "mean")
    assert abs(float(value) - float(single_value)) <= 1e-15 * abs(float(single_value))
    for a, b in zip(grads, single_grads):
        assert np.allclose(a["w"], b["w"], rtol=1e-13, atol=1e-16)


def test_threads_do_not_change_the_contracted_oracle_beyond_rounding():
    w, compiled, inputs = traced("poisson2d", 512)
    l1, g1 = contracted.value_and_grad(compiled.spec, inputs, threads=1)
    l4, g4 = contracted.value_and_grad(compiled.spec, inputs, threads=4)
    assert abs(l1 - l4) <= 1e-13 * abs(l1)
    for a, b in zip(g1, g4):
        assert relative_error(a, b) <= 1e-12


def test_a_network_cannot_mix_activations():
    import quabla_b200 as qb
    from quabla_b200._errors import UnsupportedOperationError
    from quabla_b200._transforms import CompiledLoss

    def loss(params, x):
        def u(t):
            h = qb.tanh(t.reshape(1, -1) @ params[0]["w"] + params[0]["b"])
            h = qb.sin(h @ params[1]["w"] + params[1]["b"])
            return (h @ params[2]["w"] + params[2]["b"]).reshape(())
        return qb.mean(qb.vmap(u)(x) ** 2)

    params = workloads.init_mlp(qb.random.key(0), [1, 8, 8, 1])
    with pytest.raises(UnsupportedOperationError):
        CompiledLoss(loss, (params, np.linspace(0.0, 1.0, 8)), (0,), 0, build_plan=False)


def _special_function_loss(api):
    """A 1-D loss whose residual applies log1p, expm1, erf, erfc and tan to the coordinate, to u and to
    derivatives of u, so that every chain rule of those kinds is exercised at first and second order."""
    u = workloads.make_u(api)

    def loss(params, x):
        f = lambda t: u(params, t)  # noqa: E731
        value = api.vmap(f)(x)
        slope = api.vmap(api.grad(f))(x)
        curvature = api.vmap(api.grad(api.grad(f)))(x)
        residual = (api.log1p(value * value) + api.expm1(0.3 * slope) + api.erf(curvature) * api.erfc(0.5 * x)
                    + api.tan(0.4 * value) - api.log1p(x * x) * api.erf(x))
        return api.mean(residual ** 2)

    return loss


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_special_function_chains_match_the_literal_oracle(dtype):
    import quabla_b200 as qb
    from quabla_b200._transforms import CompiledLoss

    sizes = [1, 8, 8, 1]
    params = workloads.init_mlp(qb.random.key(5), sizes, dtype)
    x = qb.random.uniform(qb.random.key(6), (24,), dtype, -1.0, 1.0)
    compiled = CompiledLoss(_special_function_loss(qb), (params, x), (0,), 0, build_plan=False)
    inputs = compiled.named_inputs((params, x))
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    value, grads = literal.value_and_grad(_special_function_loss(literal))(params, x)
    tolerance = 1e-12 if dtype == np.float64 else 5e-6
    assert relative_error(value, expected_loss) <= tolerance
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (pname, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert relative_error(np.asarray(got[pname]).reshape(expected.shape), expected) <= tolerance, pname
    # And the gradient is the derivative of the value (central differences on one weight).
    if dtype == np.float64:
        step = literal.value_and_grad(_special_function_loss(literal))
        h = 1e-6
        plus = [dict(layer) for layer in params]
        minus = [dict(layer) for layer in params]
        plus[1]["w"] = params[1]["w"].copy()
        minus[1]["w"] = params[1]["w"].copy()
        plus[1]["w"][2, 3] += h
        minus[1]["w"][2, 3] -= h
        fd = (float(step(plus, x)[0]) - float(step(minus, x)[0])) / (2 * h)
        assert abs(float(grads[1]["w"][2, 3]) - fd) <= 1e-6 * max(abs(fd), 1e-3)


def test_frozen_parameter_decay_is_the_adam_rule_with_zero_gradient_and_moments():
    # decay_frozen_parameters (crates/quabla-python/src/tensor_trace.rs:5071-5105): the shared element rule in
    # float64 with g = m = v = 0, rounded once to the parameter's dtype per step.
    from quabla_b200.optim import decay_frozen_parameter

    for dtype in (np.float32, np.float64):
        p = np.array([1.5, -2.25, 0.0, -0.0, 1e-30, 3.0e5], dtype=dtype)
        zeros = np.zeros_like(p, dtype=np.float64)
        current = p.copy()
        expected = p.copy()
        for step in range(1, 6):
            current = decay_frozen_parameter(current, 0.01, 1e-3)
            wide, _, _ = host.adam_update(expected.astype(np.float64), zeros, zeros, zeros, 1, 1e-3, 0.9, 0.999, 1e-8,
                                          0.01, np.float64)
            expected = wide.astype(dtype)
            assert current.dtype == np.dtype(dtype)
            assert current.tobytes() == expected.tobytes(), (dtype, step)
