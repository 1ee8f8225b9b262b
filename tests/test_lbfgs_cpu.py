"""The quasi-Newton logic of optim.LBFGS on the host, with an analytic evaluator in place of the
device plan (the known answers the reference's own L-BFGS tests use: the Rosenbrock valley from
the classic start, an ill-conditioned quadratic, a float32 pytree;
tests/python/test_optim_api.py:1078-1200)."""

import math

import numpy as np
import pytest

from quabla_b200.optim import LBFGS


def test_rosenbrock_converges_from_the_classic_start():
    def value_and_grad(p):
        x, y = p
        value = (1 - x) ** 2 + 100 * (y - x * x) ** 2
        return value, [np.float64(-2 * (1 - x) - 400 * x * (y - x * x)), np.float64(200 * (y - x * x))]

    solution, info = LBFGS(tolerance_grad=1e-10).minimize_with(value_and_grad, [np.float64(-1.2), np.float64(1.0)])
    assert info["converged"] and info["reason"] in ("gradient_tolerance", "change_tolerance")
    assert abs(float(solution[0]) - 1) < 1e-6 and abs(float(solution[1]) - 1) < 1e-6
    assert info["evaluations"] < 120


def test_ill_conditioned_quadratic_reaches_the_minimizer():
    scales = np.logspace(0, 4, 12)
    target = np.linspace(-1, 1, 12)

    def value_and_grad(p):
        d = p["x"] - target
        return 0.5 * float(np.sum(scales * d * d)), {"x": scales * d}

    solution, info = LBFGS(history=12, tolerance_grad=1e-9, tolerance_change=0.0, max_iterations=2000).minimize_with(
        value_and_grad, {"x": np.zeros(12)})
    assert info["reason"] == "gradient_tolerance"
    assert np.max(np.abs(solution["x"] - target)) < 1e-8


def test_float32_pytree_and_nonfinite_backtracking():
    xs = np.linspace(0.1, 2.0, 16)
    ys = 3.0 * np.exp(-1.5 * xs)

    def value_and_grad(p):
        a, k = float(p["a"]), float(p["k"])
        if k > 40.0:  # an overshoot lands in a region where the model overflows
            return math.inf, {"a": np.float32(math.nan), "k": np.float32(math.nan)}
        r = a * np.exp(-k * xs) - ys
        return float(np.mean(r * r)), {"a": np.float32(np.mean(2 * r * np.exp(-k * xs))),
                                       "k": np.float32(np.mean(2 * r * a * -xs * np.exp(-k * xs)))}

    solution, info = LBFGS(tolerance_grad=1e-10).minimize_with(
        value_and_grad, {"a": np.float32(1.0), "k": np.float32(0.2)})
    assert solution["a"].dtype == np.float32 and solution["k"].dtype == np.float32
    assert abs(float(solution["a"]) - 3.0) < 1e-2 and abs(float(solution["k"]) - 1.5) < 1e-2
    assert info["loss"] < 1e-8


def test_budgets_and_validation():
    def value_and_grad(p):
        return float(p[0] ** 2), [np.float64(2 * p[0])]

    _, info = LBFGS(max_evaluations=2, tolerance_grad=0.0, tolerance_change=0.0).minimize_with(
        value_and_grad, [np.float64(5.0)])
    assert info["reason"] in ("max_evaluations", "gradient_tolerance") and info["evaluations"] <= 3
    _, info = LBFGS(max_iterations=1, tolerance_grad=0.0, tolerance_change=0.0).minimize_with(
        lambda p: (float(np.sum(np.asarray(p[0]) ** 4)), [4 * np.asarray(p[0]) ** 3]), [np.array([1.0, -2.0])])
    assert info["reason"] == "max_iterations" and info["iterations"] == 1
    with pytest.raises(ValueError):
        LBFGS(history=0)
    with pytest.raises(ValueError):
        LBFGS(tolerance_grad=-1.0)
    with pytest.raises(ValueError):
        LBFGS(line_search="armijo")
    with pytest.raises(ValueError):
        LBFGS().minimize_with(lambda p: (math.nan, [np.float64(0.0)]), [np.float64(1.0)])


def test_tiny_gradient_does_not_divide_by_zero():
    def value_and_grad(p):
        return float(1e-300 * p[0] ** 2), [np.float64(2e-300 * p[0])]

    solution, info = LBFGS(tolerance_grad=0.0, tolerance_change=0.0, max_iterations=5).minimize_with(
        value_and_grad, [np.float64(1.0)])
    assert math.isfinite(info["loss"]) and math.isfinite(float(solution[0]))
