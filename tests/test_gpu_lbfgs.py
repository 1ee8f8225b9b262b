"""optim.LBFGS with every evaluation on the device plan."""

import numpy as np
import pytest

import quabla_b200 as qb
from quabla_b200 import workloads

pytestmark = pytest.mark.gpu


def test_lbfgs_refines_a_pinn_on_the_device(cuda_device):
    w = workloads.make("poisson1d", 128)
    start = qb.jit(qb.value_and_grad(w.loss), device="cuda:0")(w.params, *w.data)[0]
    params, info = qb.optim.LBFGS(max_iterations=60, tolerance_grad=0.0, tolerance_change=0.0).minimize(
        w.loss, w.params, *w.data, device="cuda:0")
    assert info["iterations"] >= 1 and info["evaluations"] >= info["iterations"]
    assert info["loss"] < 1e-2 * float(start)
    # The returned parameters reproduce the reported loss.
    again = qb.jit(qb.value_and_grad(w.loss), device="cuda:0")(params, *w.data)[0]
    assert abs(float(again) - info["loss"]) <= 1e-9 * max(1.0, abs(info["loss"]))
    assert [layer["w"].shape for layer in params] == [layer["w"].shape for layer in w.params]


def test_lbfgs_on_a_float32_network(cuda_device):
    w = workloads.make("poisson2d", 1024)
    start = qb.jit(qb.value_and_grad(w.loss), device="cuda:0")(w.params, *w.data)[0]
    params, info = qb.optim.LBFGS(max_iterations=15).minimize(w.loss, w.params, *w.data, device="cuda:0")
    assert info["loss"] < float(start)
    assert params[0]["w"].dtype == np.float32
