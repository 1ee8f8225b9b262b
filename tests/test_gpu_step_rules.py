"""Rules of one training step on the device: global-norm clipping, `jvp` in a residual, and what
happens to a step whose kernels reported that a bounded wait gave up."""

import math

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import adam as host
from oracle import contracted
from quabla_b200 import _lib
from quabla_b200._plan import COTANGENT_NAME, Plan, opt_config
from quabla_b200._transforms import CompiledLoss

from _util import TOLERANCE, relative_error, traced
from test_jvp_cpu import nested_loss, problem, transport_loss

pytestmark = pytest.mark.gpu


def _bound_plan(name, points):
    w, compiled, inputs = traced(name, points)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    return w, compiled, inputs, plan


def _host_clip(grads, max_norm):
    """The host rule (python/quabla/optim.py:83-123) on the leaves as the device returned them."""
    clipped, norm = qb.optim.clip_by_global_norm(grads, max_norm)
    return [np.asarray(g) for g in clipped], norm


@pytest.mark.parametrize("name,points", [("poisson2d", 1024), ("poisson1d", 128)])
def test_clipped_updates_follow_the_host_rule_below_at_and_above_the_bound(cuda_device, name, points):
    # clip_norm relative to the measured global norm: far below it (scaled down), exactly at it
    # (unchanged: norm <= max_norm), far above it (unchanged).  cuda_optimizer.rs:39-109, 423-516.
    w, compiled, inputs, plan = _bound_plan(name, points)
    dtype = np.dtype(w.dtype)
    plan.execute()
    grads = plan.outputs()[1:]
    _, norm = _host_clip(grads, 1.0)
    assert math.isfinite(norm) and norm > 0
    params = [np.array(inputs[p[0]], dtype=dtype) for p in compiled.spec.parameters]
    for factor_of_norm in (0.25, 1.0, 8.0):
        clip_norm = norm * factor_of_norm
        for (pname, _, _), value in zip(compiled.spec.parameters, params):
            plan.bind(pname, value)
        plan.execute()
        grads = plan.outputs()[1:]
        plan.optimizer_step(opt_config("sgd", 0.125, clip_norm=clip_norm))
        clipped, _ = _host_clip(grads, clip_norm)
        for index, (g, c, p) in enumerate(zip(grads, clipped, params)):
            expected = host.sgd_update(p, c.reshape(p.shape), 0.125, dtype)
            device = plan.read_parameter(index)
            if factor_of_norm > 1.0:
                assert c.tobytes() == g.tobytes()  # below the bound the rule returns the leaves unchanged
                assert device.tobytes() == expected.reshape(device.shape).tobytes()
            else:
                # The device sums the squares in another order, so its norm may differ in the last bits.
                scale = max(float(np.max(np.abs(expected))), 1e-300)
                assert np.max(np.abs(device - expected.reshape(device.shape))) <= 4 * np.finfo(dtype).eps * scale
        assert plan.query(_lib.Q_NONFINITE_CLIP_SEEN) == 0
    plan.close()


@pytest.mark.parametrize("poison", [math.inf, math.nan])
def test_a_non_finite_gradient_poisons_the_clipped_update_and_the_flag_sticks(cuda_device, poison):
    # An infinite or NaN loss cotangent makes gradient entries infinite or NaN; with clipping on, every
    # gradient then becomes NaN (factor NaN) and the sticky flag is raised and stays raised
    # (cuda_optimizer.rs:98-103, 405-420; python/quabla/optim.py:101-104).
    w, compiled, inputs, plan = _bound_plan("poisson2d", 512)
    dtype = np.dtype(w.dtype)
    plan.execute()
    plan.optimizer_step(opt_config("adam", 1e-3, clip_norm=1.0))
    assert plan.query(_lib.Q_NONFINITE_CLIP_SEEN) == 0
    plan.bind(COTANGENT_NAME, np.array(poison, dtype=dtype))
    plan.execute()
    grads = plan.outputs()[1:]
    assert not all(np.isfinite(g).all() for g in grads)
    plan.optimizer_step(opt_config("adam", 1e-3, clip_norm=1.0))
    assert plan.query(_lib.Q_NONFINITE_CLIP_SEEN) == 1
    for index in range(len(compiled.spec.parameters)):
        assert np.isnan(plan.read_parameter(index)).all()
    # A finite step afterwards does not clear it.
    for (pname, _, _) in compiled.spec.parameters:
        plan.bind(pname, inputs[pname])
    plan.bind(COTANGENT_NAME, np.array(1.0, dtype=dtype))
    plan.execute()
    plan.optimizer_step(opt_config("sgd", 1e-3, clip_norm=1.0))
    assert plan.query(_lib.Q_NONFINITE_CLIP_SEEN) == 1
    assert all(np.isfinite(plan.read_parameter(i)).all() for i in range(len(compiled.spec.parameters)))
    plan.close()


def test_clip_norm_is_validated_before_any_device_work(cuda_device):
    w, compiled, inputs, plan = _bound_plan("poisson1d", 32)
    plan.execute()
    for bad in (0.0, -1.0, math.inf, math.nan):
        with pytest.raises(_lib.BackendError) as info:
            plan.optimizer_step(opt_config("sgd", 1e-3, clip_norm=bad))
        assert info.value.status == _lib.INVALID
        assert "clip_norm must be positive and finite" in str(info.value)
    assert plan.query(_lib.Q_STEP_COUNT) == 0
    plan.close()


@pytest.mark.parametrize("engine", ["default", "layerwise"])
@pytest.mark.parametrize("make_loss,dtype", [(transport_loss, np.float64), (transport_loss, np.float32),
                                             (nested_loss, np.float64)])
def test_jvp_in_a_residual_matches_the_oracle(cuda_device, monkeypatch, make_loss, dtype, engine):
    if engine == "layerwise":
        monkeypatch.setenv("QB200_ENGINE", "layerwise")
    params, p = problem(dtype, points=300)
    args = (params, p)
    compiled = CompiledLoss(make_loss(qb), args, (0,), 0, build_plan=False)
    expected_value, expected_grads = contracted.value_and_grad(compiled.spec, compiled.named_inputs(args))
    value, grads = qb.jit(qb.value_and_grad(make_loss(qb)), device="cuda:0")(*args)
    tol = TOLERANCE[np.dtype(dtype)]
    assert relative_error(value, expected_value) <= tol
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (name, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert relative_error(got[name].reshape(expected.shape), expected) <= tol, name


@pytest.mark.parametrize("name,points", [("poisson2d", 1024), ("heat3d", 256)])
def test_a_wait_that_gave_up_skips_the_update_and_is_reported_once(cuda_device, name, points):
    # One thread waits, with a limit of 64 polls, on a barrier that nothing completes: the plan's device
    # error flag goes up as it would for a staged copy that never lands.  The step that finds the flag
    # must leave parameters and moments alone, the next host synchronisation must say so, and the plan
    # must work again afterwards.
    w, compiled, inputs, plan = _bound_plan(name, points)
    config = opt_config("adam", 1e-3)
    plan.execute()
    plan.optimizer_step(config)
    plan.synchronize()
    before = [plan.read_parameter(i) for i in range(len(compiled.spec.parameters))]
    moments = plan.read_moments(0).copy()
    plan.inject_wait_timeout()
    plan.execute()
    plan.optimizer_step(config)
    with pytest.raises(_lib.BackendError) as info:
        plan.synchronize()
    assert info.value.status == _lib.CUDA_ERROR
    assert "wait limit" in str(info.value) and "skipped" in str(info.value)
    plan.synchronize()  # reported once
    assert plan.query(_lib.Q_STEP_COUNT) == 1  # the skipped update does not count
    for index, old in enumerate(before):
        assert plan.read_parameter(index).tobytes() == old.tobytes()
    assert plan.read_moments(0).tobytes() == moments.tobytes()
    plan.execute()
    plan.optimizer_step(config)
    plan.synchronize()
    assert any(plan.read_parameter(i).tobytes() != old.tobytes() for i, old in enumerate(before))
    plan.close()
