"""Device results against the CPU oracle, through the public API and the C ABI."""

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted
from quabla_b200 import _lib, workloads
from quabla_b200 import _trace as tr
from quabla_b200._plan import Plan, opt_config

from _util import TOLERANCE, relative_error, traced

pytestmark = pytest.mark.gpu

SMALL = {"poisson1d": 128, "poisson2d": 2048, "burgers": 1024, "heat3d": 512, "beam": 2048}


FUSED = {"poisson1d", "poisson2d", "beam"}  # narrow networks take the fused engine by default


@pytest.mark.parametrize("engine", ["default", "layerwise"])
@pytest.mark.parametrize("name", workloads.ORDER)
def test_value_and_grad_matches_the_oracle(cuda_device, monkeypatch, name, engine):
    if engine == "layerwise":
        if name not in FUSED:
            pytest.skip("the default engine of this workload is already the layer-wise one")
        monkeypatch.setenv("QB200_ENGINE", "layerwise")
    w, compiled, inputs = traced(name, SMALL[name])
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    step = qb.jit(qb.value_and_grad(w.loss), device="cuda:0")
    value, grads = step(w.params, *w.data)
    used = next(iter(step._inner._cache.values())).plan.query(_lib.Q_ENGINE)
    assert (used in (1, 2)) == (name in FUSED and engine == "default")  # 1, 2: the fused engines
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert value.dtype == np.dtype(w.dtype)
    assert relative_error(value, expected_loss) <= tol
    got = {}
    for layer, tree in enumerate(grads):
        got[f"params/{layer}/w"], got[f"params/{layer}/b"] = tree["w"], tree["b"]
    for (pname, _, _), expected in zip(compiled.spec.parameters, expected_grads):
        assert got[pname].shape == np.shape(inputs[pname])
        assert relative_error(got[pname].reshape(expected.shape), expected) <= tol, pname


@pytest.mark.parametrize("name", ["poisson1d", "poisson2d"])
def test_forward_only_loss_matches_execute(cuda_device, name):
    w, compiled, inputs = traced(name, SMALL[name])
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(plan.loss(), plan.read_output(0)) <= tol
    plan.close()


@pytest.mark.parametrize("name,points", [("poisson2d", 33), ("poisson2d", 4999), ("beam", 1), ("beam", 31),
                                         ("poisson1d", 127), ("poisson1d", 129), ("poisson1d", 1000)])
def test_ragged_point_counts(cuda_device, name, points):
    # Point counts that do not fill the last tile of the fused engine.
    w, compiled, inputs = traced(name, points)
    w.data = tuple(np.ascontiguousarray(a[:points]) if a.shape[0] > points else a for a in w.data)
    args = (w.params, *w.data)
    from quabla_b200._transforms import CompiledLoss

    compiled = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    inputs = compiled.named_inputs(args)
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    outputs = plan.outputs()
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(outputs[0], expected_loss) <= tol
    for got, expected, (pname, _, _) in zip(outputs[1:], expected_grads, compiled.spec.parameters):
        assert relative_error(got.reshape(expected.shape), expected) <= tol, pname
    plan.close()


def test_repeated_steps_are_bit_identical(cuda_device):
    # The reference guarantees one bit pattern over repeated runs
    # (crates/quabla-core/tests/cuda_determinism.rs:1-11).
    w, compiled, inputs = traced("poisson2d", 4096)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    first = [o.copy() for o in plan.outputs()]
    for _ in range(20):
        plan.execute()
        for a, b in zip(first, plan.outputs()):
            assert a.tobytes() == b.tobytes()
    plan.close()


@pytest.mark.parametrize("name,rule", [("poisson1d", "adam"), ("poisson2d", "adam"), ("poisson2d", "adamw"),
                                        ("poisson1d", "sgd")])
def test_optimizer_step_matches_the_host_rule(cuda_device, name, rule):
    from oracle import adam as host

    w, compiled, inputs = traced(name, SMALL[name])
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    kind = "sgd" if rule == "sgd" else "adam"
    decay = 0.01 if rule == "adamw" else 0.0
    config = opt_config(kind, 1e-3, weight_decay=decay)
    dtype = np.dtype(w.dtype)
    params = {p[0]: np.array(inputs[p[0]], dtype=dtype) for p in compiled.spec.parameters}
    m = {k: np.zeros(v.shape, dtype=dtype) for k, v in params.items()}
    v = {k: np.zeros(p.shape, dtype=dtype) for k, p in params.items()}
    for step in range(1, 4):
        plan.execute()
        grads = plan.outputs()[1:]
        plan.optimizer_step(config)
        for (pname, _, _), g in zip(compiled.spec.parameters, grads):
            if kind == "sgd":
                params[pname] = host.sgd_update(params[pname], g.reshape(params[pname].shape), 1e-3, dtype)
            else:
                params[pname], m[pname], v[pname] = host.adam_update(
                    params[pname], g.reshape(params[pname].shape), m[pname], v[pname], step, 1e-3, 0.9, 0.999, 1e-8,
                    decay, dtype)
        for index, (pname, _, _) in enumerate(compiled.spec.parameters):
            device = plan.read_parameter(index)
            # Same rounded operations in the same order: bit-exact.
            assert device.tobytes() == params[pname].reshape(device.shape).tobytes(), (pname, step)
    assert plan.query(_lib.Q_STEP_COUNT) == 3
    plan.close()


def test_trainer_reduces_the_loss(cuda_device):
    w = workloads.make("poisson1d")
    trainer = qb.optim.Trainer(w.loss, w.params, qb.optim.Adam(learning_rate=1e-2), *w.data, device="cuda:0")
    initial = float(trainer.loss())
    for _ in range(200):
        trainer.step()
    final = float(trainer.loss())
    assert np.isfinite(final) and final < 0.2 * initial
    params = trainer.params
    assert params[0]["w"].shape == (1, 16) and params[2]["b"].shape == (1,)
    assert trainer._executor.device_buffer_count > 0


@pytest.mark.parametrize("activation", ["sin", "sigmoid", "softplus", "silu", "gelu"])
@pytest.mark.parametrize("name", ["poisson1d", "poisson2d", "burgers", "heat3d", "beam"])
def test_other_activations_match_the_oracle(cuda_device, name, activation):
    # sin runs on the same engines as tanh (the fused kernels on narrow networks); the composite activations on
    # the layer-wise engine, whatever the width.  The jets of every activation go up to the order the workload
    # needs (four on the beam, plus one in the reverse sweep).
    w, compiled, inputs = traced(name, SMALL[name], activation)
    assert compiled.spec.activation == activation
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    fused = activation == "sin" and name in FUSED
    assert (plan.query(_lib.Q_ENGINE) in (1, 2)) == fused
    outputs = plan.outputs()
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(outputs[0], expected_loss) <= tol
    for got, expected, (pname, _, _) in zip(outputs[1:], expected_grads, compiled.spec.parameters):
        assert relative_error(got.reshape(expected.shape), expected) <= tol, pname
    plan.close()


def test_trainer_applies_the_schedule_at_the_completed_step(cuda_device):
    # Rates 0, r, r, 0, 0: the first update runs at schedule(0), and three scheduled steps equal two
    # steps at the constant rate r bit for bit.
    w = workloads.make("poisson1d")
    rate = 0.01
    schedule = qb.optim.piecewise_constant([1, 3], [0.0, rate, 0.0])
    scheduled = qb.optim.Trainer(w.loss, w.params, qb.optim.SGD(schedule), *w.data, device="cuda:0")
    fixed = qb.optim.Trainer(w.loss, w.params, qb.optim.SGD(rate), *w.data, device="cuda:0")

    def leaves(trainer):
        return [np.asarray(leaf) for leaf in tr.flatten(trainer.params)[0]]

    start = leaves(scheduled)
    scheduled.step()
    assert all(a.tobytes() == b.tobytes() for a, b in zip(leaves(scheduled), start))
    scheduled.step()
    scheduled.step()
    fixed.step()
    fixed.step()
    after = leaves(scheduled)
    assert all(a.tobytes() == b.tobytes() for a, b in zip(after, leaves(fixed)))
    assert any(a.tobytes() != b.tobytes() for a, b in zip(after, start))
    scheduled.step()
    scheduled.step()
    assert all(a.tobytes() == b.tobytes() for a, b in zip(leaves(scheduled), after))
    assert scheduled._executor.learning_rate == 0.0


@pytest.mark.parametrize("rule", ["adam", "sgd"])
def test_trainer_resumes_bit_for_bit_from_a_saved_state(cuda_device, tmp_path, rule):
    # Five steps in one run == two steps, save, load into a fresh trainer, three more steps.
    w = workloads.make("poisson1d")
    schedule = qb.optim.warmup_cosine_decay(0.0, 0.02, 2, 8, end_value=0.002)

    def build():
        optimizer = qb.optim.AdamW(schedule, weight_decay=0.01) if rule == "adam" else qb.optim.SGD(schedule)
        return qb.optim.Trainer(w.loss, w.params, optimizer, *w.data, device="cuda:0")

    def leaves(tree):
        return [np.asarray(leaf) for leaf in tr.flatten(tree)[0]]

    straight = build()
    for _ in range(5):
        straight.step()

    first = build()
    first.step()
    first.step()
    path = tmp_path / f"{rule}.qb"
    qb.save(path, first.export_state())
    state = qb.load(path)
    assert state["step"] == 2 and state["optimizer"]["step"] == 2
    assert ("m" in state["optimizer"]) == (rule == "adam")

    resumed = build()
    resumed.import_state(state)
    for _ in range(3):
        resumed.step()
    for a, b in zip(leaves(resumed.params), leaves(straight.params)):
        assert a.tobytes() == b.tobytes()
    assert float(resumed.value) == float(straight.value)
    final = resumed.export_state()
    reference = straight.export_state()
    assert final["step"] == reference["step"] == 5
    if rule == "adam":
        for key in ("m", "v"):
            for name, value in final["optimizer"][key].items():
                assert value.tobytes() == reference["optimizer"][key][name].tobytes(), (key, name)

    # Validation happens before anything is written.
    bad = qb.load(path)
    if rule == "adam":
        name = next(iter(bad["optimizer"]["m"]))
        bad["optimizer"]["m"][name] = bad["optimizer"]["m"][name].astype(np.float32)
        with pytest.raises(ValueError):
            resumed.import_state(bad)
    bad = qb.load(path)
    bad["params"] = leaves(bad["params"])[:-1]
    with pytest.raises(ValueError):
        resumed.import_state(bad)


@pytest.mark.parametrize("dtype,width", [(np.float64, 16), (np.float32, 64), (np.float32, 128)])
def test_special_functions_in_the_residual_program(cuda_device, dtype, width):
    # log1p, expm1, erf, erfc and tan of the coordinate, of u and of its derivatives, on the fused
    # engines (widths 16 and 64) and the layer-wise one (128).
    from test_oracle_pins import _special_function_loss

    sizes = [1, width, width, 1]
    params = workloads.init_mlp(qb.random.key(5), sizes, dtype)
    x = qb.random.uniform(qb.random.key(6), (999,), dtype, -1.0, 1.0)
    loss = _special_function_loss(qb)
    from quabla_b200._transforms import CompiledLoss

    compiled = CompiledLoss(loss, (params, x), (0,), 0, build_plan=False)
    inputs = compiled.named_inputs((params, x))
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    outputs = plan.outputs()
    plan.close()
    tol = TOLERANCE[np.dtype(dtype)]
    assert relative_error(outputs[0], expected_loss) <= tol
    for got, expected, (pname, _, _) in zip(outputs[1:], expected_grads, compiled.spec.parameters):
        assert relative_error(got.reshape(expected.shape), expected) <= tol, pname
