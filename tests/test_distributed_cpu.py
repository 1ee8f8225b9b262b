"""Host-side data-parallel logic without a GPU: argument validation, what the
wrapper hands the native factory (checked with a CPU stand-in that combines two
replicas as NCCL would, the reference's own technique,
tests/python/test_distributed_api.py:142-237), and the shard / all-reduce rule
across two gloo ranks."""

import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import literal
from quabla_b200 import distributed, workloads
from quabla_b200._errors import UnsupportedOperationError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def toy_loss(api):
    u = workloads.make_u(api)

    def loss(params, x):
        return api.mean(api.vmap(lambda t: u(params, t))(x) ** 2)

    return loss


def test_argument_validation_follows_the_reference():
    loss = toy_loss(literal)
    with pytest.raises(TypeError):
        distributed.value_and_grad(loss, devices="cuda:0", shard_argnums=1)
    with pytest.raises(ValueError, match="at least two"):
        distributed.value_and_grad(loss, devices=["cuda:0"], shard_argnums=1)
    with pytest.raises(ValueError, match="duplicate"):
        distributed.value_and_grad(loss, devices=["cuda:0", "cuda:0"], shard_argnums=1)
    with pytest.raises(UnsupportedOperationError):
        distributed.value_and_grad(loss, devices=["cpu", "cuda:0"], shard_argnums=1)
    with pytest.raises(ValueError, match="reduction"):
        distributed.value_and_grad(loss, devices=["cuda:0", "cuda:1"], shard_argnums=1, reduction="max")
    dp = distributed.value_and_grad(loss, devices=["cuda:0", "cuda:1"], shard_argnums=1)
    params = workloads.init_mlp(__import__("quabla_b200").random.key(0), [1, 4, 1])
    with pytest.raises(ValueError, match="divisible"):
        dp(params, np.zeros(3))
    with pytest.raises(ValueError, match="mapped-input gradients"):
        distributed.value_and_grad(loss, devices=["cuda:0", "cuda:1"], shard_argnums=0, argnums=0)(params, np.zeros(4))
    with pytest.raises(TypeError, match="positional"):
        dp(params, x=np.zeros(4))


def test_wrapper_and_two_cpu_replicas_match_the_single_device_result(monkeypatch):
    import quabla_b200 as qb

    seen = {}

    def cpu_constructor(function, input_specs, parameter_names, mapped_input_names, device_ordinals, reduction):
        seen.update(specs=input_specs, parameters=parameter_names, mapped=mapped_input_names,
                    ordinals=device_ordinals, reduction=reduction)
        names = [name for name, _, _ in input_specs]

        def run(inputs):
            # Two replicas on the CPU, combined as the collectives would combine them.
            n = len(device_ordinals)
            total_value, total = None, {}
            for rank in range(n):
                local = [distributed.shard(inputs[k], rank, n) if k in mapped_input_names else inputs[k] for k in names]
                positions = [names.index(p) for p in parameter_names]
                value, grads = literal.value_and_grad(function, argnums=positions[0])(*local) \
                    if len(positions) == 1 else (None, None)
                scale = 1.0 / n if reduction == "mean" else 1.0
                total_value = value * scale if total_value is None else total_value + value * scale
                total[parameter_names[0]] = grads * scale if rank == 0 else total[parameter_names[0]] + grads * scale
            return total_value, total

        run.replica_count = len(device_ordinals)
        return run

    monkeypatch.setattr(distributed, "tensor_value_and_grad_data_parallel_cuda_fn", cpu_constructor)

    def loss(w, x):
        return literal.mean(literal.sin(x * w) ** 2)

    w, x = np.array(0.7), np.linspace(0.0, 1.0, 8)
    value, grad = distributed.value_and_grad(loss, devices=["cuda:0", "cuda:1"], shard_argnums=1)(w, x)
    single_value, single_grad = literal.value_and_grad(loss)(w, x)
    assert seen["parameters"] == ["w"] and seen["mapped"] == ["x"] and seen["ordinals"] == [0, 1]
    assert seen["reduction"] == "mean" and [s[0] for s in seen["specs"]] == ["w", "x"]
    assert abs(float(value) - float(single_value)) < 1e-15
    assert abs(float(grad) - float(single_grad)) < 1e-15
    assert qb.distributed is distributed


def test_shard_rejects_uneven_batches_and_keeps_rank_order():
    x = np.arange(12.0).reshape(6, 2)
    assert distributed.shard(x, 1, 3).tolist() == [[4.0, 5.0], [6.0, 7.0]]
    with pytest.raises(ValueError):
        distributed.shard(x, 0, 4)
    with pytest.raises(ValueError):
        distributed.shard(np.array(1.0), 0, 1)


def test_two_gloo_ranks_reproduce_the_full_batch_gradient():
    script = os.path.join(ROOT, "tests", "_gloo_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, script, str(rank), "2"], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = [p.communicate(timeout=300)[0] for p in procs]
    for p, out in zip(procs, outputs):
        assert p.returncode == 0, out
    assert "PARITY OK" in outputs[0]
