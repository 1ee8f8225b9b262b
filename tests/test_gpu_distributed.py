"""Data-parallel plans on real devices.  Multi-device cases need >= 2 GPUs and
skip otherwise; failures are injected on the host, never on a GPU."""

import os
import subprocess
import sys

import numpy as np
import pytest

import quabla_b200 as qb
from oracle import contracted
from quabla_b200 import _lib, distributed, workloads
from quabla_b200._plan import DataParallelPlan, opt_config
from quabla_b200._transforms import CompiledLoss

from _util import TOLERANCE, relative_error

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def devices() -> int:
    return _lib.load().qb200_device_count()


def shard_problem(name: str, points: int, world: int):
    w = workloads.make(name, points)
    args = (w.params, *w.data)
    full = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    local_args = (w.params, *(distributed.shard(a, 0, world) for a in w.data))
    local = CompiledLoss(w.loss, local_args, (0,), 0, build_plan=False)
    return w, args, full, local


def test_single_replica_plan_equals_the_plain_plan(cuda_device):
    w, args, full, local = shard_problem("poisson2d", 256, 1)
    dp = DataParallelPlan(local.spec, [0])
    inputs = full.named_inputs(args)
    for name in full.param_names:
        dp.bind_replicated(name, inputs[name])
    for name in full.data_names:
        dp.bind_sharded(name, inputs[name])
    timing = dp.step("mean")
    assert set(timing) == {"replica_enqueue", "collective", "output_readback"}
    expected_loss, expected_grads = contracted.value_and_grad(full.spec, inputs)
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(dp.read_output(0), expected_loss) <= tol
    for i, g in enumerate(expected_grads):
        assert relative_error(dp.read_output(1 + i).reshape(g.shape), g) <= tol
    dp.close()


@pytest.mark.parametrize("name,points", [("poisson2d", 512), ("poisson1d", 128)])
def test_two_replicas_match_the_full_batch_oracle(cuda_device, name, points):
    if devices() < 2:
        pytest.skip("needs two GPUs")
    w, args, full, local = shard_problem(name, points, 2)
    if any(a.shape[0] % 2 for a in w.data):
        pytest.skip("a point set does not split into two equal shards")
    inputs = full.named_inputs(args)
    dp = DataParallelPlan(local.spec, [0, 1])
    for pname in full.param_names:
        dp.bind_replicated(pname, inputs[pname])
    for dname in full.data_names:
        dp.bind_sharded(dname, inputs[dname])
    dp.step("mean")
    expected_loss, expected_grads = contracted.value_and_grad(full.spec, inputs)
    tol = TOLERANCE[np.dtype(w.dtype)]
    assert relative_error(dp.read_output(0), expected_loss) <= tol
    for i, g in enumerate(expected_grads):
        assert relative_error(dp.read_output(1 + i).reshape(g.shape), g) <= tol
    # Every replica applies the same update to the same reduced gradients.
    dp.optimizer_step(opt_config("adam", 1e-3))
    a, b = dp.replica(0), dp.replica(1)
    for i in range(len(full.spec.parameters)):
        assert a.read_parameter(i).tobytes() == b.read_parameter(i).tobytes()
    # Host-injected failure: the call fails, the communicators are dropped, the next call works.
    dp.inject_host_failure(1)
    with pytest.raises(_lib.BackendError, match="next call recreates them"):
        dp.step("mean")
    dp.step("mean")
    dp.close()


def test_distributed_value_and_grad_over_two_devices(cuda_device):
    if devices() < 2:
        pytest.skip("needs two GPUs")
    w = workloads.make("poisson2d", 512)
    p, pb = w.data
    # Mapped leaves must share one batch size (python/quabla/distributed.py:107-111): the
    # interior points are sharded, the small boundary set is replicated.
    step = qb.distributed.value_and_grad(w.loss, devices=["cuda:0", "cuda:1"], shard_argnums=1)
    value, grads = step(w.params, p, pb)
    single_value, single_grads = qb.jit(qb.value_and_grad(w.loss), device="cuda:0")(w.params, p, pb)
    assert relative_error(value, single_value) <= 1e-5
    for a, b in zip(grads, single_grads):
        assert relative_error(a["w"], b["w"]) <= 1e-5
    assert step.last_executable.replica_count == 2


def test_one_process_per_gpu_bench_line(cuda_device):
    if devices() < 2:
        pytest.skip("needs two GPUs")
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
               "--master-addr", "127.0.0.1", "--master-port", "29655", os.path.join(ROOT, "bench.py"), "--gpus", "2",
               "--steps", "3", "--warmup", "3", "--points", "4096"]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout + done.stderr
    assert '"n_gpus": 2' in done.stdout
