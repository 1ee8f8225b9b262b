"""Single-node data-parallel differentiation over NCCL, with the surface of
python/quabla/distributed.py.

Batch arguments hold full, equally sized axis-zero batches; parameters are
replicated and only their gradients are reduced.  The reduction combines
per-shard losses: `sum` adds them, `mean` averages them, whatever the loss's
own reduction is (python/quabla/distributed.py:1-7).

Two launch models:

* one process, several GPUs -- `value_and_grad(fun, devices=[...], ...)`, the
  reference's model (one host thread drives every replica,
  crates/quabla-core/src/tensor_ir/cuda.rs:681-854);
* one process per GPU (torchrun) -- `shard` cuts this rank's rows out of a
  full batch and `attach` gives a plan or Trainer a communicator, after which
  every step ends with one all-reduce of the flat [loss, gradients] buffer.
"""

from __future__ import annotations

from typing import Any, Callable, Sequence

import numpy as np

from . import _trace as tr
from ._devices import parse_device
from ._errors import UnsupportedOperationError
from ._plan import DataParallelPlan, nccl_unique_id
from ._transforms import CompiledLoss, _is_array, _normalize_argnums

__all__ = ["value_and_grad", "shard", "attach"]


def shard(array, rank: int, world: int) -> np.ndarray:
    """Rows [rank*n/world, (rank+1)*n/world) of a full batch: contiguous equal
    axis-zero shards in rank order (crates/quabla-python/src/tensor_trace.rs:4772-4775)."""
    array = np.asarray(array)
    if array.ndim < 1:
        raise ValueError("every mapped batch leaf must have rank at least one")
    extent = array.shape[0]
    if extent == 0 or extent % world:
        raise ValueError("batch size must be positive and divisible into equal device shards")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} of world {world}")
    n = extent // world
    return np.ascontiguousarray(array[rank * n:(rank + 1) * n])


def broadcast_unique_id(rank: int, make_id: Callable[[], bytes] = nccl_unique_id) -> bytes:
    """Rank 0 makes the 128-byte NCCL id; every rank of the default
    torch.distributed process group returns the same bytes."""
    import torch.distributed as dist

    holder = [make_id() if rank == 0 else None]
    dist.broadcast_object_list(holder, src=0)
    return holder[0]


def attach(target, reduction: str = "mean") -> None:
    """Give a Plan or Trainer of this rank a communicator over the default
    torch.distributed process group (one process per GPU)."""
    import torch.distributed as dist

    if reduction not in ("sum", "mean"):
        raise ValueError("reduction must be 'sum' or 'mean'")
    plan = getattr(getattr(target, "_executor", target), "plan", target)
    rank, world = dist.get_rank(), dist.get_world_size()
    plan.attach_comm(broadcast_unique_id(rank), rank, world, reduction)


class DataParallelExecutable:
    """What the reference's tensor_value_and_grad_data_parallel_cuda_fn returns
    (crates/quabla-python/src/tensor_trace.rs:4622-4882): callable(inputs) ->
    (loss, gradients by name), `.replica_count`, `.device_ordinals`, `.last_timing`."""

    def __init__(self, function: Callable, input_specs, parameter_names, mapped_input_names, device_ordinals,
                 reduction: str) -> None:
        self.device_ordinals = list(device_ordinals)
        self.replica_count = len(self.device_ordinals)
        self._reduction = reduction
        self._parameter_names = list(parameter_names)
        self._mapped = set(mapped_input_names)
        self._names = [name for name, _, _ in input_specs]
        # Trace the loss at SHARD shape (tensor_trace.rs:4688-4710).
        arrays = []
        for name, shape, dtype in input_specs:
            shape = tuple(shape)
            if name in self._mapped:
                shape = (shape[0] // self.replica_count,) + shape[1:]
            arrays.append(np.zeros(shape, dtype=dtype))
        positions = [i for i, name in enumerate(self._names) if name in set(parameter_names)]

        def flat(*leaves):
            return function(*leaves)

        internal = [f"in{i}" for i in range(len(self._names))]
        self._internal = dict(zip(self._names, internal))
        compiled = CompiledLoss(_Named(flat, internal), tuple(arrays), tuple(positions), 0, build_plan=False)
        self._compiled = compiled
        self._plan = DataParallelPlan(compiled.spec, self.device_ordinals)
        self._active = {name for name, _, _ in compiled.spec.parameters}
        self._shapes = dict(zip(compiled.param_names, compiled.param_shapes))
        self.last_timing = None

    def __call__(self, inputs: dict):
        for name in self._names:
            value, internal = inputs[name], self._internal[name]
            if name in self._mapped:
                self._plan.bind_sharded(internal, value)
            elif internal in self._active or name not in self._parameter_names:
                self._plan.bind_replicated(internal, value)
        self.last_timing = self._plan.step(self._reduction)
        value = self._plan.read_output(0)
        gradients = {}
        index = {name: i for i, (name, _, _) in enumerate(self._compiled.spec.parameters)}
        for name in self._parameter_names:
            internal = self._internal[name]
            if internal in index:
                gradients[name] = self._plan.read_output(1 + index[internal]).reshape(self._shapes[internal])
            else:
                gradients[name] = np.zeros(self._shapes[internal], dtype=self._compiled.dtype)
        return value, gradients

    @property
    def plan(self) -> DataParallelPlan:
        return self._plan


class _Named:
    """A callable whose positional parameters carry the given names, so that
    traced inputs are named like the caller's leaves."""

    def __init__(self, function: Callable, names: Sequence[str]) -> None:
        import inspect

        self._function = function
        self.__signature__ = inspect.Signature(
            [inspect.Parameter(n, inspect.Parameter.POSITIONAL_ONLY) for n in names])

    def __call__(self, *args):
        return self._function(*args)


def tensor_value_and_grad_data_parallel_cuda_fn(function, input_specs, parameter_names, mapped_input_names,
                                                device_ordinals, reduction="mean"):
    """Factory with the reference's argument list; tests replace it with a CPU
    constructor (tests/python/test_distributed_api.py:142-237)."""
    return DataParallelExecutable(function, input_specs, parameter_names, mapped_input_names, device_ordinals,
                                  reduction)


class _DistributedValueAndGrad:
    def __init__(self, fun, devices, shard_argnums, argnums, reduction) -> None:
        # Validation order and messages of python/quabla/distributed.py:34-64.
        if not callable(fun):
            raise TypeError("distributed.value_and_grad requires a callable")
        if isinstance(devices, str):
            raise TypeError("devices must be a sequence of CUDA devices")
        ordinals = []
        for device in devices:
            target, ordinal = parse_device(device)
            if target != "cuda":
                raise UnsupportedOperationError("distributed.value_and_grad requires CUDA devices and NCCL",
                                                op="distributed.value_and_grad", device=device)
            ordinals.append(ordinal)
        if len(ordinals) < 2:
            raise ValueError("distributed.value_and_grad requires at least two CUDA devices")
        if len(set(ordinals)) != len(ordinals):
            raise ValueError("devices must not contain duplicate CUDA ordinals")
        if reduction not in ("sum", "mean"):
            raise ValueError("reduction must be 'sum' or 'mean'")
        self._fun = fun
        self._devices = ordinals
        self._shard_argnums = shard_argnums
        self._argnums = argnums
        self._reduction = reduction
        self._cache: dict = {}

    def __call__(self, *args, **kwargs):
        if kwargs:
            raise TypeError("distributed.value_and_grad takes positional arguments only")
        count = len(args)
        argnums = _normalize_argnums(self._argnums, count)
        shard_argnums = _normalize_argnums(self._shard_argnums, count)
        if not argnums:
            raise ValueError("argnums must select at least one replicated parameter")
        if not shard_argnums:
            raise ValueError("shard_argnums must select at least one batch argument")
        if set(argnums) & set(shard_argnums):
            raise ValueError("mapped-input gradients are unsupported; argnums must be replicated")
        from ._transforms import _parameter_names

        roots = _parameter_names(self._fun, count)
        names, leaves, owner, rebuilds = [], [], [], []
        for index, (arg, root) in enumerate(zip(args, roots)):
            arg_leaves, rebuild = tr.flatten(arg)
            rebuilds.append((rebuild, len(arg_leaves)))
            for leaf, path in zip(arg_leaves, tr.leaf_paths(arg, root)):
                if tr.is_traced(leaf):
                    raise UnsupportedOperationError("distributed.value_and_grad cannot run inside another transform",
                                                    op="distributed.value_and_grad", device="cuda")
                names.append(path)
                leaves.append(leaf)
                owner.append(index)
        mapped = [i for i, o in enumerate(owner) if o in shard_argnums]
        parameters = [i for i, o in enumerate(owner) if o in argnums]
        if not mapped or not parameters:
            raise ValueError("batch and parameter arguments must have array leaves")
        batch_size = None
        for i in mapped:
            leaf = leaves[i]
            if not _is_array(leaf):
                raise TypeError("every mapped batch leaf must be an array")
            if np.ndim(leaf) < 1:
                raise ValueError("every mapped batch leaf must have rank at least one")
            extent = np.shape(leaf)[0]
            if extent == 0 or extent % len(self._devices):
                raise ValueError("batch size must be positive and divisible into equal device shards")
            if batch_size is not None and extent != batch_size:
                raise ValueError("all mapped batch leaves must have the same axis-zero batch size")
            batch_size = extent
        for i in parameters:
            if not _is_array(leaves[i]):
                raise TypeError("every differentiated parameter leaf must be an array")
        array_positions = [i for i, leaf in enumerate(leaves) if _is_array(leaf)]
        key = tuple((names[i], tuple(np.shape(leaves[i])), str(np.asarray(leaves[i]).dtype)) for i in array_positions)
        executable = self._cache.get(key)
        if executable is None:
            template = [None if _is_array(leaf) else leaf for leaf in leaves]

            def flat_loss(*inputs):
                values = list(template)
                for position, value in zip(array_positions, inputs):
                    values[position] = value
                it = iter(values)
                rebuilt = [rebuild([next(it) for _ in range(n)]) for rebuild, n in rebuilds]
                return self._fun(*rebuilt)

            specs = [(names[i], np.shape(leaves[i]), np.asarray(leaves[i]).dtype) for i in array_positions]
            executable = tensor_value_and_grad_data_parallel_cuda_fn(
                flat_loss, specs, [names[i] for i in parameters], [names[i] for i in mapped], self._devices,
                self._reduction)
            if len(self._cache) >= 8:
                self._cache.pop(next(iter(self._cache)))
            self._cache[key] = executable
        value, gradients = executable({names[i]: leaves[i] for i in array_positions})
        self.last_executable = executable
        trees = []
        for argnum in argnums:
            rebuild, _ = rebuilds[argnum]
            trees.append(rebuild([gradients[names[i]] for i in parameters if owner[i] == argnum]))
        return value, (trees[0] if isinstance(self._argnums, int) else tuple(trees))


def value_and_grad(fun: Callable, *, devices: Sequence[str], shard_argnums, argnums=0, reduction: str = "mean"):
    """A scalar loss and replicated parameter gradients over several CUDA devices
    (python/quabla/distributed.py:197-214)."""
    return _DistributedValueAndGrad(fun, devices, shard_argnums, argnums, reduction)
