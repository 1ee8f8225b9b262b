"""Python mirror of the plan description and the plan handle of the C ABI.

`PlanSpec` is what the fusion pass (quabla_b200/_trace.py) or a caller that
already knows its PDE hands to the backend; `Plan` wraps a `qb200_plan*` with
the method set of the reference's `CudaExecutionPlan`
(crates/quabla-core/src/tensor_ir/cuda.rs:1119-1490,
crates/quabla-core/src/tensor_ir/cuda_optimizer.rs:207-420).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._symbolic import Program

COTANGENT_NAME = "__quabla_loss_cotangent"


@dataclass
class SetSpec:
    """One point set: weight * sum over points of program(point)."""

    n_points: int
    weight: float
    columns: list[tuple[int, int]]            # (input index, column); network inputs first
    directions: list[tuple[tuple[float, ...], int]]  # (vector, order)
    program: Program
    # One weight per direction when the set carries the merged second-order stream
    # sum_j w_j d^2u/dv_j^2 as its last stream (qb200_desc_set_merge_second_order); else None.
    merge_weights: list[float] | None = None

    @property
    def streams(self) -> int:
        return 1 + sum(order for _, order in self.directions) + (0 if self.merge_weights is None else 1)


@dataclass
class PlanSpec:
    dtype: np.dtype
    sizes: list[int]
    parameters: list[tuple[str, int, int]] = field(default_factory=list)   # (name, layer, kind)
    inputs: list[tuple[str, int, int, bool]] = field(default_factory=list)  # (name, rows, cols, retained)
    sets: list[SetSpec] = field(default_factory=list)
    activation: str = "tanh"   # of the hidden layers: one of _lib.ACTIVATIONS
    # The same loss traced without the merged stream (one second-order stream per direction, what
    # QB200_MERGE=0 traces), when some set of this spec uses the merged stream; None otherwise.  Either
    # form can be handed to Plan: they compute the same value and gradients with different stream counts.
    unmerged: "PlanSpec | None" = None

    def parameter_shape(self, index: int) -> tuple[int, ...]:
        _, layer, kind = self.parameters[index]
        if kind == _lib.WEIGHT:
            return (self.sizes[layer], self.sizes[layer + 1])
        return (self.sizes[layer + 1],)


def dtype_code(dtype) -> int:
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return _lib.F32
    if dtype == np.float64:
        return _lib.F64
    raise TypeError(f"a plan has one floating dtype, float32 or float64; got {dtype}")


def _int32_array(values) -> C.Array:
    values = [int(v) for v in values]
    return (C.c_int32 * max(1, len(values)))(*values)


def _double_array(values) -> C.Array:
    values = [float(v) for v in values]
    return (C.c_double * max(1, len(values)))(*values)


def build_desc(spec: PlanSpec) -> C.c_void_p:
    """A qb200_desc* for `spec`; the caller destroys it."""
    lib = _lib.load()
    desc = C.c_void_p()
    _lib.check(lib.qb200_desc_create(dtype_code(spec.dtype), C.byref(desc)))
    try:
        _lib.check(lib.qb200_desc_set_network(desc, _int32_array(spec.sizes), len(spec.sizes)))
        if spec.activation != "tanh":
            _lib.check(lib.qb200_desc_set_activation(desc, _lib.ACTIVATIONS[spec.activation]))
        for name, layer, kind in spec.parameters:
            _lib.check(lib.qb200_desc_add_parameter(desc, name.encode(), layer, kind))
        for name, rows, cols, retained in spec.inputs:
            index = C.c_int32()
            _lib.check(lib.qb200_desc_add_input(desc, name.encode(), rows, cols, int(retained), C.byref(index)))
        for s in spec.sets:
            index = C.c_int32()
            _lib.check(lib.qb200_desc_add_set(desc, s.n_points, float(s.weight), C.byref(index)))
            for input_index, column in s.columns:
                _lib.check(lib.qb200_desc_set_add_column(desc, index.value, input_index, column))
            for vector, order in s.directions:
                _lib.check(lib.qb200_desc_set_add_direction(desc, index.value, _double_array(vector), order))
            if s.merge_weights is not None:
                _lib.check(lib.qb200_desc_set_merge_second_order(desc, index.value, _double_array(s.merge_weights),
                                                                 len(s.merge_weights)))
            p = s.program
            _lib.check(lib.qb200_desc_set_program(
                desc, index.value, _int32_array(p.code), p.n_instr, _double_array(p.consts), len(p.consts),
                p.n_regs, p.value_reg, _int32_array(p.grad_regs), len(p.grad_regs)))
    except Exception:
        lib.qb200_desc_destroy(desc)
        raise
    return desc


def opt_config(rule: str, learning_rate: float, beta1: float = 0.9, beta2: float = 0.999, epsilon: float = 1e-8,
               weight_decay: float = 0.0, clip_norm: float | None = None) -> _lib.OptConfig:
    if rule not in ("adam", "sgd"):
        raise ValueError(f"optimizer must be 'adam' or 'sgd', got {rule!r}")
    return _lib.OptConfig(
        rule=_lib.ADAM if rule == "adam" else _lib.SGD,
        has_clip=0 if clip_norm is None else 1,
        learning_rate=float(learning_rate), beta1=float(beta1), beta2=float(beta2), epsilon=float(epsilon),
        weight_decay=float(weight_decay), clip_norm=0.0 if clip_norm is None else float(clip_norm))


class Plan:
    """A compiled single-device plan (qb200_plan*)."""

    def __init__(self, spec: PlanSpec, device_ordinal: int = 0, _handle=None) -> None:
        self.spec = spec
        self.dtype = np.dtype(spec.dtype)
        self._lib = _lib.load()
        self._owned = _handle is None
        if _handle is not None:
            self._handle = _handle
            return
        desc = build_desc(spec)
        try:
            handle = C.c_void_p()
            _lib.check(self._lib.qb200_plan_create(desc, int(device_ordinal), C.byref(handle)))
        finally:
            self._lib.qb200_desc_destroy(desc)
        self._handle = handle

    def close(self) -> None:
        if getattr(self, "_handle", None) and self._owned:
            self._lib.qb200_plan_destroy(self._handle)
        self._handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    def _host(self, value) -> np.ndarray:
        return np.ascontiguousarray(np.asarray(value), dtype=self.dtype)

    def bind(self, name: str, value) -> None:
        host = self._host(value)
        _lib.check(self._lib.qb200_plan_bind(self._handle, name.encode(), host.ctypes.data, host.nbytes))

    def bind_raw(self, name: str, address: int, nbytes: int) -> None:
        """Bind from a host address (for example a pinned staging buffer)."""
        _lib.check(self._lib.qb200_plan_bind(self._handle, name.encode(), C.c_void_p(address), nbytes))

    def execute(self) -> None:
        _lib.check(self._lib.qb200_plan_execute(self._handle))

    def read_output(self, index: int) -> np.ndarray:
        shape = () if index == 0 else self.spec.parameter_shape(index - 1)
        out = np.empty(shape, dtype=self.dtype)
        _lib.check(self._lib.qb200_plan_read_output(self._handle, index, out.ctypes.data, out.nbytes))
        return out

    def outputs(self) -> list[np.ndarray]:
        return [self.read_output(i) for i in range(1 + len(self.spec.parameters))]

    def optimizer_step(self, config: _lib.OptConfig) -> None:
        _lib.check(self._lib.qb200_plan_optimizer_step(self._handle, C.byref(config)))

    def loss(self) -> np.ndarray:
        out = np.empty((), dtype=self.dtype)
        _lib.check(self._lib.qb200_plan_loss(self._handle, out.ctypes.data))
        return out

    def read_input(self, name: str, shape) -> np.ndarray:
        out = np.empty(shape, dtype=self.dtype)
        _lib.check(self._lib.qb200_plan_read_input(self._handle, name.encode(), out.ctypes.data, out.nbytes))
        return out

    def sample_uniform(self, name: str, column: int, key, minval: float = 0.0, maxval: float = 1.0) -> None:
        """Resample one column of a data input on the device: the values of
        random.uniform(key, (rows,), dtype, minval, maxval), bit for bit, with no host copy."""
        value = getattr(key, "value", key)
        _lib.check(self._lib.qb200_plan_sample_uniform(self._handle, name.encode(), int(column),
                                                       int(value) & 0xFFFFFFFFFFFFFFFF, float(minval), float(maxval)))

    def read_parameter(self, index: int) -> np.ndarray:
        return self.read_input(self.spec.parameters[index][0], self.spec.parameter_shape(index))

    def read_moments(self, which: int) -> np.ndarray:
        out = np.empty((self.query(_lib.Q_PARAMETER_COUNT),), dtype=self.dtype)
        _lib.check(self._lib.qb200_plan_read_moments(self._handle, which, out.ctypes.data, out.nbytes))
        return out

    def write_moments(self, which: int, values, step_count: int) -> None:
        host = self._host(values).reshape(-1)
        _lib.check(self._lib.qb200_plan_write_moments(self._handle, which, host.ctypes.data, host.nbytes,
                                                      int(step_count)))

    def query(self, key: int) -> int:
        out = C.c_int64()
        _lib.check(self._lib.qb200_plan_query(self._handle, key, C.byref(out)))
        return out.value

    def synchronize(self) -> None:
        _lib.check(self._lib.qb200_plan_synchronize(self._handle))

    def set_option(self, key: int, value: int) -> None:
        _lib.check(self._lib.qb200_plan_set_option(self._handle, int(key), int(value)))

    def inject_wait_timeout(self) -> None:
        """Test seam: enqueue a bounded wait that gives up, which raises the plan's device error flag."""
        _lib.check(self._lib.qb200_plan_inject_wait_timeout(self._handle))

    def attach_comm(self, unique_id: bytes, rank: int, world: int, reduction: str = "mean") -> None:
        if len(unique_id) != 128:
            raise ValueError("an NCCL unique id is 128 bytes")
        buffer = C.create_string_buffer(unique_id, 128)
        code = {"sum": _lib.REDUCE_SUM, "mean": _lib.REDUCE_MEAN}[reduction]
        _lib.check(self._lib.qb200_plan_attach_comm(self._handle, buffer, rank, world, code))

    def detach_comm(self) -> None:
        _lib.check(self._lib.qb200_plan_detach_comm(self._handle))

    @property
    def device_buffer_count(self) -> int:
        return self.query(_lib.Q_DEVICE_BUFFER_COUNT)


def nccl_unique_id() -> bytes:
    buffer = C.create_string_buffer(128)
    _lib.check(_lib.load().qb200_nccl_unique_id(buffer))
    return buffer.raw


class DataParallelPlan:
    """A single-process data-parallel plan (qb200_dp*): one replica per device,
    driven by one host thread, the shape of the reference's
    CudaDataParallelExecutionPlan (crates/quabla-core/src/tensor_ir/cuda.rs:116-170, 621-866).
    `spec` describes ONE shard."""

    def __init__(self, spec: PlanSpec, ordinals) -> None:
        self.spec = spec
        self.dtype = np.dtype(spec.dtype)
        self.ordinals = [int(o) for o in ordinals]
        self._lib = _lib.load()
        desc = build_desc(spec)
        try:
            handle = C.c_void_p()
            _lib.check(self._lib.qb200_dp_create(desc, _int32_array(self.ordinals), len(self.ordinals),
                                                 C.byref(handle)))
        finally:
            self._lib.qb200_desc_destroy(desc)
        self._handle = handle
        self.last_timing = None

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.qb200_dp_destroy(self._handle)
        self._handle = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    @property
    def replica_count(self) -> int:
        return self._lib.qb200_dp_replica_count(self._handle)

    def _host(self, value) -> np.ndarray:
        return np.ascontiguousarray(np.asarray(value), dtype=self.dtype)

    def bind_sharded(self, name: str, value) -> None:
        host = self._host(value)
        _lib.check(self._lib.qb200_dp_bind_sharded(self._handle, name.encode(), host.ctypes.data, host.nbytes))

    def bind_replicated(self, name: str, value) -> None:
        host = self._host(value)
        _lib.check(self._lib.qb200_dp_bind_replicated(self._handle, name.encode(), host.ctypes.data, host.nbytes))

    def step(self, reduction: str = "mean") -> dict:
        timing = _lib.DpTiming()
        code = {"sum": _lib.REDUCE_SUM, "mean": _lib.REDUCE_MEAN}[reduction]
        _lib.check(self._lib.qb200_dp_step(self._handle, code, C.byref(timing)))
        self.last_timing = {"replica_enqueue": timing.replica_enqueue, "collective": timing.collective,
                            "output_readback": timing.output_readback}
        return self.last_timing

    def read_output(self, index: int) -> np.ndarray:
        shape = () if index == 0 else self.spec.parameter_shape(index - 1)
        out = np.empty(shape, dtype=self.dtype)
        _lib.check(self._lib.qb200_dp_read_output(self._handle, index, out.ctypes.data, out.nbytes))
        return out

    def optimizer_step(self, config: _lib.OptConfig) -> None:
        _lib.check(self._lib.qb200_dp_optimizer_step(self._handle, C.byref(config)))

    def replica(self, rank: int) -> Plan:
        handle = self._lib.qb200_dp_replica(self._handle, rank)
        if not handle:
            raise IndexError(f"replica {rank} of {self.replica_count}")
        return Plan(self.spec, _handle=C.c_void_p(handle))

    def inject_host_failure(self, rank: int) -> None:
        _lib.check(self._lib.qb200_dp_inject_host_failure(self._handle, rank))
