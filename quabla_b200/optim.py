"""Optimizers and the device Trainer, with the surface of python/quabla/optim.py.

`Trainer` keeps parameters and Adam moments on the device and runs
value-and-gradient plus the update as device kernels every step
(reference: optim.py:351-550 on top of
crates/quabla-python/src/tensor_trace.rs:118-199, 5062-5390).  The pure
`update` methods are the reference's host optimizer (optim.py:200-234,
crates/quabla-python/src/tensor.rs:1675-1778) for code that drives
`jit(value_and_grad(...))` by hand; the Trainer never calls them.
"""

from __future__ import annotations

import math
import operator
from typing import Any, Callable, Sequence

import numpy as np

from . import _trace as tr
from ._devices import require_device
from ._errors import UnsupportedOperationError
from ._lbfgs import LBFGS
from ._plan import COTANGENT_NAME, opt_config
from ._schedules import constant, cosine_decay, exponential_decay, piecewise_constant, warmup_cosine_decay
from ._transforms import CompiledLoss, _is_array

__all__ = ["Adam", "AdamW", "SGD", "LBFGS", "Trainer", "clip_by_global_norm", "constant", "cosine_decay",
           "exponential_decay", "piecewise_constant", "warmup_cosine_decay"]


def _positive(value, name: str) -> float:
    value = float(value)
    if not (math.isfinite(value) and value > 0):
        raise ValueError(f"{name} must be positive and finite, got {value!r}")
    return value


def _learning_rate(value):
    return value if callable(value) else _positive(value, "learning_rate")


def _rate_at(learning_rate, step: int) -> float:
    if not callable(learning_rate):
        return learning_rate
    value = float(learning_rate(step))
    if not math.isfinite(value) or value < 0:
        raise ValueError(
            f"learning-rate schedule returned {value!r} at step {step}; rates must be finite and nonnegative")
    return value


def clip_by_global_norm(grads: Any, max_norm: float) -> tuple[Any, float]:
    """Scale a gradient pytree so its global L2 norm is at most `max_norm`
    (host version; rule of python/quabla/optim.py:83-123)."""
    max_norm = _positive(max_norm, "max_norm")
    leaves, rebuild = tr.flatten(grads)
    wide = [np.asarray(leaf, dtype=np.float64) for leaf in leaves if np.size(leaf)]
    peaks = [float(np.max(np.abs(v))) for v in wide]
    peak = math.nan if any(math.isnan(p) for p in peaks) else max(peaks, default=0)
    scale = peak if math.isfinite(peak) and peak > 0 else 1.0
    total = sum(float(np.sum((v / scale) * (v / scale))) for v in wide)
    root = math.sqrt(total)
    norm = scale * root
    if norm <= max_norm:
        return grads, norm
    if math.isfinite(norm):
        factor = max_norm / norm
    elif math.isfinite(peak):
        factor = (max_norm / scale) / root
    else:
        factor = math.nan
    clipped = [(np.asarray(leaf, dtype=np.float64) * factor).astype(np.asarray(leaf).dtype) for leaf in leaves]
    return rebuild(clipped), norm


class _AdamBase:
    weight_decay = 0.0

    def _configure(self, learning_rate, b1, b2, eps, beta1, beta2, epsilon, clip_norm) -> None:
        self.learning_rate = _learning_rate(learning_rate)
        self.b1 = float(b1 if beta1 is None else beta1)
        self.b2 = float(b2 if beta2 is None else beta2)
        self.eps = _positive(eps if epsilon is None else epsilon, "epsilon")
        if not (0 <= self.b1 < 1 and 0 <= self.b2 < 1):
            raise ValueError("Adam betas must be in [0, 1)")
        self.clip_norm = None if clip_norm is None else _positive(clip_norm, "clip_norm")

    def init(self, params: Any) -> dict:
        leaves, rebuild = tr.flatten(params)
        zeros = lambda: rebuild([np.zeros(np.shape(p), dtype=np.float64) for p in leaves])  # noqa: E731
        return {"step": 0, "m": zeros(), "v": zeros()}

    def update(self, params: Any, grads: Any, state: dict) -> tuple[Any, dict]:
        """Pure host update: moments in float64, the parameter rounded once to
        its dtype (element rule of device_optimizer.rs:241-285)."""
        if type(state) is not dict or set(state) != {"step", "m", "v"}:
            raise ValueError("Adam state must contain step, m, and v")
        p_leaves, rebuild = tr.flatten(params)
        g_leaves, _ = tr.flatten(grads)
        m_leaves, _ = tr.flatten(state["m"])
        v_leaves, _ = tr.flatten(state["v"])
        if not (len(p_leaves) == len(g_leaves) == len(m_leaves) == len(v_leaves)):
            raise ValueError("gradient and moment trees must match the parameters")
        if self.clip_norm is not None:
            clipped, _ = clip_by_global_norm(g_leaves, self.clip_norm)
            g_leaves = list(clipped)
        step = state["step"] + 1
        lr = _rate_at(self.learning_rate, state["step"])
        c1, c2 = 1 - self.b1**step, 1 - self.b2**step
        new_p, new_m, new_v = [], [], []
        for p, g, m, v in zip(p_leaves, g_leaves, m_leaves, v_leaves):
            p64, g64 = np.asarray(p, dtype=np.float64), np.asarray(g, dtype=np.float64)
            first = m * self.b1 + g64 * (1.0 - self.b1)
            second = v * self.b2 + (g64 * g64) * (1.0 - self.b2)
            delta = (first / c1) / (np.sqrt(second / c2) + self.eps)
            if self.weight_decay != 0.0:
                delta = delta + self.weight_decay * p64
            new_p.append((p64 - delta * lr).astype(np.asarray(p).dtype))
            new_m.append(first)
            new_v.append(second)
        return rebuild(new_p), {"step": step, "m": rebuild(new_m), "v": rebuild(new_v)}


class Adam(_AdamBase):
    def __init__(self, learning_rate=1e-3, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, *,
                 beta1: float | None = None, beta2: float | None = None, epsilon: float | None = None,
                 clip_norm: float | None = None) -> None:
        self._configure(learning_rate, b1, b2, eps, beta1, beta2, epsilon, clip_norm)


class AdamW(_AdamBase):
    def __init__(self, learning_rate=1e-3, b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8,
                 weight_decay: float = 1e-2, *, beta1: float | None = None, beta2: float | None = None,
                 epsilon: float | None = None, clip_norm: float | None = None) -> None:
        self._configure(learning_rate, b1, b2, eps, beta1, beta2, epsilon, clip_norm)
        weight_decay = float(weight_decay)
        if not (math.isfinite(weight_decay) and weight_decay >= 0):
            raise ValueError("weight_decay must be finite and nonnegative")
        self.weight_decay = weight_decay


class SGD:
    def __init__(self, learning_rate=1e-2, *, clip_norm: float | None = None) -> None:
        self.learning_rate = _learning_rate(learning_rate)
        self.clip_norm = None if clip_norm is None else _positive(clip_norm, "clip_norm")

    def init(self, params: Any):
        return {"step": 0} if callable(self.learning_rate) else None

    def update(self, params: Any, grads: Any, state=None):
        p_leaves, rebuild = tr.flatten(params)
        g_leaves, _ = tr.flatten(grads)
        if callable(self.learning_rate):
            rate = _rate_at(self.learning_rate, state["step"])
            state = {"step": state["step"] + 1}
        else:
            rate = self.learning_rate
        if self.clip_norm is not None:
            clipped, _ = clip_by_global_norm(g_leaves, self.clip_norm)
            g_leaves = list(clipped)
        updated = [(np.asarray(p, dtype=np.float64) - np.asarray(g, dtype=np.float64) * rate)
                   .astype(np.asarray(p).dtype) for p, g in zip(p_leaves, g_leaves)]
        return rebuild(updated), state


def decay_frozen_parameter(value: np.ndarray, weight_decay: float, learning_rate: float) -> np.ndarray:
    """AdamW's decoupled decay of a parameter the loss ignores: gradient and moments are zero, so the
    element rule reduces to p - (0 + weight_decay * p) * learning_rate, evaluated in float64 and rounded
    once to the parameter's dtype every step (decay_frozen_parameters,
    crates/quabla-python/src/tensor_trace.rs:5071-5105; the `0 +` keeps the rule's signed-zero result)."""
    value = np.asarray(value)
    wide = value.astype(np.float64)
    with np.errstate(all="ignore"):
        return (wide - (0.0 + weight_decay * wide) * learning_rate).astype(value.dtype)


class CudaTrainerExecutor:
    """What the reference's `_quabla._cuda_trainer_optimizer(...)` returns
    (crates/quabla-python/src/tensor_trace.rs:5108-5289): `step`, `loss`,
    `parameters`, `learning_rate`, `device_buffer_count` over one device plan."""

    def __init__(self, compiled: CompiledLoss, parameter_names: Sequence[str], inputs: dict,
                 retained_input_names: Sequence[str], *, optimizer: str, learning_rate: float, beta1: float,
                 beta2: float, epsilon: float, weight_decay: float, clip_norm: float | None,
                 precision: str | None = None, device_ordinal: int = 0) -> None:
        if precision not in (None, "float64"):
            raise ValueError(f'precision must be None or "float64", got {precision!r}')
        self._compiled = compiled
        self._plan = compiled.plan
        self._parameter_names = list(parameter_names)
        self._rule = dict(rule=optimizer, beta1=beta1, beta2=beta2, epsilon=epsilon, weight_decay=weight_decay,
                          clip_norm=clip_norm)
        self.learning_rate = learning_rate
        active = {name for name, _, _ in compiled.spec.parameters}
        self._frozen = {}
        for name, value in inputs.items():
            if name in active or name in compiled.data_names:
                self._plan.bind(name, value)
            elif name in self._parameter_names:
                # The loss ignores this parameter: it only decays, on the host, stored in its own dtype
                # (crates/quabla-python/src/tensor_trace.rs:5071-5105).
                self._frozen[name] = np.array(value, dtype=compiled.dtype)
        self._dtype = compiled.dtype
        self._shapes = dict(zip(compiled.param_names, compiled.param_shapes))
        self._active = active

    @property
    def learning_rate(self) -> float:
        return self._learning_rate

    @learning_rate.setter
    def learning_rate(self, value: float) -> None:
        value = float(value)
        if not (math.isfinite(value) and value >= 0):
            raise ValueError("device optimizer learning_rate must be finite and nonnegative")
        self._learning_rate = value

    def _config(self):
        return opt_config(learning_rate=self._learning_rate, **self._rule)

    def step(self, inputs: dict | None = None) -> None:
        config = self._config()
        for name, value in (inputs or {}).items():
            self._plan.bind(name, value)
        self._plan.execute()
        self._plan.optimizer_step(config)
        if self._frozen and self._rule["rule"] == "adam" and self._rule["weight_decay"] != 0.0:
            for name in self._frozen:
                self._frozen[name] = decay_frozen_parameter(self._frozen[name], self._rule["weight_decay"],
                                                            self._learning_rate)

    def loss(self, inputs: dict | None = None) -> np.ndarray:
        for name, value in (inputs or {}).items():
            self._plan.bind(name, value)
        return self._plan.loss()

    def last_value(self) -> np.ndarray:
        """The loss the most recent step computed (at the parameters before its update)."""
        return self._plan.read_output(0)

    def parameters(self) -> dict:
        out = {}
        for name in self._parameter_names:
            if name in self._active:
                out[name] = self._plan.read_input(name, self._shapes[name])
            else:
                out[name] = self._frozen[name].copy()
        return out

    def _moment_layout(self):
        """(name, shape, first element, element count) of every active parameter, in the plan's flat order."""
        layout, offset = [], 0
        for name, _, _ in self._compiled.spec.parameters:
            shape = tuple(self._shapes[name])
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            layout.append((name, shape, offset, count))
            offset += (count + 3) // 4 * 4  # leaves start on 4-element boundaries; the padding stays zero
        return layout

    def export_state(self) -> dict:
        """Optimizer state as host arrays: `{"step": n}` plus, for Adam, `"m"` and `"v"` (name -> array in the
        plan dtype).  One device-to-host read per moment buffer (qb200_plan_read_moments)."""
        from . import _lib

        state: dict = {"step": int(self._plan.query(_lib.Q_STEP_COUNT))}
        if self._rule["rule"] == "adam":
            for key, which in (("m", 0), ("v", 1)):
                flat = self._plan.read_moments(which)
                state[key] = {name: flat[first:first + count].reshape(shape).copy()
                              for name, shape, first, count in self._moment_layout()}
        return state

    def _checked_moments(self, state: dict):
        """The flat moment vectors (or None for SGD) and the step count of a state; raises on any mismatch."""
        step = operator.index(state["step"])
        if step < 0:
            raise ValueError("optimizer step count must be nonnegative")
        if self._rule["rule"] != "adam":
            if "m" in state or "v" in state:
                raise ValueError("this optimizer has no moments")
            return None, step
        from . import _lib

        layout = self._moment_layout()
        total = int(self._plan.query(_lib.Q_PARAMETER_COUNT))
        flats = []
        for key in ("m", "v"):
            moments = state[key]
            if set(moments) != {name for name, _, _, _ in layout}:
                raise ValueError(f'optimizer state "{key}" must hold exactly the trained parameters')
            flat = np.zeros((total,), dtype=self._dtype)
            for name, shape, first, count in layout:
                value = np.asarray(moments[name])
                if value.shape != shape or value.dtype != self._dtype:
                    raise ValueError(f'optimizer state "{key}"["{name}"] must be {self._dtype} of shape {shape}, '
                                     f"got {value.dtype} of shape {value.shape}")
                flat[first:first + count] = value.reshape(-1)
            flats.append(flat)
        return flats, step

    def _checked_parameters(self, values: dict) -> dict:
        checked = {}
        for name, value in values.items():
            value = np.asarray(value)
            if name in self._active:
                if value.shape != tuple(self._shapes[name]) or value.dtype != self._dtype:
                    raise ValueError(f'parameter "{name}" must be {self._dtype} of shape {tuple(self._shapes[name])}, '
                                     f"got {value.dtype} of shape {value.shape}")
            elif name not in self._frozen:
                raise ValueError(f'no parameter named "{name}"')
            checked[name] = value
        return checked

    def import_state(self, state: dict, parameters: dict | None = None) -> None:
        """Inverse of `export_state`, optionally with new parameter values by name.  Names, shapes and dtypes of
        everything are validated first; then the parameters are bound and both moment buffers and the step
        counter uploaded (qb200_plan_write_moments)."""
        flats, step = self._checked_moments(state)
        values = self._checked_parameters(parameters or {})
        for name, value in values.items():
            if name in self._active:
                self._plan.bind(name, value)
            else:
                self._frozen[name] = np.array(value, dtype=self._dtype)
        for which, flat in enumerate(flats or ()):
            self._plan.write_moments(which, flat, step)

    @property
    def device_buffer_count(self) -> int:
        return self._plan.device_buffer_count

    @property
    def plan(self):
        return self._plan


def _cuda_trainer_optimizer(compiled: CompiledLoss, parameter_names, inputs, retained_input_names, **rule):
    """Factory with the argument list of the reference's native factory
    (python/quabla/optim.py:458-487); tests replace it with a fake."""
    return CudaTrainerExecutor(compiled, parameter_names, inputs, retained_input_names, **rule)


class Trainer:
    """Trace `loss(params, *data)` once and keep optimizer state on the device.

    `batch_argnums` indexes the data arguments (excluding parameters);
    `step(*batch)` replaces those arguments in the declared order, an empty
    call reuses the latest batch, `loss()` evaluates the current parameters,
    `params` reads the parameters back (python/quabla/optim.py:351-550).
    """

    def __init__(self, loss: Callable, params: Any, optimizer, *data: Any, device: str = "cuda",
                 batch_argnums: int | Sequence[int] = (), precision: str | None = None) -> None:
        if not callable(loss):
            raise TypeError("loss must be callable")
        if not isinstance(optimizer, (Adam, AdamW, SGD)):
            raise TypeError("optimizer must be Adam, AdamW, or SGD")
        if precision not in (None, "float64"):
            raise ValueError(f'precision must be None or "float64", got {precision!r}')
        _, ordinal = require_device(device, "Trainer")
        leaves, self._rebuild_params = tr.flatten(params)
        if not leaves:
            raise ValueError("optimizer requires at least one parameter")
        if isinstance(batch_argnums, int):
            batch_argnums = (batch_argnums,)
        self._batch_argnums = tuple(operator.index(i) for i in batch_argnums)
        if len(set(self._batch_argnums)) != len(self._batch_argnums):
            raise ValueError("batch_argnums must be distinct")
        if any(i < 0 or i >= len(data) for i in self._batch_argnums):
            raise ValueError("batch_argnums indexes data arguments, excluding params")
        self._data = tuple(data)
        self._optimizer = optimizer
        arguments = (params, *self._data)
        retained = [i + 1 for i in range(len(data)) if i not in self._batch_argnums]
        compiled = CompiledLoss(loss, arguments, (0,), ordinal, retained=retained)
        self._compiled = compiled
        self._parameter_names = compiled.param_names
        self._batch_names = [[n for n, a in zip(compiled.data_names, compiled.data_arg) if a == i + 1]
                             for i in range(len(data))]
        self._batch_specs = []
        for i in self._batch_argnums:
            arrays = [np.asarray(l) for l in tr.flatten(self._data[i])[0] if _is_array(l)]
            self._batch_specs.append([(a.shape, a.dtype) for a in arrays])
        named = dict(zip(compiled.param_names, compiled.leaves_of(arguments)[0]))
        named.update(zip(compiled.data_names, compiled.leaves_of(arguments)[1]))
        if isinstance(optimizer, SGD):
            rule = dict(optimizer="sgd", beta1=0.0, beta2=0.0, epsilon=1.0, weight_decay=0.0)
        else:
            rule = dict(optimizer="adam", beta1=optimizer.b1, beta2=optimizer.b2, epsilon=optimizer.eps,
                        weight_decay=optimizer.weight_decay)
        rule.update(precision=precision, device_ordinal=ordinal)
        retained_names = [n for n, r in zip(compiled.data_names, compiled.data_retained) if r]
        self._executor = _cuda_trainer_optimizer(
            compiled, self._parameter_names, named, retained_names,
            learning_rate=_rate_at(optimizer.learning_rate, 0), clip_norm=optimizer.clip_norm, **rule)
        self._device_steps = 0

    def _device_step(self, *inputs) -> None:
        schedule = self._optimizer.learning_rate
        if callable(schedule):
            self._executor.learning_rate = _rate_at(schedule, self._device_steps)
        result = self._executor.step(*inputs)
        self._device_steps += 1
        return result

    @property
    def params(self) -> Any:
        values = self._executor.parameters()
        return self._rebuild_params([values[name] for name in self._parameter_names])

    def step(self, *batch: Any) -> None:
        if not batch:
            return self._device_step()
        if len(batch) != len(self._batch_argnums):
            raise ValueError("batch argument count must match batch_argnums")
        inputs = {}
        data = list(self._data)
        for value, index, specs in zip(batch, self._batch_argnums, self._batch_specs):
            arrays = [np.asarray(l) for l in tr.flatten(value)[0] if _is_array(l)]
            if len(arrays) != len(specs) or any(a.shape != s or a.dtype != d for a, (s, d) in zip(arrays, specs)):
                raise ValueError("batch shapes and dtypes must match initial data")
            inputs.update(zip(self._batch_names[index], arrays))
            data[index] = value
        result = self._device_step(inputs)
        self._data = tuple(data)
        return result

    def export_state(self) -> dict:
        """Everything a run needs to resume: `{"step", "params", "optimizer"}` as host arrays and Python
        scalars, a tree that `quabla_b200.save` writes as it is.  `params` is the parameter pytree,
        `optimizer` holds the device step counter and, for Adam, both moment buffers by parameter name.
        The reference's Trainer keeps this state inside its native executor and exposes only
        `params` (python/quabla/optim.py:351-550); checkpointing a device run needs the moments too.
        """
        return {"step": self._device_steps, "params": self.params, "optimizer": self._executor.export_state()}

    def import_state(self, state: dict) -> None:
        """Resume from `export_state()` (of a trainer built with the same loss, parameter shapes and
        optimizer rule): the next `step()` continues bit for bit where the exporting run stood."""
        step = operator.index(state["step"])
        if step < 0:
            raise ValueError("step must be nonnegative")
        leaves, _ = tr.flatten(state["params"])
        if len(leaves) != len(self._parameter_names):
            raise ValueError(f"state holds {len(leaves)} parameter arrays, the trainer has {len(self._parameter_names)}")
        self._executor.import_state(state["optimizer"], dict(zip(self._parameter_names, leaves)))
        self._device_steps = step

    def resample(self, index: int, key, bounds: Sequence[tuple[float, float]]) -> None:
        """Redraw batch argument `index` (one array of shape [rows, d]) on the device.

        Column j becomes `random.uniform(random.fold_in(key, j), (rows,), dtype, *bounds[j])`, bit for
        bit, generated by a kernel: no host array is built and nothing is copied to the device.
        The next `step()` without arguments trains on the new batch.  Not part of the reference's
        Trainer, which redraws on the host and passes the batch to `step`
        (python/quabla/optim.py:490-550).
        """
        from . import random as qrandom

        index = operator.index(index)
        if index not in self._batch_argnums:
            raise ValueError("resample takes one of batch_argnums")
        names = self._batch_names[index]
        specs = self._batch_specs[self._batch_argnums.index(index)]
        if len(names) != 1 or len(specs) != 1 or len(specs[0][0]) != 2:
            raise ValueError("resample needs a batch argument that is one array of shape [rows, columns]")
        columns = specs[0][0][1]
        if len(bounds) != columns:
            raise ValueError(f"bounds must have one (minval, maxval) pair per column, {columns} here")
        plan = self._executor.plan
        for j, (low, high) in enumerate(bounds):
            plan.sample_uniform(names[0], j, qrandom.fold_in(key, j), low, high)

    def loss(self):
        return self._executor.loss()

    @property
    def value(self):
        """The loss computed by the most recent `step` (before its update); one
        device-to-host read, no extra evaluation."""
        return self._executor.last_value()
