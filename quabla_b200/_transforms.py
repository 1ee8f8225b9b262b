"""Public transforms: jit, value_and_grad, grad, vmap, hessian, jvp.

Same call shapes as python/quabla/_transforms.py (`_ValueAndGrad` :912-950,
`_Vmap` :1644-1734, hessian :2173-2179, `_Jit` :977-1173).  Called on traced
per-point values the transforms work symbolically (quabla_b200/_trace.py);
called on concrete arrays, `value_and_grad`/`grad`/`jit` compile the loss to a
device plan and run it on a CUDA device.
"""

from __future__ import annotations

import inspect
import math
from collections import OrderedDict
from typing import Any, Callable, Sequence

import numpy as np

from . import _trace as tr
from ._devices import require_device
from ._errors import UnsupportedOperationError
from ._plan import Plan

_MAX_TRACES = 8  # python/quabla/_transforms.py trace cache bound


def _parameter_names(fun: Callable, count: int) -> list[str]:
    names = [f"arg{i}" for i in range(count)]
    try:
        parameters = list(inspect.signature(fun).parameters.values())
    except (TypeError, ValueError):
        return names
    for index, parameter in enumerate(parameters[:count]):
        if parameter.kind not in (parameter.POSITIONAL_ONLY, parameter.POSITIONAL_OR_KEYWORD):
            break
        names[index] = parameter.name
    return names


def _is_array(leaf) -> bool:
    return isinstance(leaf, (np.ndarray, np.generic))


def _any_traced(args) -> bool:
    for arg in args:
        leaves, _ = tr.flatten(arg)
        if any(tr.is_traced(leaf) for leaf in leaves):
            return True
    return False


def _normalize_argnums(argnums, count: int) -> tuple[int, ...]:
    values = (argnums,) if isinstance(argnums, int) else tuple(argnums)
    out = []
    for value in values:
        if not -count <= value < count:
            raise ValueError(f"argnums {value} is out of range for {count} positional arguments")
        out.append(value % count)
    if len(set(out)) != len(out):
        raise ValueError("argnums must be distinct")
    return tuple(out)


class CompiledLoss:
    """A loss traced for given argument signatures and compiled to a device plan.

    Inputs are named by pytree key paths rooted at the loss's parameter names
    (`params/0/w`), as the reference names graph inputs
    (python/quabla/_transforms.py:363-377)."""

    def __init__(self, fun: Callable, args: tuple, argnums: tuple[int, ...], device_ordinal: int,
                 retained: Sequence[int] = (), build_plan: bool = True) -> None:
        roots = _parameter_names(fun, len(args))
        self.argnums = argnums
        self.param_names: list[str] = []
        self.param_shapes: list[tuple[int, ...]] = []
        self.data_names: list[str] = []
        self.data_shapes: list[tuple[int, ...]] = []
        self.data_retained: list[bool] = []
        self.data_arg: list[int] = []
        dtype = None
        call = []
        self._rebuild = []
        for index, (arg, root) in enumerate(zip(args, roots)):
            leaves, rebuild = tr.flatten(arg)
            paths = tr.leaf_paths(arg, root)
            self._rebuild.append(rebuild)
            traced = []
            for leaf, path in zip(leaves, paths):
                if not _is_array(leaf):
                    traced.append(leaf)  # a static Python value
                    continue
                leaf = np.asarray(leaf)
                if leaf.dtype not in (np.float32, np.float64):
                    raise TypeError(f"input '{path}' must be float32 or float64, got {leaf.dtype}")
                if dtype is None:
                    dtype = leaf.dtype
                elif leaf.dtype != dtype:
                    raise UnsupportedOperationError(
                        "mixed float32/float64 programs are rejected: a plan has one floating dtype",
                        op="compile", device="cuda")
                if index in argnums:
                    self.param_names.append(path)
                    self.param_shapes.append(tuple(leaf.shape))
                    traced.append(tr.ParamRef(path, leaf.shape, leaf.dtype))
                else:
                    self.data_names.append(path)
                    self.data_shapes.append(tuple(leaf.shape))
                    self.data_retained.append(index in retained)
                    self.data_arg.append(index)
                    traced.append(tr.data_leaf(path, tuple(leaf.shape), leaf.dtype))
            call.append(rebuild(traced))
        if dtype is None or not self.param_names:
            raise ValueError("the loss needs at least one floating-point parameter array")
        self.dtype = np.dtype(dtype)
        result = fun(*call)
        if isinstance(result, tr.TraceValue):
            raise UnsupportedOperationError(
                "the loss must reduce over the collocation points with mean or sum", op="loss", device="cuda")
        self.spec = tr.build_plan_spec(
            result, list(zip(self.param_names, self.param_shapes)),
            list(zip(self.data_names, self.data_shapes, self.data_retained)), self.dtype)
        # build_plan=False stops after the fusion pass (the description alone
        # needs no device).
        self.plan = Plan(self.spec, device_ordinal) if build_plan else None
        self._active = {name: i for i, (name, _, _) in enumerate(self.spec.parameters)}

    # -- running --------------------------------------------------------------
    def named_inputs(self, args: tuple) -> dict:
        """Every array leaf of `args` under its input name."""
        params, data = self.leaves_of(args)
        named = dict(zip(self.param_names, params))
        named.update(zip(self.data_names, data))
        return named

    def leaves_of(self, args: tuple) -> tuple[list, list]:
        params, data = [], []
        for index, arg in enumerate(args):
            leaves, _ = tr.flatten(arg)
            arrays = [np.asarray(leaf) for leaf in leaves if _is_array(leaf)]
            (params if index in self.argnums else data).extend(arrays)
        return params, data

    def bind(self, args: tuple, skip_retained_bound: bool = False) -> None:
        params, data = self.leaves_of(args)
        for name, value in zip(self.param_names, params):
            if name in self._active:
                self.plan.bind(name, value)
        for name, value in zip(self.data_names, data):
            self.plan.bind(name, value)

    def gradients(self, args: tuple):
        """(value, grads) with grads shaped like the differentiated arguments."""
        outputs = self.plan.outputs()
        value = outputs[0]
        flat = []
        for name, shape in zip(self.param_names, self.param_shapes):
            if name in self._active:
                flat.append(outputs[1 + self._active[name]].reshape(shape))
            else:
                # A parameter the loss ignores has a zero gradient
                # (crates/quabla-python/src/tensor_trace.rs:5351-5363).
                flat.append(np.zeros(shape, dtype=self.dtype))
        it = iter(flat)
        trees = []
        for index in self.argnums:
            leaves, rebuild = tr.flatten(args[index])
            trees.append(rebuild([next(it) if _is_array(leaf) else None for leaf in leaves]))
        return value, trees


def _signature(args: tuple, argnums, device) -> tuple:
    parts = []
    for arg in args:
        leaves, _ = tr.flatten(arg)
        paths = tuple(tr.leaf_paths(arg, ""))
        parts.append((paths, tuple((tuple(np.shape(l)), str(np.asarray(l).dtype)) if _is_array(l) else ("static", l)
                                   for l in leaves)))
    return (tuple(parts), argnums, device)


class _Transform:
    def __init__(self, fun: Callable) -> None:
        if not callable(fun):
            raise TypeError("a transform requires a callable")
        self._fun = fun
        self._cache: OrderedDict = OrderedDict()

    def _lookup(self, key, build):
        found = self._cache.get(key)
        if found is not None:
            self._cache.move_to_end(key)
            return found
        built = build()
        self._cache[key] = built
        while len(self._cache) > _MAX_TRACES:
            _, evicted = self._cache.popitem(last=False)
            evicted.plan.close()
        return built


class _ValueAndGrad(_Transform):
    def __init__(self, fun: Callable, argnums=0, mode: str = "value_and_grad") -> None:
        super().__init__(fun)
        self._argnums = argnums
        self._mode = mode

    def __call__(self, *args):
        if _any_traced(args):
            if not isinstance(self._argnums, int):
                raise UnsupportedOperationError("a nested grad differentiates one argument", op="grad", device="cuda")
            argnum = self._argnums % len(args)
            value, grads = tr.symbolic_value_and_grad(self._fun, argnum, args)
            return grads if self._mode == "grad" else (value, grads)
        return self._run(args, 0)

    def _run(self, args: tuple, device_ordinal: int):
        argnums = _normalize_argnums(self._argnums, len(args))
        key = _signature(args, argnums, device_ordinal)
        compiled = self._lookup(key, lambda: CompiledLoss(self._fun, args, argnums, device_ordinal))
        compiled.bind(args)
        compiled.plan.execute()
        value, trees = compiled.gradients(args)
        grads = trees[0] if isinstance(self._argnums, int) else tuple(trees)
        return grads if self._mode == "grad" else (value, grads)


class _LossOnly(_Transform):
    """jit(loss): forward evaluation of the loss on the device."""

    def _run(self, args: tuple, device_ordinal: int):
        key = _signature(args, (0,), device_ordinal)
        compiled = self._lookup(key, lambda: CompiledLoss(self._fun, args, (0,), device_ordinal))
        compiled.bind(args)
        return compiled.plan.loss()

    def __call__(self, *args):
        if _any_traced(args):
            return self._fun(*args)
        return self._run(args, 0)


class _Jit:
    def __init__(self, fun: Callable, device: str | None = None, precision: str | None = None) -> None:
        if precision not in (None, "float64"):
            raise ValueError(f'precision must be None or "float64", got {precision!r}')
        _, self._ordinal = require_device(device, "jit")
        self._inner = fun if isinstance(fun, (_ValueAndGrad, _LossOnly)) else _LossOnly(fun)
        self.__wrapped__ = fun

    def __call__(self, *args, **kwargs):
        if kwargs:
            raise TypeError("jit-compiled losses take positional arguments only")
        if _any_traced(args):
            return self._inner(*args)
        return self._inner._run(args, self._ordinal)


class _Vmap:
    def __init__(self, fun: Callable, in_axes=0) -> None:
        self._fun = fun
        self._in_axes = in_axes

    def __call__(self, *args):
        if not _any_traced(args):
            raise UnsupportedOperationError(
                "vmap runs inside a traced loss; evaluating a vmapped function on concrete arrays is outside the "
                "training step this backend implements", op="vmap", device="cuda")
        return tr.symbolic_vmap(self._fun, self._in_axes, args)


class _Hessian:
    def __init__(self, fun: Callable, argnums: int = 0) -> None:
        self._fun = fun
        self._argnums = argnums

    def __call__(self, *args):
        if not _any_traced(args):
            raise UnsupportedOperationError("hessian runs inside a traced loss", op="hessian", device="cuda")
        return tr.symbolic_hessian(self._fun, self._argnums % len(args), args)


def jit(fun: Callable, *, device: str | None = None, precision: str | None = None) -> Callable:
    """Compile `fun` (a loss, or value_and_grad/grad of one) for a CUDA device."""
    return _Jit(fun, device, precision)


def value_and_grad(fun: Callable, argnums=0) -> Callable:
    return _ValueAndGrad(fun, argnums, "value_and_grad")


def grad(fun: Callable, argnums=0) -> Callable:
    return _ValueAndGrad(fun, argnums, "grad")


def vmap(fun: Callable, in_axes=0) -> Callable:
    return _Vmap(fun, in_axes)


def hessian(fun: Callable, argnums: int = 0) -> Callable:
    return _Hessian(fun, argnums)


def jvp(fun: Callable, primals, tangents):
    primals, tangents = tuple(primals), tuple(tangents)
    if not _any_traced(primals):
        raise UnsupportedOperationError("jvp runs inside a traced loss", op="jvp", device="cuda")
    return tr.symbolic_jvp(fun, primals, tangents)


# -- array functions on traced values ----------------------------------------
def _unary(kind: str, numpy_function: Callable) -> Callable:
    def apply(x):
        if isinstance(x, tr.TraceValue):
            return x._unary(kind)
        if isinstance(x, tr.ParamRef):
            return x._reject()
        return numpy_function(x)

    apply.__name__ = kind
    return apply


tanh = _unary("tanh", np.tanh)
sin = _unary("sin", np.sin)
cos = _unary("cos", np.cos)
exp = _unary("exp", np.exp)
log = _unary("log", np.log)
sqrt = _unary("sqrt", np.sqrt)
log1p = _unary("log1p", np.log1p)
expm1 = _unary("expm1", np.expm1)
tan = _unary("tan", np.tan)
erf = _unary("erf", np.vectorize(math.erf, otypes=[np.float64]))
erfc = _unary("erfc", np.vectorize(math.erfc, otypes=[np.float64]))


def _host_sigmoid(x):
    x = np.asarray(x, dtype=np.float64)
    e = np.exp(-np.abs(x))
    return np.where(x > 0, 1.0 / (1.0 + e), e / (1.0 + e))


def _host_gelu(x):
    x = np.asarray(x, dtype=np.float64)
    tail = np.abs(x) > 40.0
    safe = np.where(tail, 0.0, x)
    value = safe * _host_sigmoid(safe * (safe * safe * 0.044715 + 1.0) * (2.0 * math.sqrt(2.0 / math.pi)))
    return np.where(tail, np.where(x > 0.0, x, -0.0), value)


# Hidden-layer activations beyond tanh and sin, with the reference's definitions: sigmoid and softplus
# (crates/quabla-python/src/composite.rs:178-209), silu and the tanh-approximated gelu
# (python/quabla/_ops.py:475-505).  On traced values they are recognised as the activation of a layer.
sigmoid = _unary("sigmoid", _host_sigmoid)
softplus = _unary("softplus", lambda x: np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x))))
silu = _unary("silu", lambda x: np.asarray(x) * _host_sigmoid(x))
gelu = _unary("gelu", _host_gelu)


def mean(x, axis=None):
    if isinstance(x, tr.TraceValue):
        return x.mean(axis)
    return np.mean(x, axis=axis)


def sum(x, axis=None):  # noqa: A001 - mirrors quabla.sum
    if isinstance(x, tr.TraceValue):
        return x.sum(axis)
    return np.sum(x, axis=axis)


def trace(x):
    """Sum of the diagonal of a per-point matrix (python/quabla/_ops.py:997-1027)."""
    if isinstance(x, tr.TraceValue):
        if x.batch is not None:
            a = x.array()
            if a.ndim != 2 or a.shape[0] != a.shape[1]:
                raise ValueError("trace requires square matrices")
            return x._like(np.asarray(np.trace(a), dtype=object).reshape(()))
        a = x.array()
        if a.ndim != 2 or a.shape[0] != a.shape[1]:
            raise ValueError("trace requires a square matrix")
        cell = np.empty((), dtype=object)
        cell[()] = np.trace(a)
        return x._like(cell)
    return np.trace(x)


def stack(values, axis: int = 0):
    if any(isinstance(v, tr.TraceValue) for v in values):
        first = next(v for v in values if isinstance(v, tr.TraceValue))
        if first.batch is not None:
            raise UnsupportedOperationError("stack of batched values", op="stack", device="cuda")
        arrays = [v.array() if isinstance(v, tr.TraceValue) else np.asarray(v, dtype=object) for v in values]
        return first._like(np.stack(arrays, axis=axis))
    return np.stack(values, axis=axis)


def reshape(x, shape):
    return x.reshape(shape)
