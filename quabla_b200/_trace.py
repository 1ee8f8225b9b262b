"""Tracer and fusion pass: from a Python loss to a PlanSpec.

The reference traces a loss into a tensor program, expands `grad`/`vmap`/
`hessian` by graph transforms and lowers every node to a kernel
(python/quabla/_transforms.py:825-950, 1644-1758, 1812-2036;
crates/quabla-core/src/tensor_ir.rs:2612-2690, 3359-3906).  This tracer keeps
the structure instead of expanding it:

* a value inside `vmap` is a small array of per-point symbolic expressions
  (`_symbolic.Expr`);
* `x @ w + b` and `tanh` on such values build a lazy description of the MLP
  (`_Pending`), which becomes a `NetJet` leaf when its scalar output is used;
* `grad`, `hessian` and `jvp` differentiate the per-point expressions
  symbolically; differentiating a `NetJet` raises its derivative word, which
  the device kernels realise as one more stream of the Taylor jet;
* `mean`/`sum` over the batch axis produce loss terms.

`build_plan_spec` then groups the loss terms into point sets and compiles the
residual programs.  Anything outside this family raises
UnsupportedOperationError: there is no fallback path.
"""

from __future__ import annotations

import itertools
import math
import os
from typing import Any, Callable

import numpy as np

from . import _lib
from . import _symbolic as sx
from ._errors import UnsupportedOperationError
from ._plan import PlanSpec, SetSpec

_fresh = itertools.count()


def _unsupported(message: str, op: str = "trace") -> UnsupportedOperationError:
    return UnsupportedOperationError(message, op=op, device="cuda")


# --------------------------------------------------------------------------
# Parameters and networks
# --------------------------------------------------------------------------
class ParamRef:
    """A parameter leaf seen by the tracer (a replicated, differentiated input)."""

    __array_priority__ = 1000
    __array_ufunc__ = None  # NumPy operands defer to the reflected methods here

    def __init__(self, name: str, shape: tuple[int, ...], dtype, stored_shape=None) -> None:
        self.name = name
        self.shape = tuple(shape)
        self.dtype = np.dtype(dtype)
        self.stored_shape = tuple(shape) if stored_shape is None else stored_shape

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def reshape(self, *shape) -> "ParamRef":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = _resolve_shape(shape, int(np.prod(self.shape, dtype=np.int64)))
        return ParamRef(self.name, shape, self.dtype, self.stored_shape)

    def astype(self, dtype) -> "ParamRef":
        if np.dtype(dtype) != self.dtype:
            raise _unsupported("a plan has one floating dtype; casting a parameter is not supported", "astype")
        return self

    def _reject(self, *_):
        raise _unsupported(
            f"parameter '{self.name}' is used outside the Linear+tanh pattern (x @ w + b, tanh) "
            "that the fused kernels implement")

    __mul__ = __rmul__ = __sub__ = __rsub__ = __truediv__ = __rtruediv__ = __neg__ = __pow__ = _reject
    __matmul__ = __getitem__ = _reject

    def __add__(self, other):
        if isinstance(other, TraceValue):
            return other.__add__(self)
        return self._reject()

    __radd__ = __add__

    def __rmatmul__(self, other):
        return as_trace(other).__matmul__(self)


def _resolve_shape(shape: tuple, total: int) -> tuple[int, ...]:
    shape = tuple(int(s) for s in shape)
    if shape.count(-1) > 1:
        raise ValueError("reshape accepts at most one -1")
    if -1 in shape:
        known = int(np.prod([s for s in shape if s != -1], dtype=np.int64))
        if known == 0 or total % known:
            raise ValueError(f"cannot reshape {total} elements into {shape}")
        shape = tuple(total // known if s == -1 else s for s in shape)
    if int(np.prod(shape, dtype=np.int64)) != total:
        raise ValueError(f"cannot reshape {total} elements into {shape}")
    return shape


class Network:
    """An MLP applied to per-point inputs: layers of (weight, bias, d_in, d_out),
    tanh between them, linear last layer; `inputs` are the per-point expressions
    feeding the first layer."""

    __slots__ = ("layers", "inputs", "activation", "_hash")

    def __init__(self, layers: tuple, inputs: tuple, activation: str = "tanh") -> None:
        self.layers = tuple(layers)
        self.inputs = tuple(inputs)
        self.activation = activation
        self._hash = hash((self.layers, self.inputs, self.activation))

    def __hash__(self) -> int:
        return self._hash

    def __eq__(self, other) -> bool:
        return (isinstance(other, Network) and self.layers == other.layers and self.inputs == other.inputs
                and self.activation == other.activation)

    def __repr__(self) -> str:
        return f"Network({[l[2] for l in self.layers] + [self.layers[-1][3]]})"

    def substituted(self, mapping: dict) -> "Network":
        return Network(self.layers, tuple(sx.substitute(e, mapping) for e in self.inputs), self.activation)

    def direction(self, variable: sx.Expr) -> tuple[float, ...]:
        """d(inputs)/d(variable), which must be constant (affine input maps)."""
        out = []
        for e in self.inputs:
            d = sx.derivative(e, lambda leaf: sx.ONE if leaf is variable else sx.ZERO)
            if not sx.is_const(d):
                raise _unsupported("the network input must be an affine function of the differentiation variable",
                                   "grad")
            out.append(d.args[0])
        return tuple(out)


def _cells(value):
    """NumPy returns a bare object for 0-d results; keep them as 0-d arrays."""
    if isinstance(value, (np.ndarray, _Pending)):
        return value
    cell = np.empty((), dtype=object)
    cell[()] = value
    return cell


class _Pending:
    """A per-point MLP prefix that has not been reduced to a scalar yet."""

    def __init__(self, layers: list, inputs: tuple, activated: bool, shape: tuple[int, ...],
                 activation: str | None = None) -> None:
        self.layers = layers        # [[w_name, b_name, d_in, d_out], ...]
        self.inputs = inputs
        self.activated = activated  # the activation already applied to the last layer
        self.shape = shape
        self.activation = activation  # the hidden layers' activation, once one has been applied

    @property
    def width(self) -> int:
        return self.layers[-1][3]

    def finalize(self) -> np.ndarray:
        if self.activated or self.width != 1:
            raise _unsupported(
                "a hidden layer of the network is used outside x @ w + b / tanh; only the scalar output of the "
                "last linear layer can enter the residual")
        network = Network(tuple(tuple(l) for l in self.layers), self.inputs, self.activation or "tanh")
        out = np.empty(self.shape, dtype=object)
        out[...] = sx.net(network, ())
        return out


# --------------------------------------------------------------------------
# Traced values
# --------------------------------------------------------------------------
class TraceValue:
    """A traced array: per-point expressions, optionally with a leading batch axis."""

    __array_priority__ = 2000
    __array_ufunc__ = None  # NumPy operands defer to the reflected methods here

    def __init__(self, inner, batch: int | None, dtype) -> None:
        self.inner = inner
        self.batch = batch
        self.dtype = np.dtype(dtype)

    # -- structure ----------------------------------------------------------
    @property
    def point_shape(self) -> tuple[int, ...]:
        return tuple(self.inner.shape)

    @property
    def shape(self) -> tuple[int, ...]:
        return self.point_shape if self.batch is None else (self.batch,) + self.point_shape

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def array(self) -> np.ndarray:
        """The per-point expressions, finalising a pending network output."""
        if isinstance(self.inner, _Pending):
            self.inner = self.inner.finalize()
        return self.inner

    def _like(self, inner) -> "TraceValue":
        return TraceValue(_cells(inner), self.batch, self.dtype)

    def reshape(self, *shape) -> "TraceValue":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = tuple(int(s) for s in shape)
        if self.batch is not None:
            if not shape or shape[0] not in (self.batch, -1) or -1 in shape[1:] and shape[0] == -1:
                raise _unsupported("a reshape must keep the batch axis", "reshape")
            point = _resolve_shape(shape[1:], int(np.prod(self.point_shape, dtype=np.int64)))
        else:
            point = _resolve_shape(shape, int(np.prod(self.point_shape, dtype=np.int64)))
        if isinstance(self.inner, _Pending):
            p = self.inner
            return self._like(_Pending(p.layers, p.inputs, p.activated, point, p.activation))
        return self._like(self.inner.reshape(point))

    def astype(self, dtype) -> "TraceValue":
        if np.dtype(dtype) != self.dtype:
            raise _unsupported("a plan has one floating dtype; casts inside the loss are not supported", "astype")
        return self

    def __getitem__(self, index) -> "TraceValue":
        if not isinstance(index, tuple):
            index = (index,)
        if self.batch is not None:
            first, index = index[0], index[1:]
            if not (isinstance(first, slice) and first == slice(None)) and first is not Ellipsis:
                raise _unsupported("indexing the batch axis is not supported; use vmap", "getitem")
            if first is Ellipsis:
                index = (Ellipsis,) + index
        picked = self.array()[index] if index else self.array()
        if not isinstance(picked, np.ndarray):
            cell = np.empty((), dtype=object)
            cell[()] = picked
            picked = cell
        return self._like(picked)

    @property
    def T(self) -> "TraceValue":
        if self.batch is not None:
            raise _unsupported("transposing across the batch axis is not supported", "transpose")
        return self._like(self.array().T)

    # -- arithmetic ---------------------------------------------------------
    def _binary(self, other, op: Callable, reverse: bool = False) -> "TraceValue":
        if isinstance(other, ParamRef):
            return other._reject()
        batch = self.batch
        if isinstance(other, TraceValue):
            if other.dtype != self.dtype:
                raise _unsupported("mixed float32/float64 programs are rejected", "binary")
            if batch is None:
                batch = other.batch
            elif other.batch is not None and other.batch != batch:
                raise ValueError(f"batch sizes {batch} and {other.batch} do not match")
            rhs = other.array()
            # Align per-point shapes under batch-level broadcasting rules.
            if self.batch is None and other.batch is not None and self.point_shape != ():
                raise _unsupported("broadcasting an unbatched array against a batch is not supported", "binary")
        elif isinstance(other, np.ndarray):
            if other.shape != () and batch is not None:
                raise _unsupported("combine a batch with per-point data through an argument, not a closure",
                                   "binary")
            rhs = other.astype(object) if other.shape != () else float(other)
        elif isinstance(other, (int, float)) and not isinstance(other, bool):
            rhs = float(other)
        else:
            return NotImplemented
        lhs = self.array()
        result = op(rhs, lhs) if reverse else op(lhs, rhs)
        if not isinstance(result, np.ndarray):
            cell = np.empty((), dtype=object)
            cell[()] = result
            result = cell
        return TraceValue(result, batch, self.dtype)

    def __add__(self, other):
        if isinstance(other, ParamRef) and isinstance(self.inner, _Pending):
            return self._add_bias(other)
        return self._binary(other, np.add)

    def __radd__(self, other):
        if isinstance(other, ParamRef) and isinstance(self.inner, _Pending):
            return self._add_bias(other)
        return self._binary(other, np.add, True)

    def __sub__(self, other):
        return self._binary(other, np.subtract)

    def __rsub__(self, other):
        return self._binary(other, np.subtract, True)

    def __mul__(self, other):
        return self._binary(other, np.multiply)

    def __rmul__(self, other):
        return self._binary(other, np.multiply, True)

    def __truediv__(self, other):
        return self._binary(other, np.true_divide)

    def __rtruediv__(self, other):
        return self._binary(other, np.true_divide, True)

    def __neg__(self):
        return self._like(-self.array())

    def __pos__(self):
        return self

    def __pow__(self, exponent):
        if isinstance(exponent, TraceValue):
            raise _unsupported("only integer powers are supported", "pow")
        return self._like(self.array() ** exponent)

    def _add_bias(self, bias: ParamRef) -> "TraceValue":
        p = self.inner
        if p.activated or p.layers[-1][1] is not None:
            raise _unsupported("a bias is added after the linear map and before tanh, once per layer", "add")
        if int(np.prod(bias.shape, dtype=np.int64)) != p.width or (bias.shape and bias.shape[-1] != p.width):
            raise ValueError(f"bias '{bias.name}' of shape {bias.shape} does not match layer width {p.width}")
        layers = [list(l) for l in p.layers]
        layers[-1][1] = bias.name
        return self._like(_Pending(layers, p.inputs, False, p.shape, p.activation))

    def __matmul__(self, weight):
        if not isinstance(weight, ParamRef):
            raise _unsupported("matmul is supported between a per-point activation and a parameter matrix", "matmul")
        if weight.ndim != 2:
            raise _unsupported("the weight of a layer must be a matrix [in, out]", "matmul")
        d_in, d_out = weight.shape
        if isinstance(self.inner, _Pending):
            p = self.inner
            if not p.activated:
                raise _unsupported("two linear maps in a row without tanh between them", "matmul")
            if p.width != d_in or not p.shape or p.shape[-1] != d_in:
                raise ValueError(f"matmul of a width-{p.width} activation with '{weight.name}' {weight.shape}")
            layers = [list(l) for l in p.layers] + [[weight.name, None, d_in, d_out]]
            return self._like(_Pending(layers, p.inputs, False, p.shape[:-1] + (d_out,), p.activation))
        a = self.array()
        # A rank-1 operand is a row vector (python/quabla/_ops.py:366-387).
        if a.ndim == 0 or a.shape[-1] != d_in or int(np.prod(a.shape[:-1], dtype=np.int64)) != 1:
            raise _unsupported(
                f"the first layer takes one point of shape [{d_in}] or [1, {d_in}], got {list(a.shape)}", "matmul")
        inputs = tuple(a.reshape(-1))
        return self._like(_Pending([[weight.name, None, d_in, d_out]], inputs, False, a.shape[:-1] + (d_out,)))

    def _unary(self, kind: str) -> "TraceValue":
        if kind in _lib.ACTIVATIONS and isinstance(self.inner, _Pending) and not self.inner.activated:
            p = self.inner
            if p.activation not in (None, kind):
                raise _unsupported(f"one network mixes {p.activation} and {kind} activations; hidden layers share one",
                                   kind)
            return self._like(_Pending(p.layers, p.inputs, True, p.shape, kind))
        if kind in ("sigmoid", "softplus", "silu", "gelu"):
            raise _unsupported(f"{kind} is supported as the activation of a hidden layer (applied to h @ w + b), "
                               "not inside a residual expression", kind)
        a = self.array()
        out = np.empty(a.shape, dtype=object)
        flat_in, flat_out = a.reshape(-1), out.reshape(-1)
        for i in range(flat_in.size):
            flat_out[i] = sx.unary(kind, flat_in[i])
        return self._like(out)

    def _reduce(self, kind: str, axis=None):
        if axis is not None and self.batch is not None:
            axes = (axis,) if isinstance(axis, int) else tuple(axis)
            axes = tuple(a % self.ndim for a in axes)
            if 0 in axes:
                raise _unsupported("reduce over the batch axis only as a full mean or sum", kind)
            reduced = self.array().sum(axis=tuple(a - 1 for a in axes))
            if kind == "mean":
                reduced = reduced * (1.0 / np.prod([self.shape[a] for a in axes]))
            return self._like(np.asarray(reduced, dtype=object))
        if self.batch is None:
            a = self.array()
            total = a.sum(axis=axis)
            if kind == "mean":
                count = a.size if axis is None else np.prod([a.shape[i] for i in np.atleast_1d(axis)])
                total = total * (1.0 / count)
            cell = np.empty(np.shape(total), dtype=object)
            cell[...] = total
            return self._like(cell)
        flat = self.array().reshape(-1)
        expr = flat[0]
        for e in flat[1:]:
            expr = expr + e
        count = self.batch * flat.size
        return LossValue([(1.0 / count if kind == "mean" else 1.0, self.batch, sx.as_expr(expr))], 0.0, self.dtype)

    def sum(self, axis=None):
        return self._reduce("sum", axis)

    def mean(self, axis=None):
        return self._reduce("mean", axis)

    def item(self):
        raise _unsupported("a traced value has no concrete value", "item")


class LossValue:
    """A scalar: a linear combination of batch reductions of per-point expressions."""

    __array_ufunc__ = None

    def __init__(self, terms: list, constant: float, dtype) -> None:
        self.terms = terms  # [(weight, batch, Expr)]
        self.constant = constant
        self.dtype = np.dtype(dtype)
        self.shape = ()

    def _scaled(self, factor: float) -> "LossValue":
        return LossValue([(w * factor, b, e) for w, b, e in self.terms], self.constant * factor, self.dtype)

    def __add__(self, other):
        if isinstance(other, LossValue):
            if other.dtype != self.dtype:
                raise _unsupported("mixed float32/float64 programs are rejected", "add")
            return LossValue(self.terms + other.terms, self.constant + other.constant, self.dtype)
        if isinstance(other, (int, float)) and not isinstance(other, bool):
            return LossValue(self.terms, self.constant + float(other), self.dtype)
        return NotImplemented

    __radd__ = __add__

    def __neg__(self):
        return self._scaled(-1.0)

    def __sub__(self, other):
        if isinstance(other, (LossValue, int, float)):
            return self + (-other)
        return NotImplemented

    def __rsub__(self, other):
        return (-self) + other

    def __mul__(self, other):
        if isinstance(other, (int, float)) and not isinstance(other, bool):
            return self._scaled(float(other))
        raise _unsupported("a loss term can be scaled by a Python number only", "mul")

    __rmul__ = __mul__

    def __truediv__(self, other):
        if isinstance(other, (int, float)) and not isinstance(other, bool):
            return self._scaled(1.0 / float(other))
        raise _unsupported("a loss term can be divided by a Python number only", "div")

    def reshape(self, *shape):
        return self


def as_trace(value) -> TraceValue:
    if isinstance(value, TraceValue):
        return value
    raise _unsupported(f"expected a traced array, got {type(value).__name__}")


def is_traced(value) -> bool:
    return isinstance(value, (TraceValue, ParamRef, LossValue))


def data_leaf(name: str, shape: tuple[int, ...], dtype) -> TraceValue:
    """The tracer of a data input [batch, ...]: its per-point entries are table columns."""
    if not shape:
        raise _unsupported(f"data input '{name}' is a scalar; pass per-point data with a leading batch axis")
    point = tuple(shape[1:])
    cells = np.empty(point, dtype=object)
    flat = cells.reshape(-1)
    for i in range(flat.size):
        flat[i] = sx.sym(("col", name, i))
    return TraceValue(cells, int(shape[0]), dtype)


# --------------------------------------------------------------------------
# Symbolic transforms on per-point values
# --------------------------------------------------------------------------
def _point_scalar(value, what: str) -> sx.Expr:
    if isinstance(value, TraceValue):
        if value.batch is not None:
            raise _unsupported(f"{what} of a batched value; wrap the per-point function in vmap", what)
        a = value.array()
        if a.size != 1:
            raise ValueError(f"{what} requires a scalar output, got shape {list(a.shape)}")
        return sx.as_expr(a.reshape(-1)[0])
    if isinstance(value, (int, float)) and not isinstance(value, bool):
        return sx.const(value)
    raise _unsupported(f"{what} requires a scalar traced output, got {type(value).__name__}", what)


def _lift_rule(variable: sx.Expr) -> Callable[[sx.Expr], sx.Expr]:
    def rule(leaf: sx.Expr) -> sx.Expr:
        if leaf.kind == "sym":
            return sx.ONE if leaf is variable else sx.ZERO
        network, word = leaf.args
        direction = network.direction(variable)
        if not any(direction):
            return sx.ZERO
        return sx.net(network, word + (direction,))

    return rule


class _Variables:
    """Fresh differentiation variables standing in for a per-point argument."""

    def __init__(self, argument: TraceValue) -> None:
        if argument.batch is not None:
            raise _unsupported("differentiate with respect to one point; wrap the function in vmap", "grad")
        self.source = argument.array()
        tag = next(_fresh)
        self.cells = np.empty(self.source.shape, dtype=object)
        flat = self.cells.reshape(-1)
        for i in range(flat.size):
            flat[i] = sx.sym(("var", tag, i))
        self.value = TraceValue(self.cells, None, argument.dtype)
        self.mapping = {v: sx.as_expr(s) for v, s in zip(flat, self.source.reshape(-1))}

    def restore(self, e: sx.Expr) -> sx.Expr:
        return sx.substitute(e, self.mapping)


def symbolic_value_and_grad(fun: Callable, argnum: int, args: tuple):
    variables = _Variables(as_trace(args[argnum]))
    call = list(args)
    call[argnum] = variables.value
    value = _point_scalar(fun(*call), "grad")
    grads = np.empty(variables.cells.shape, dtype=object)
    flat_v, flat_g = variables.cells.reshape(-1), grads.reshape(-1)
    for i in range(flat_v.size):
        flat_g[i] = variables.restore(sx.derivative(value, _lift_rule(flat_v[i])))
    dtype = args[argnum].dtype
    cell = np.empty((), dtype=object)
    cell[()] = variables.restore(value)
    return TraceValue(cell, None, dtype), TraceValue(grads, None, dtype)


def symbolic_hessian(fun: Callable, argnum: int, args: tuple) -> TraceValue:
    variables = _Variables(as_trace(args[argnum]))
    call = list(args)
    call[argnum] = variables.value
    value = _point_scalar(fun(*call), "hessian")
    flat_v = variables.cells.reshape(-1)
    n = flat_v.size
    first = [sx.derivative(value, _lift_rule(v)) for v in flat_v]
    out = np.empty((n, n), dtype=object)
    for i in range(n):
        for j in range(n):
            out[i, j] = variables.restore(sx.derivative(first[i], _lift_rule(flat_v[j])))
    shape = variables.cells.shape
    return TraceValue(out.reshape(shape + shape), None, args[argnum].dtype)


def symbolic_jvp(fun: Callable, primals: tuple, tangents: tuple):
    """(outputs, tangents of the outputs) of `fun` at the per-point `primals` along `tangents`; the
    outputs may be any pytree of per-point arrays (python/quabla/_transforms.py:1273-1361)."""
    if len(primals) != len(tangents):
        raise ValueError("jvp requires one tangent per primal")
    variables = [_Variables(as_trace(p)) for p in primals]
    weights = []
    for v, tangent in zip(variables, tangents):
        t = tangent.array() if isinstance(tangent, TraceValue) else tangent
        weights.append(np.broadcast_to(np.asarray(t, dtype=object), v.cells.shape).reshape(-1))
    dtype = primals[0].dtype

    def restore(e: sx.Expr) -> sx.Expr:
        for v in variables:
            e = v.restore(e)
        return e

    leaves, rebuild = _flatten(fun(*[v.value for v in variables]))
    out_values, out_tangents = [], []
    for leaf in leaves:
        if isinstance(leaf, (int, float)) and not isinstance(leaf, bool):
            cells = np.empty((), dtype=object)
            cells[()] = sx.const(leaf)
        else:
            leaf = as_trace(leaf)
            if leaf.batch is not None:
                raise _unsupported("jvp of a batched value; wrap the per-point function in vmap", "jvp")
            cells = leaf.array()
        value_cells = np.empty(cells.shape, dtype=object)
        tangent_cells = np.empty(cells.shape, dtype=object)
        flat_in, flat_v, flat_t = cells.reshape(-1), value_cells.reshape(-1), tangent_cells.reshape(-1)
        for i in range(flat_in.size):
            value = sx.as_expr(flat_in[i])
            total = sx.ZERO
            for v, t in zip(variables, weights):
                for cell, weight in zip(v.cells.reshape(-1), t):
                    total = total + sx.as_expr(weight) * sx.derivative(value, _lift_rule(cell))
            flat_v[i], flat_t[i] = restore(value), restore(total)
        out_values.append(TraceValue(value_cells, None, dtype))
        out_tangents.append(TraceValue(tangent_cells, None, dtype))
    return rebuild(out_values), rebuild(out_tangents)


def symbolic_vmap(fun: Callable, in_axes, args: tuple):
    if isinstance(in_axes, int) or in_axes is None:
        in_axes = (in_axes,) * len(args)
    if len(in_axes) != len(args):
        raise ValueError("in_axes must match the positional arguments")
    batch = None
    call = []
    for axis, arg in zip(in_axes, args):
        if axis is None:
            call.append(arg)
            continue
        if axis != 0:
            raise _unsupported("vmap maps axis 0 only", "vmap")
        leaves_in, rebuild = _flatten(arg)
        mapped = []
        for leaf in leaves_in:
            leaf = as_trace(leaf)
            if leaf.batch is None:
                raise _unsupported("nested vmap is not supported", "vmap")
            if batch is not None and leaf.batch != batch:
                raise ValueError("vmap arguments must share the mapped axis size")
            batch = leaf.batch
            mapped.append(TraceValue(leaf.inner, None, leaf.dtype))
        call.append(rebuild(mapped))
    if batch is None:
        raise ValueError("vmap needs at least one mapped argument")
    result = fun(*call)
    leaves_out, rebuild = _flatten(result)
    lifted = []
    for leaf in leaves_out:
        if isinstance(leaf, (int, float)):
            cell = np.empty((), dtype=object)
            cell[()] = sx.const(leaf)
            leaf = TraceValue(cell, None, np.float64)
        leaf = as_trace(leaf)
        if leaf.batch is not None:
            raise _unsupported("the vmapped function returned a batched value", "vmap")
        lifted.append(TraceValue(leaf.inner, batch, leaf.dtype))
    return rebuild(lifted)


# --------------------------------------------------------------------------
# Pytrees (dict / list / tuple of leaves), with the reference's leaf names
# (python/quabla/_transforms.py:363-377: key paths rooted at parameter names).
# --------------------------------------------------------------------------
def _flatten(tree) -> tuple[list, Callable[[list], Any]]:
    leaves: list = []

    def walk(node):
        if isinstance(node, dict):
            keys = sorted(node)
            subs = [walk(node[k]) for k in keys]
            return lambda it: {k: s(it) for k, s in zip(keys, subs)}
        if isinstance(node, (list, tuple)) and not hasattr(node, "_fields"):
            subs = [walk(child) for child in node]
            kind = type(node)
            return lambda it: kind(s(it) for s in subs)
        if node is None:
            return lambda it: None
        leaves.append(node)
        return lambda it: next(it)

    builder = walk(tree)
    return leaves, lambda values: builder(iter(values))


def leaf_paths(tree, root: str) -> list[str]:
    paths: list[str] = []

    def walk(node, path):
        if isinstance(node, dict):
            for k in sorted(node):
                walk(node[k], f"{path}/{k}")
        elif isinstance(node, (list, tuple)) and not hasattr(node, "_fields"):
            for i, child in enumerate(node):
                walk(child, f"{path}/{i}")
        elif node is not None:
            paths.append(path)

    walk(tree, root)
    return paths


flatten = _flatten


# --------------------------------------------------------------------------
# Fusion pass: loss terms -> point sets and residual programs
# --------------------------------------------------------------------------
def _single_direction(word: tuple) -> tuple[tuple[float, ...], int]:
    first = word[0]
    if any(d != first for d in word):
        raise _unsupported(
            "mixed partial derivatives of the network (such as u_xy) are not carried by the fused kernels; "
            "pure derivatives along a direction up to order 4 are", "grad")
    return first, len(word)


def _is_pure(word: tuple) -> bool:
    return all(d == word[0] for d in word)


def _canonical(direction: tuple[float, ...], order: int) -> tuple[tuple[float, ...], float]:
    """(direction with its first non-zero component positive, sign): D^k along -v is (-1)^k D^k along v."""
    for c in direction:
        if c != 0.0:
            if c < 0.0:
                return tuple(-x for x in direction), -1.0 if order % 2 else 1.0
            break
    return direction, 1.0


def _resolve_mixed_partials(total: sx.Expr) -> sx.Expr:
    """Rewrites every mixed partial derivative of the network (an off-diagonal Hessian entry, u_xxy, ...) as a
    combination of pure derivatives along sums of its directions, which the kernels carry as streams.

    Polarisation: D_{v1}...D_{vk} u = 1/(k! 2^k) * sum over signs e of (e_1...e_k) D^k along (e_1 v1 + ... + e_k vk).
    A second-order mixed partial whose two directions are carried to second order anyway uses
    u_ab = (D^2_{a+b} - D^2_a - D^2_b) / 2 instead: one new direction, not two.  The reference computes the
    same entries by differentiating the gradient graph once more along a basis
    (python/quabla/_transforms.py:1812-2036)."""
    nets = sx.leaves([total], "net")
    pure_order: dict = {}
    for leaf in nets:
        word = leaf.args[1]
        if word and word != sx.MERGED_WORD and _is_pure(word):
            pure_order[word[0]] = max(pure_order.get(word[0], 0), len(word))
    mapping: dict = {}
    for leaf in nets:
        network, word = leaf.args
        if not word or word == sx.MERGED_WORD or _is_pure(word):
            continue
        k = len(word)
        if k > 4:
            raise _unsupported(f"derivative order {k}; orders 1..4 are supported", "grad")
        terms: dict = {}

        def add_term(direction, coefficient: float) -> None:
            if not any(direction):
                return
            direction, sign = _canonical(tuple(float(x) for x in direction), k)
            terms[direction] = terms.get(direction, 0.0) + sign * coefficient

        if k == 2 and pure_order.get(word[0], 0) >= 2 and pure_order.get(word[1], 0) >= 2:
            a, b = word
            add_term(tuple(x + y for x, y in zip(a, b)), 0.5)
            add_term(a, -0.5)
            add_term(b, -0.5)
        else:
            scale = 1.0 / (math.factorial(k) * 2.0**k)
            for signs in itertools.product((1.0, -1.0), repeat=k):
                direction = tuple(sum(e * v[c] for e, v in zip(signs, word)) for c in range(len(word[0])))
                add_term(direction, scale * math.prod(signs))
        replacement = sx.ZERO
        for direction, coefficient in sorted(terms.items(), reverse=True):
            if coefficient != 0.0:
                replacement = replacement + sx.const(coefficient) * sx.net(network, (direction,) * k)
        mapping[leaf] = replacement
    return sx.substitute(total, mapping) if mapping else total


def _merge_enabled() -> bool:
    """QB200_MERGE=0 keeps one second-order stream per direction (for comparisons)."""
    return os.environ.get("QB200_MERGE", "1") != "0"


def build_plan_spec(loss: LossValue, parameters: list[tuple[str, tuple[int, ...]]],
                    data: list[tuple[str, tuple[int, ...], bool]], dtype, merge: bool | None = None) -> PlanSpec:
    """parameters: (name, shape) in gradient-output order; data: (name, shape, retained).

    With `merge` (default: on unless QB200_MERGE=0) a set whose residual uses the second derivatives
    along two or more directions only through one weighted sum (a Laplacian, a heat operator) carries
    that sum as a single stream; `spec.unmerged` then holds the unmerged spec of the same loss.
    """
    if merge is None:
        merge = _merge_enabled()
    if not isinstance(loss, LossValue):
        raise _unsupported("the loss must be a mean or sum over collocation points (or a sum of those)", "loss")
    if loss.constant != 0.0:
        raise _unsupported("a constant added to the loss is not supported", "loss")
    dtype = np.dtype(dtype)
    if loss.dtype != dtype:
        raise _unsupported("mixed float32/float64 programs are rejected", "loss")
    param_shapes = dict(parameters)
    data_index = {name: i for i, (name, _, _) in enumerate(data)}
    data_shapes = {name: shape for name, shape, _ in data}

    layers = None
    activation = "tanh"
    groups: dict = {}
    order: list = []
    for weight, batch, expr in loss.terms:
        nets = sx.leaves([expr], "net")
        if not nets:
            raise _unsupported("a loss term that does not involve the network is not supported", "loss")
        network = nets[0].args[0]
        for leaf in nets:
            if leaf.args[0] != network:
                raise _unsupported("one loss term evaluates the network at two different inputs", "loss")
        if layers is None:
            layers = network.layers
            activation = network.activation
        elif network.layers != layers or network.activation != activation:
            raise _unsupported("the loss uses more than one network", "loss")
        key = (batch, network.inputs)
        if key not in groups:
            groups[key] = []
            order.append(key)
        groups[key].append((weight, expr, network))
    assert layers is not None

    sizes = [layers[0][2]] + [l[3] for l in layers]
    for (w_name, b_name, d_in, d_out), d_prev in zip(layers, sizes):
        if d_in != d_prev:
            raise ValueError("layer widths do not chain")
        if tuple(param_shapes.get(w_name, ())) != (d_in, d_out):
            raise ValueError(f"weight '{w_name}' must have shape [{d_in}, {d_out}]")
    used = [name for l in layers for name in (l[0], l[1]) if name is not None]
    if len(set(used)) != len(used):
        raise _unsupported("a parameter is shared between layers", "loss")
    if sizes[-1] != 1:
        raise _unsupported("the network output must be one scalar per point", "loss")
    spec = PlanSpec(dtype=dtype, sizes=sizes, activation=activation)
    layer_of = {}
    for index, (w_name, b_name, _, _) in enumerate(layers):
        layer_of[w_name] = (index, _lib.WEIGHT)
        if b_name is not None:
            layer_of[b_name] = (index, _lib.BIAS)
    for name, _ in parameters:
        if name in layer_of:
            spec.parameters.append((name, *layer_of[name]))
    for name, shape, retained in data:
        rows = int(shape[0])
        cols = int(np.prod(shape[1:], dtype=np.int64))
        spec.inputs.append((name, rows, cols, bool(retained)))

    merged_any = False
    for key in order:
        batch, inputs = key
        members = groups[key]
        set_weight = members[0][0]
        if set_weight == 0.0:
            raise _unsupported("a loss term with zero weight", "loss")
        total = sx.ZERO
        for weight, expr, _ in members:
            total = total + sx.const(weight / set_weight) * expr
        network = members[0][2]
        # Point-table columns: the network inputs first, then auxiliary data.
        columns: list[tuple[int, int]] = []
        column_of: dict = {}
        for e in inputs:
            if e.kind != "sym" or e.args[0][0] != "col":
                raise _unsupported("the network input must be the point's coordinates themselves "
                                   "(a data column), not an expression of them", "loss")
            _, name, col = e.args[0]
            columns.append((data_index[name], col))
        for leaf in sx.leaves([total], "sym"):
            if leaf.args[0][0] != "col":
                raise _unsupported("a free differentiation variable escaped its transform", "loss")
            _, name, col = leaf.args[0]
            if int(data_shapes[name][0]) != batch:
                raise ValueError(f"input '{name}' does not have the batch size {batch} of its loss term")
            if leaf not in column_of:
                entry = (data_index[name], col)
                if entry in columns:
                    column_of[leaf] = columns.index(entry)
                else:
                    column_of[leaf] = len(columns)
                    columns.append(entry)
        for e in inputs:
            _, name, _ = e.args[0]
            if int(data_shapes[name][0]) != batch:
                raise ValueError(f"input '{name}' does not have the batch size {batch} of its loss term")
        total = _resolve_mixed_partials(total)
        # Streams.
        orders: dict = {}
        for leaf in sx.leaves([total], "net"):
            word = leaf.args[1]
            if word:
                direction, m = _single_direction(word)
                orders[direction] = max(orders.get(direction, 0), m)
        # Second derivatives along directions of order exactly two are candidates for the merged stream.
        merge_weights = None
        targets = [leaf for leaf in sx.leaves([total], "net")
                   if len(leaf.args[1]) == 2 and orders[_single_direction(leaf.args[1])[0]] == 2]
        rewritten = None
        if merge and len(targets) >= 2:
            rewritten = sx.merge_weighted_sum(total, targets, sx.Expr("net", (network, sx.MERGED_WORD)))
        weight_of: dict = {}
        if rewritten is not None:
            total, by_target = rewritten
            weight_of = {_single_direction(t.args[1])[0]: w for t, w in by_target.items()}
            for direction in weight_of:
                orders[direction] = 1  # the merged stream needs their first-order streams only
            merged_any = True
        directions = sorted(orders.items(), key=lambda kv: kv[0], reverse=True)
        base = {}
        next_stream = 1
        for direction, m in directions:
            if m > 4:
                raise _unsupported(f"derivative order {m} along one direction; orders 1..4 are supported", "grad")
            base[direction] = next_stream
            next_stream += m
        merged_stream = -1
        if rewritten is not None:
            merge_weights = [weight_of.get(direction, 0.0) for direction, _ in directions]
            merged_stream = next_stream  # the last stream
            next_stream += 1

        def stream_of(leaf: sx.Expr) -> int:
            word = leaf.args[1]
            if not word:
                return 0
            if word == sx.MERGED_WORD:
                return merged_stream
            direction, m = _single_direction(word)
            return base[direction] + m - 1

        by_stream: dict[int, sx.Expr] = {stream_of(leaf): leaf for leaf in sx.leaves([total], "net")}
        grads: list = []
        for s in range(next_stream):
            leaf = by_stream.get(s)
            if leaf is None:
                grads.append(None)
            else:
                grads.append(sx.derivative(total, lambda l, target=leaf: sx.ONE if l is target else sx.ZERO))
        program = sx.compile_program(total, grads, lambda leaf: column_of[leaf], stream_of)
        spec.sets.append(SetSpec(n_points=batch, weight=set_weight, columns=columns,
                                 directions=[(d, m) for d, m in directions], program=program,
                                 merge_weights=merge_weights))
    if merged_any:
        spec.unmerged = build_plan_spec(loss, parameters, data, dtype, merge=False)
    return spec
