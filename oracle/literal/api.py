"""The reference's Python surface over the literal IR — TEST INFRASTRUCTURE.

Staging follows python/quabla/_transforms.py: a transform called on tracers
stages its function in a graph of its own, with one input per argument leaf
and one per closed-over tracer of an enclosing trace ("captures", :380-400),
transforms that graph, and splices the result into the caller's graph
(`_call_traced` :768-777, `_inline` :490-501):

  grad / value_and_grad   symbolic VJP with a ones seed (:825-894, :912-950);
  vmap                    stage for ONE example, splice with inline_batched (:1658-1734);
  hessian                 forward-mode JVP of the gradient graph, batched over a
                          one-hot basis (:1812-2036, :2173-2179).
"""

from __future__ import annotations

import math

import numpy as np

from . import transforms as tf
from .interp import evaluate
from .ir import F32, F64, Graph

_DTYPES = {np.dtype(np.float32): F32, np.dtype(np.float64): F64}
_NUMPY = {F32: np.float32, F64: np.float64}


class _Trace:
    def __init__(self, graph: Graph) -> None:
        self.graph = graph
        self.captures: dict = {}   # capture input name -> outer Tracer
        self._lifted: dict = {}    # id(outer tracer node) -> inner node

    def lift(self, outer: "Tracer") -> int:
        key = (id(outer.graph), outer.node)
        if key not in self._lifted:
            name = f"capture/{len(self.captures)}"
            info = outer.graph.node(outer.node)
            self._lifted[key] = self.graph.input(name, info.shape, info.dtype)
            self.captures[name] = outer
        return self._lifted[key]


_stack: list[_Trace] = []


def _current() -> _Trace:
    return _stack[-1]


class Tracer:
    """A traced array: a node of the graph being staged."""

    __array_ufunc__ = None

    def __init__(self, graph: Graph, node: int) -> None:
        self.graph = graph
        self.node = node

    @property
    def shape(self) -> tuple:
        return self.graph.shape(self.node)

    @property
    def dtype(self):
        return _NUMPY[self.graph.node(self.node).dtype]

    def _here(self) -> int:
        trace = _current()
        return self.node if self.graph is trace.graph else trace.lift(self)

    def _wrap(self, node: int) -> "Tracer":
        return Tracer(_current().graph, node)

    def _operand(self, other) -> int:
        g = _current().graph
        if isinstance(other, Tracer):
            return other._here()
        if isinstance(other, (int, float)) and not isinstance(other, bool):
            return g.scalar_constant(float(other))
        other = np.asarray(other)
        return g.constant(other, _DTYPES[other.dtype])

    def _binary(self, other, op: str, reverse: bool = False) -> "Tracer":
        g = _current().graph
        a, b = self._here(), self._operand(other)
        if reverse:
            a, b = b, a
        return self._wrap(getattr(g, op)(a, b))

    def __add__(self, o):
        return self._binary(o, "add")

    def __radd__(self, o):
        return self._binary(o, "add", True)

    def __sub__(self, o):
        return self._binary(o, "sub")

    def __rsub__(self, o):
        return self._binary(o, "sub", True)

    def __mul__(self, o):
        return self._binary(o, "mul")

    def __rmul__(self, o):
        return self._binary(o, "mul", True)

    def __truediv__(self, o):
        return self._binary(o, "div")

    def __rtruediv__(self, o):
        return self._binary(o, "div", True)

    def __gt__(self, o):
        return self._binary(o, "greater")

    def __neg__(self):
        g = _current().graph
        return self._wrap(g.sub(g.scalar_constant(0.0), self._here()))

    def __pow__(self, exponent):
        # `x ** 2` with a Python int is Powi (crates/quabla-python/src/tensor_trace.rs:3023-3036).
        if isinstance(exponent, bool) or not isinstance(exponent, int):
            raise TypeError("the literal oracle supports integer powers only")
        return self._wrap(_current().graph.powi(self._here(), exponent))

    def __matmul__(self, other):
        # Rank-1 operands become a row / a column (python/quabla/_ops.py:366-387).
        g = _current().graph
        a, b = self._here(), self._operand(other)
        sa, sb = g.shape(a), g.shape(b)
        if len(sa) == 1:
            a = g.reshape(a, (1, sa[0]))
        if len(sb) == 1:
            b = g.reshape(b, (sb[0], 1))
        out = g.matmul(a, b)
        shape = g.shape(out)
        if len(sa) == 1:
            shape = shape[:-2] + shape[-1:]
            out = g.reshape(out, shape)
        if len(sb) == 1:
            out = g.reshape(out, shape[:-1])
        return self._wrap(out)

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        total = int(np.prod(self.shape, dtype=np.int64))
        shape = tuple(total // max(1, -int(np.prod(shape))) if s == -1 else int(s) for s in shape)
        return self._wrap(_current().graph.reshape(self._here(), shape))

    def __getitem__(self, index):
        # Integer and full-slice indexing as slice + reshape
        # (crates/quabla-python/src/tensor_trace.rs:1808-1827).
        if not isinstance(index, tuple):
            index = (index,)
        g = _current().graph
        node = self._here()
        axis = 0
        for item in index:
            if isinstance(item, slice) and item == slice(None):
                axis += 1
                continue
            extent = g.shape(node)[axis]
            position = int(item) % extent
            node = g.slice(node, axis, position, 1)
            shape = g.shape(node)
            node = g.reshape(node, shape[:axis] + shape[axis + 1:])
        return self._wrap(node)


# -- array functions ---------------------------------------------------------------------
def _unary(kind: str, numpy_function):
    def apply(x):
        if isinstance(x, Tracer):
            return x._wrap(_current().graph.unary(x._here(), kind))
        return numpy_function(x)

    return apply


tanh = _unary("tanh", np.tanh)
sin = _unary("sin", np.sin)
cos = _unary("cos", np.cos)
exp = _unary("exp", np.exp)
log1p = _unary("log1p", np.log1p)
expm1 = _unary("expm1", np.expm1)
tan = _unary("tan", np.tan)
erf = _unary("erf", np.vectorize(math.erf, otypes=[np.float64]))
erfc = _unary("erfc", np.vectorize(math.erfc, otypes=[np.float64]))


def where(condition, on_true, on_false):
    """Selection by a Bool tracer (python/quabla/_ops.py `where`): operands may be tracers or Python numbers."""
    g = _current().graph
    lift = lambda v: v._here() if isinstance(v, Tracer) else g.scalar_constant(float(v))  # noqa: E731
    return condition._wrap(g.where(condition._here(), lift(on_true), lift(on_false)))


# The reference builds these from where / exp / log1p, so that no branch overflows and the gradients of the
# unselected branch stay finite (crates/quabla-python/src/composite.rs:160-209, python/quabla/_ops.py:475-505).
# relu's NaN clause (`nan_or`) is left out: the oracle is run on finite inputs.
def _abs(x):
    return where(x > 0.0, x, 0.0 - x)


def _exp_negative_abs(x):
    return exp(_abs(x) * -1.0)


def relu(x):
    return where(x > 0.0, x, 0.0)


def sigmoid(x):
    if not isinstance(x, Tracer):
        x = np.asarray(x, dtype=np.float64)
        e = np.exp(-np.abs(x))
        return np.where(x > 0, 1.0 / (1.0 + e), e / (1.0 + e))
    decay = _exp_negative_abs(x)
    denominator = decay + 1.0
    positive = 1.0 / denominator
    negative = decay / denominator
    return where(x > 0.0, positive, negative)


def softplus(x):
    return relu(x) + log1p(_exp_negative_abs(x))


def silu(x):
    return x * sigmoid(x)


_GELU_SCALE = 2.0 * math.sqrt(2.0 / math.pi)


def gelu(x):
    tail = _abs(x) > 40.0
    safe = where(tail, 0.0, x)
    value = safe * sigmoid(safe * (safe * safe * 0.044715 + 1.0) * _GELU_SCALE)
    return where(tail, where(x > 0.0, x, -0.0), value)


def mean(x):
    return x._wrap(_current().graph.mean(x._here())) if isinstance(x, Tracer) else np.mean(x)


def sum(x, axis=None):  # noqa: A001
    if not isinstance(x, Tracer):
        return np.sum(x, axis=axis)
    g = _current().graph
    return x._wrap(g.sum(x._here()) if axis is None else g.sum_axis(x._here(), axis))


def trace(x):
    """Sum of the diagonal: the diagonal entries picked by indexing, then added
    (python/quabla/_ops.py:997-1027 extracts the diagonal with strided slicing and sums it)."""
    if not isinstance(x, Tracer):
        return np.trace(x)
    n = x.shape[-1]
    total = x[0, 0]
    for i in range(1, n):
        total = total + x[i, i]
    return total


def array(value, dtype=None):
    out = np.asarray(value, dtype=dtype)
    return out.astype(np.float64) if dtype is None and out.dtype != np.float32 else out


def zeros(shape, dtype=np.float64):
    return np.zeros(shape, dtype=dtype)


# -- pytrees --------------------------------------------------------------------------------
def _flatten(tree):
    leaves = []

    def walk(node):
        if isinstance(node, dict):
            keys = sorted(node)
            subs = [walk(node[k]) for k in keys]
            return lambda it: {k: s(it) for k, s in zip(keys, subs)}
        if isinstance(node, (list, tuple)):
            subs = [walk(c) for c in node]
            kind = type(node)
            return lambda it: kind(s(it) for s in subs)
        leaves.append(node)
        return lambda it: next(it)

    builder = walk(tree)
    return leaves, lambda values: builder(iter(values))


# -- staging ----------------------------------------------------------------------------------
def _stage(fun, args, example_shapes=None):
    """Trace fun(*args) in a fresh graph: one input per array/tracer leaf of args.
    Returns (trace, input names per leaf, leaves, rebuild, output tracers flat, out rebuild)."""
    trace = _Trace(Graph())
    _stack.append(trace)
    try:
        leaves, rebuild = _flatten(list(args))
        names, traced = [], []
        for index, leaf in enumerate(leaves):
            if isinstance(leaf, Tracer):
                info = leaf.graph.node(leaf.node)
                shape, dtype = info.shape, info.dtype
            elif isinstance(leaf, (np.ndarray, np.generic)):
                shape, dtype = np.shape(leaf), _DTYPES[np.asarray(leaf).dtype]
            else:
                names.append(None)
                traced.append(leaf)
                continue
            if example_shapes is not None and example_shapes[index] is not None:
                shape = example_shapes[index]
            name = f"arg/{index}"
            names.append(name)
            traced.append(Tracer(trace.graph, trace.graph.input(name, shape, dtype)))
        result = fun(*rebuild(traced))
        out_leaves, out_rebuild = _flatten(result)
        out_nodes = []
        for leaf in out_leaves:
            if not isinstance(leaf, Tracer):
                leaf = Tracer(trace.graph, trace.graph.scalar_constant(float(leaf)))
            out_nodes.append(leaf._here())
    finally:
        _stack.pop()
    return trace, names, leaves, out_nodes, out_rebuild


def _bindings(trace: _Trace, names, leaves) -> dict:
    """Caller-side nodes for the staged graph's inputs (arguments and captures)."""
    g = _current().graph
    bound = {}
    for name, leaf in zip(names, leaves):
        if name is None:
            continue
        if isinstance(leaf, Tracer):
            bound[name] = leaf._here()
        else:
            leaf = np.asarray(leaf)
            bound[name] = g.constant(leaf, _DTYPES[leaf.dtype])
    for name, outer in trace.captures.items():
        bound[name] = outer._here()
    return bound


def _any_tracer(args) -> bool:
    return any(isinstance(leaf, Tracer) for leaf in _flatten(list(args))[0])


class _ValueAndGrad:
    def __init__(self, fun, argnums=0, mode="value_and_grad") -> None:
        self.fun, self.argnums, self.mode = fun, argnums, mode

    def _graph(self, args):
        """The VJP graph of fun at args: (trace, names, leaves, graph, value node, gradient nodes of the
        differentiated leaves, rebuild of the gradient pytree)."""
        trace, names, leaves, out_nodes, _ = _stage(self.fun, args)
        if len(out_nodes) != 1 or trace.graph.shape(out_nodes[0]) != ():
            raise ValueError("grad requires a scalar output")
        g2, values, _, gradients = tf.symbolic_vjp(trace.graph, [(out_nodes[0], None)])
        counts = [len(_flatten([a])[0]) for a in args]
        start = int(np.sum(counts[: self.argnums]))
        wanted = names[start:start + counts[self.argnums]]
        _, grad_rebuild = _flatten(args[self.argnums])
        return trace, names, leaves, g2, values[out_nodes[0]], [gradients[n] for n in wanted], grad_rebuild

    def __call__(self, *args):
        if not _stack:
            return self._top_level(args)
        trace, names, leaves, g2, value, grads, grad_rebuild = self._graph(args)
        spliced = tf.inline(_current().graph, g2, _bindings(trace, names, leaves), [value] + grads)
        tracers = [Tracer(_current().graph, n) for n in spliced]
        gradient = grad_rebuild(tracers[1:])
        return gradient if self.mode == "grad" else (tracers[0], gradient)

    def _top_level(self, args):
        trace, names, leaves, g2, value, grads, grad_rebuild = self._graph(args)
        if trace.captures:
            raise ValueError("a top-level transform cannot capture tracers")
        inputs = {n: np.asarray(l) for n, l in zip(names, leaves) if n is not None}
        results = evaluate(g2, inputs, [value] + grads)
        self.last_graph = g2
        dtypes = [g2.node(n).dtype for n in [value] + grads]
        arrays = [np.asarray(r, dtype=_NUMPY[d]) for r, d in zip(results, dtypes)]
        gradient = grad_rebuild(arrays[1:])
        return gradient if self.mode == "grad" else (arrays[0], gradient)


def value_and_grad(fun, argnums=0):
    return _ValueAndGrad(fun, argnums, "value_and_grad")


def grad(fun, argnums=0):
    return _ValueAndGrad(fun, argnums, "grad")


def vmap(fun, in_axes=0):
    def mapped(*args):
        axes = (in_axes,) * len(args) if isinstance(in_axes, int) or in_axes is None else tuple(in_axes)
        leaves, _ = _flatten(list(args))
        counts = [len(_flatten([a])[0]) for a in args]
        leaf_axes = [axis for axis, count in zip(axes, counts) for _ in range(count)]
        batch = None
        example_shapes = []
        for leaf, axis in zip(leaves, leaf_axes):
            if axis is None or not isinstance(leaf, (Tracer, np.ndarray)):
                example_shapes.append(None)
                continue
            shape = tuple(leaf.shape)
            batch = shape[0]
            example_shapes.append(shape[1:])
        trace, names, leaves, out_nodes, out_rebuild = _stage(fun, args, example_shapes)
        bound = _bindings(trace, names, leaves)
        bindings = {}
        for name, node in bound.items():
            index = names.index(name) if name in names else None
            is_mapped = index is not None and example_shapes[index] is not None
            bindings[name] = (node, is_mapped)
        g = _current().graph
        spliced = tf.inline_batched(g, trace.graph, bindings, batch, out_nodes)
        results = []
        for (node, is_mapped), out in zip(spliced, out_nodes):
            if not is_mapped:
                node = g.broadcast_to(node, (batch,) + g.shape(node))
            results.append(Tracer(g, node))
        return out_rebuild(results)

    return mapped


def hessian(fun, argnums=0):
    def apply(*args):
        x = args[argnums]
        # Stage the gradient function, take its JVP with a tangent input, and batch the
        # tangent over a one-hot basis.
        def gradient(*inner):
            return grad(fun, argnums)(*inner)

        trace, names, leaves, out_nodes, _ = _stage(gradient, args)
        counts = [len(_flatten([a])[0]) for a in args]
        target = names[int(np.sum(counts[:argnums]))]
        g3, _, tangents = tf.symbolic_jvp(trace.graph, out_nodes, {target: "tangent"})
        n = int(np.prod(x.shape, dtype=np.int64))
        g = _current().graph
        dtype = x.graph.node(x.node).dtype
        basis = g.constant(np.eye(n).reshape((n,) + tuple(x.shape)), dtype)
        bindings = {name: (node, False) for name, node in _bindings(trace, names, leaves).items()}
        bindings["tangent"] = (basis, True)
        (node, _), = tf.inline_batched(g, g3, bindings, n, tangents)
        return Tracer(g, g.reshape(node, tuple(x.shape) + tuple(x.shape)))

    return apply


def jvp(fun, primals, tangents):
    """`jvp(fun, primals, tangents)` called on tracers (python/quabla/_transforms.py:1273-1361): stage
    `fun` once, build the forward-mode graph with one tangent input per floating primal leaf
    (`graph._symbolic_jvp(traced, tangent_names)`, tensor_ir.rs:2999-3319 through op/jvp.rs), and splice it
    into the caller's graph with the primals and the tangents bound (`_call_traced` -> `_splice`,
    _transforms.py:768-777, 490-501).  Returns (primal outputs, tangent outputs)."""
    primals, tangents = tuple(primals), tuple(tangents)
    if len(primals) != len(tangents):
        raise ValueError("jvp requires one tangent per primal")
    trace, names, leaves, out_nodes, out_rebuild = _stage(fun, primals)
    tangent_leaves, _ = _flatten(list(tangents))
    if len(tangent_leaves) != len(leaves):
        raise ValueError("jvp tangents must have the tree structure of the primals")
    tangent_names = {name: "tangent/" + name for name in names if name is not None}
    g3, values, tangent_nodes = tf.symbolic_jvp(trace.graph, out_nodes, tangent_names)
    g = _current().graph
    bound = _bindings(trace, names, leaves)
    for name, leaf, tangent in zip(names, leaves, tangent_leaves):
        if name is None:
            continue
        if isinstance(tangent, Tracer):
            bound[tangent_names[name]] = tangent._here()
        else:
            dtype = g.node(bound[name]).dtype
            tangent = np.broadcast_to(np.asarray(tangent, dtype=np.float64), g.shape(bound[name]))
            bound[tangent_names[name]] = g.constant(np.array(tangent), dtype)
    spliced = tf.inline(g, g3, bound, list(values) + list(tangent_nodes))
    count = len(out_nodes)
    return (out_rebuild([Tracer(g, n) for n in spliced[:count]]),
            out_rebuild([Tracer(g, n) for n in spliced[count:]]))


def value_and_grad_data_parallel(fun, params, shards: list, reduction: str = "mean"):
    """CPU data-parallel oracle (value_and_vjp_data_parallel,
    crates/quabla-core/src/tensor_ir.rs:11622-11724): per-shard value-and-gradient, the
    local cotangent scaled by 1/shards for a mean, losses and gradients summed in shard order."""
    scale = 1.0 / len(shards) if reduction == "mean" else 1.0
    total_value, total_grads = None, None
    for shard in shards:
        value, grads = value_and_grad(fun)(params, *shard)
        leaves, rebuild = _flatten(grads)
        leaves = [np.asarray(np.asarray(l, dtype=np.float64) * scale, dtype=l.dtype) for l in leaves]
        value = np.asarray(np.float64(value) * scale, dtype=value.dtype)
        if total_value is None:
            total_value, total_grads = value, leaves
        else:
            total_value = np.asarray(total_value + value, dtype=value.dtype)
            total_grads = [np.asarray(a + b, dtype=a.dtype) for a, b in zip(total_grads, leaves)]
    return total_value, rebuild(total_grads)
