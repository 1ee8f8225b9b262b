"""A plan description from the reference's program text, without the Python tracer.

The reference prints a traced program one node per line,
`%k = op(%i, %j, attributes) : tensor<dims x dtype>`
(`TensorIr::lower_text`, crates/quabla-core/src/tensor_ir.rs:6605-6836; format pinned by
crates/quabla-core/tests/snapshots/tensor_op_transforms.txt).  A host that already holds such a program (the
reference's Rust side after its own tracing) can hand that text over instead of a Python loss:
`plan_spec_from_text` parses it and recognises the PINN structure in it, or refuses with
`UnsupportedOperationError` (QB200_UNSUPPORTED at the C level: "no silent fallback").

What the text of a PINN loss looks like.  The derivative transforms are already expanded: `grad(grad(u))` under
`vmap` is some ninety nodes of transposes, adjoint products and tanh chain rules, and nothing names "u_xx".
Recognition is therefore semantic, in three steps, all at plan-build time on the host:

1. Structure that IS explicit is read off the text: the loss as a sum of `mean` / `sum` reductions of per-point
   expressions, the elementwise residual algebra inside each of them, the scalar constants, the data columns, and
   the network's layers from the shapes of the named parameter inputs.
2. Every per-point scalar that depends on the parameters and is not produced by an elementwise op (the end of an
   adjoint chain, one entry of a gradient or Hessian) is a LEAF.  The text is evaluated in float64 on a handful
   of random points with random parameters (a small interpreter of the ops below), the network's directional
   Taylor jets are computed directly on the same points, and a leaf is identified as the derivative
   d^k u / dx_a .. dx_b whose values it reproduces to 1e-9 on every point of every trial.  A leaf that matches
   nothing refuses the program; two different polynomials in random weights do not agree by accident.
3. The identified leaves become network-derivative symbols of the fusion pass (`_trace.build_plan_spec`), which
   turns them into streams and the residual into a register program exactly as it does for a traced loss
   (mixed partials, merged Laplacian streams included).

The text does not carry the elements of dense constants (`constant[dense]`, e.g. the one-hot basis `hessian`
batches over); the caller passes them by node id, as the reference has them in memory next to the text.
"""

from __future__ import annotations

import itertools
import math
import re
from dataclasses import dataclass

import numpy as np

from . import _symbolic as sx
from . import _trace as tr
from ._errors import UnsupportedOperationError
from ._plan import COTANGENT_NAME, PlanSpec

_UNARY = {"tanh": np.tanh, "sin": np.sin, "cos": np.cos, "exp": np.exp, "log": np.log, "log1p": np.log1p,
          "expm1": np.expm1, "tan": np.tan, "sqrt": np.sqrt,
          "erf": np.vectorize(math.erf, otypes=[np.float64]), "erfc": np.vectorize(math.erfc, otypes=[np.float64])}
_BINARY = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide}
_DTYPES = {"f32": np.float32, "f64": np.float64}
_LINE = re.compile(r"^%(\d+) = ([a-z_0-9]+)(?:\[([^\]]*)\])?(?:\(([^)]*)\))?((?: [a-z]+=[^:]+)?) : tensor<([^>]+)>$")
_PROBE_POINTS = 5
_PROBE_TRIALS = 2
_MATCH_TOLERANCE = 1e-9
_MAX_ORDER = 4  # highest derivative order a stream carries


def _refuse(message: str) -> UnsupportedOperationError:
    return UnsupportedOperationError(f"plan text not recognised: {message}", op="plan_text", device="cuda")


@dataclass
class Node:
    op: str            # the text's op name; unary kinds keep their own name
    inputs: tuple
    attrs: dict
    shape: tuple
    dtype: str         # "f32", "f64" or "i1"


def parse(text: str) -> list[Node]:
    """The node list of a program text; node k must be defined on line k."""
    nodes: list[Node] = []
    for line_number, line in enumerate(text.strip().splitlines()):
        match = _LINE.match(line.strip())
        if match is None:
            raise _refuse(f"line {line_number + 1} is not `%k = op(...) : tensor<...>`: {line.strip()[:80]!r}")
        index, op, bracket, operands, trailing, kind = match.groups()
        if int(index) != len(nodes):
            raise _refuse(f"node %{index} is defined on line {line_number + 1}")
        *dims, dtype = kind.split("x")
        if dtype not in ("f32", "f64", "i1"):
            raise _refuse(f"node %{index} has element type {dtype!r}")
        shape = tuple(int(d) for d in dims)
        inputs, attrs = [], {}
        fields = [f.strip() for f in _split_top_level(operands or "")] + ([trailing.strip()] if trailing.strip() else [])
        for position, field in enumerate(f for f in fields if f):
            if field.startswith("%"):
                inputs.append(int(field[1:]))
            elif "=" in field:
                key, value = field.split("=", 1)
                attrs[key.strip()] = value.strip()
            else:
                attrs[f"arg{position}"] = field  # powi's bare exponent
        if bracket is not None:
            if "=" in bracket:
                key, value = bracket.split("=", 1)
                attrs[key] = value
            else:
                attrs[bracket] = True
        for i in inputs:
            if i >= len(nodes):
                raise _refuse(f"node %{index} reads %{i} before it is defined")
        nodes.append(Node(op, tuple(inputs), attrs, shape, dtype))
    if not nodes:
        raise _refuse("the text is empty")
    return nodes


def _split_top_level(text: str) -> list[str]:
    parts, depth, current = [], 0, []
    for ch in text:
        if ch == "[":
            depth += 1
        elif ch == "]":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append("".join(current))
            current = []
        else:
            current.append(ch)
    parts.append("".join(current))
    return parts


def _int_list(text: str) -> tuple:
    return tuple(int(v) for v in text.strip("[] ").split(",") if v.strip())


def evaluate(nodes: list[Node], inputs: dict, constants: dict) -> list:
    """float64 values of every node (Bool nodes as booleans).  Only the recogniser's probes run this."""
    values: list = []
    for index, node in enumerate(nodes):
        x = [values[i] for i in node.inputs]
        op, a = node.op, node.attrs
        if op == "input":
            v = np.asarray(inputs[a["name"]], dtype=np.float64).reshape(node.shape)
        elif op == "constant":
            if "value" in a:
                v = np.float64(float(a["value"]))
            elif index in constants:
                v = np.asarray(constants[index], dtype=np.float64).reshape(node.shape)
            else:
                raise _refuse(f"node %{index} is a dense constant; the text does not carry its elements, pass them "
                              f"in `constants`")
        elif op in _BINARY:
            v = _BINARY[op](x[0], x[1])
        elif op in _UNARY:
            with np.errstate(all="ignore"):
                v = _UNARY[op](x[0])
        elif op == "cast":
            v = x[0]
        elif op == "powi":
            v = np.asarray(x[0]) ** int(a["arg1"])
        elif op == "matmul":
            v = np.matmul(x[0], x[1])
        elif op in ("sum", "mean"):
            reducer = np.sum if op == "sum" else np.mean
            v = reducer(x[0], axis=int(a["axis"])) if "axis" in a else reducer(x[0])
        elif op in ("reshape", "broadcast"):
            v = np.reshape(x[0], node.shape) if op == "reshape" else np.broadcast_to(x[0], node.shape)
        elif op == "transpose":
            v = np.transpose(x[0], _int_list(a["axes"]))
        elif op == "slice":
            start, length = int(a["start"]), int(a["length"])
            v = np.take(x[0], np.arange(start, start + length), axis=int(a["axis"]))
        elif op == "pad_slice":
            axis, start = int(a["axis"]), int(a["start"])
            v = np.zeros(node.shape)
            window = [slice(None)] * len(node.shape)
            window[axis] = slice(start, start + np.shape(x[0])[axis])
            v[tuple(window)] = x[0]
        elif op == "concat":
            v = np.concatenate([np.asarray(t) for t in x], axis=int(a["axis"]))
        elif op == "greater":
            v = np.asarray(x[0]) > np.asarray(x[1])
        elif op == "where":
            v = np.where(x[0], x[1], x[2])
        elif op == "stop_gradient":
            v = x[0]
        else:
            raise _refuse(f"node %{index} uses op {op!r}, which is outside the PINN family")
        v = np.asarray(v)
        if v.shape != node.shape:
            v = np.broadcast_to(v, node.shape) if v.size != int(np.prod(node.shape, dtype=np.int64)) else v.reshape(node.shape)
        values.append(v)
    return values


# -- the network's jets, computed directly -----------------------------------------------------------------------
def _activation_derivatives(kind: str, z: np.ndarray) -> list:
    if kind == "sin":
        s, c = np.sin(z), np.cos(z)
        return [s, c, -s, -c, s]
    t = np.tanh(z)
    d1 = 1.0 - t * t
    d2 = -2.0 * t * d1
    d3 = -2.0 * (d1 * d1 + t * d2)
    d4 = -2.0 * (3.0 * d1 * d2 + t * d3)
    return [t, d1, d2, d3, d4]


def directional_jets(weights: list, biases: list, activation: str, points: np.ndarray, direction, order: int) -> list:
    """[u, D u, .., D^order u] per point, D the derivative along `direction` (Taylor-mode through the layers)."""
    streams = [points] + [np.broadcast_to(np.asarray(direction, dtype=np.float64), points.shape) if m == 0
                          else np.zeros_like(points) for m in range(order)]
    for layer, (w, b) in enumerate(zip(weights, biases)):
        z = [s @ w for s in streams]
        if b is not None:
            z[0] = z[0] + b
        if layer == len(weights) - 1:
            streams = z
            break
        f = _activation_derivatives(activation, z[0])
        h = [f[0]]
        if order >= 1:
            h.append(f[1] * z[1])
        if order >= 2:
            h.append(f[2] * z[1] ** 2 + f[1] * z[2])
        if order >= 3:
            h.append(f[3] * z[1] ** 3 + 3.0 * f[2] * z[1] * z[2] + f[1] * z[3])
        if order >= 4:
            h.append(f[4] * z[1] ** 4 + 6.0 * f[3] * z[1] ** 2 * z[2] + f[2] * (3.0 * z[2] ** 2 + 4.0 * z[1] * z[3])
                     + f[1] * z[4])
        streams = h
    return [s.reshape(-1) for s in streams]


def _partial(word: tuple, jets) -> np.ndarray:
    """The partial derivative along the unit directions in `word` (indices into the input), by polarisation."""
    k = len(word)
    if k == 0:
        return jets((), 0)[0]
    total = 0.0
    for signs in itertools.product((1.0, -1.0), repeat=k):
        direction = {}
        for sign, axis in zip(signs, word):
            direction[axis] = direction.get(axis, 0.0) + sign
        key = tuple(sorted((axis, c) for axis, c in direction.items() if c != 0.0))
        if not key:
            continue
        total = total + math.prod(signs) * jets(key, k)[k]
    return total / (math.factorial(k) * 2.0**k)


# -- recognition ---------------------------------------------------------------------------------------------------
_ELEMENTWISE = set(_BINARY) | set(_UNARY) | {"powi", "cast"}


class _Recogniser:
    def __init__(self, nodes: list[Node], parameter_names: list[str], constants: dict) -> None:
        self.nodes = nodes
        self.constants = constants
        self.inputs = {n.attrs["name"]: (i, n) for i, n in enumerate(nodes) if n.op == "input"}
        missing = [p for p in parameter_names if p not in self.inputs]
        if missing:
            raise _refuse(f"parameter {missing[0]!r} is not an input of the program")
        self.parameter_names = list(parameter_names)
        self.data_names = [name for name in self.inputs if name not in parameter_names and name != COTANGENT_NAME]
        # One floating dtype for every input; weak float64 scalars that are cast to it are part of the format.
        floating = {n.dtype for n in nodes if n.op == "input"}
        if len(floating) != 1 or not floating <= set(_DTYPES):
            raise _refuse("mixed float32/float64 programs are rejected")
        self.dtype = np.dtype(_DTYPES[floating.pop()])
        self.depends_on_parameters = []
        parameter_ids = {self.inputs[p][0] for p in parameter_names}
        for i, n in enumerate(nodes):
            self.depends_on_parameters.append(i in parameter_ids or any(self.depends_on_parameters[j] for j in n.inputs))
        self._layers()
        self._probe()
        self._memo: dict = {}

    # The network: weights [d_in, d_out] and biases [d_out] among the named parameters, chained by shape.
    def _layers(self) -> None:
        weights = [(name, self.inputs[name][1].shape) for name in self.parameter_names if len(self.inputs[name][1].shape) == 2]
        biases = [(name, self.inputs[name][1].shape) for name in self.parameter_names if len(self.inputs[name][1].shape) == 1]
        if len(weights) + len(biases) != len(self.parameter_names) or not weights:
            raise _refuse("the parameters must be weight matrices [d_in, d_out] and bias vectors [d_out]")
        for (_, a), (_, b) in zip(weights, weights[1:]):
            if a[1] != b[0]:
                raise _refuse("the weight matrices do not chain in the order the parameters are named")
        if weights[-1][1][1] != 1:
            raise _refuse("the network output must be one scalar per point")
        layers = []
        unused = list(biases)
        for name, (d_in, d_out) in weights:
            prefix = name.rsplit("/", 1)[0]
            bias = next((b for b in unused if b[0].rsplit("/", 1)[0] == prefix and b[1] == (d_out,)), None)
            if bias is not None:
                unused.remove(bias)
            layers.append((name, None if bias is None else bias[0], d_in, d_out))
        if unused:
            raise _refuse(f"bias {unused[0][0]!r} does not belong to a layer")
        self.layers = tuple(layers)
        kinds = {n.op for i, n in enumerate(self.nodes) if n.op in _UNARY and self.depends_on_parameters[i] and len(n.shape) >= 2}
        if kinds <= {"tanh"}:
            self.activation = "tanh"
        elif kinds <= {"sin", "cos"} and "sin" in kinds:
            self.activation = "sin"
        else:
            raise _refuse(f"hidden layers with {sorted(kinds)}: tanh or sin networks are recognised from text")

    # Random parameters and points; every node's values per trial.
    def _probe(self) -> None:
        generator = np.random.default_rng(20240607)
        self.trials = []
        for _ in range(_PROBE_TRIALS):
            feed = {}
            for name, (_, node) in self.inputs.items():
                if name == COTANGENT_NAME:
                    feed[name] = np.ones(node.shape)
                elif name in self.parameter_names:
                    scale = 1.0 / math.sqrt(max(1, node.shape[0])) if len(node.shape) == 2 else 0.3
                    feed[name] = generator.normal(size=node.shape) * scale
                else:
                    feed[name] = generator.uniform(-1.0, 1.0, size=node.shape)
            self.trials.append((feed, evaluate(self.nodes, feed, self.constants)))

    def _values(self, index: int, rows: int) -> np.ndarray:
        """Node `index` per point, over the first probe points of every trial."""
        return np.concatenate([np.asarray(values[index], dtype=np.float64).reshape(rows, -1)[:_PROBE_POINTS].reshape(-1)
                               for _, values in self.trials])

    # -- the loss: weighted batch reductions -----------------------------------------------------------------------
    def loss_terms(self, index: int, scale: float = 1.0) -> list:
        node = self.nodes[index]
        if node.shape != () and int(np.prod(node.shape)) != 1:
            raise _refuse(f"the loss node %{index} is not a scalar")
        op = node.op
        if op in ("reshape", "cast", "stop_gradient"):
            return self.loss_terms(node.inputs[0], scale)
        if op in ("add", "sub"):
            sign = 1.0 if op == "add" else -1.0
            return self.loss_terms(node.inputs[0], scale) + self.loss_terms(node.inputs[1], sign * scale)
        if op in ("mul", "div"):
            lhs, rhs = node.inputs
            if self._is_scalar_constant(rhs):
                c = self._constant(rhs)
                return self.loss_terms(lhs, scale * c if op == "mul" else scale / c)
            if op == "mul" and self._is_scalar_constant(lhs):
                return self.loss_terms(rhs, scale * self._constant(lhs))
            raise _refuse(f"the loss node %{index} multiplies two computed scalars")
        if op in ("sum", "mean") and "axis" not in node.attrs:
            operand = node.inputs[0]
            batch = int(np.prod(self.nodes[operand].shape, dtype=np.int64))
            weight = scale / batch if op == "mean" else scale
            return [(weight, batch, self.expression(operand, batch))]
        raise _refuse(f"the loss node %{index} ({op}) is not a sum of mean / sum reductions over points")

    def _is_scalar_constant(self, index: int) -> bool:
        node = self.nodes[index]
        if node.op in ("reshape", "cast", "broadcast"):
            return self._is_scalar_constant(node.inputs[0])
        return node.op == "constant" and "value" in node.attrs

    def _constant(self, index: int) -> float:
        node = self.nodes[index]
        if node.op in ("reshape", "cast", "broadcast"):
            return self._constant(node.inputs[0])
        value = float(node.attrs["value"])
        return float(self.dtype.type(value))  # a weak scalar adopts the plan dtype (tensor_ir.rs:6995-7004)

    # -- per-point expressions -------------------------------------------------------------------------------------
    def expression(self, index: int, batch: int) -> sx.Expr:
        key = (index, batch)
        if key not in self._memo:
            self._memo[key] = self._expression(index, batch)
        return self._memo[key]

    def _expression(self, index: int, batch: int) -> sx.Expr:
        node = self.nodes[index]
        count = int(np.prod(node.shape, dtype=np.int64))
        if self._is_scalar_constant(index):
            return sx.const(self._constant(index))
        if count != batch:
            raise _refuse(f"node %{index} of shape {list(node.shape)} is not one scalar per point of a batch of {batch}")
        op = node.op
        if self.depends_on_parameters[index]:
            # A derivative of the network, whatever chain of ops produced it (the head's `matmul + bias` is u,
            # the end of an adjoint chain a gradient entry) ...
            leaf = self._network_leaf(index, batch)
            if leaf is not None:
                return leaf
        if op in ("reshape", "cast", "stop_gradient"):
            return self.expression(node.inputs[0], batch)
        # ... or residual algebra over such derivatives and the point's data.
        if op in _BINARY:
            lhs, rhs = (self.expression(i, batch) for i in node.inputs)
            return {"add": sx.add, "sub": sx.sub, "mul": sx.mul, "div": sx.div}[op](lhs, rhs)
        if op == "powi":
            return sx.powi(self.expression(node.inputs[0], batch), int(node.attrs["arg1"]))
        if op in _UNARY:
            return sx.unary(op, self.expression(node.inputs[0], batch))
        if not self.depends_on_parameters[index]:
            return self._data_column(index, batch)
        raise _refuse(f"node %{index} ({op}) depends on the parameters but is neither a derivative (order <= "
                      f"{_MAX_ORDER}) of the network at a data input's points nor elementwise algebra over such")

    def _columns_of(self, batch: int) -> list:
        """(name, flat column, values) of every data column with `batch` rows."""
        out = []
        for name in self.data_names:
            input_index, node = self.inputs[name]
            if not node.shape or node.shape[0] != batch:
                continue
            width = int(np.prod(node.shape[1:], dtype=np.int64))
            for column in range(width):
                values = np.concatenate([np.asarray(v[input_index], dtype=np.float64).reshape(batch, width)[:_PROBE_POINTS, column]
                                         for _, v in self.trials])
                out.append((name, column, values))
        return out

    def _data_column(self, index: int, batch: int) -> sx.Expr:
        values = self._values(index, batch)
        for name, column, candidate in self._columns_of(batch):
            if np.array_equal(values, candidate):
                return sx.sym(("col", name, column))
        raise _refuse(f"node %{index} is per-point data that is not a column of an input")

    def _network_leaf(self, index: int, batch: int):
        """The network-derivative symbol node `index` equals on every probe, or None."""
        values = self._values(index, batch)
        d0 = self.layers[0][2]
        for name in self.data_names:
            input_index, node = self.inputs[name]
            width = int(np.prod(node.shape[1:], dtype=np.int64)) if node.shape else 0
            if not node.shape or node.shape[0] != batch or width != d0:
                continue
            cache: dict = {}

            def jets(direction_key: tuple, order: int, input_index=input_index):
                key = (direction_key, order)
                if key not in cache:
                    vector = np.zeros(d0)
                    for axis, c in direction_key:
                        vector[axis] = c
                    per_trial = []
                    for feed, trial_values in self.trials:
                        points = np.asarray(trial_values[input_index], dtype=np.float64).reshape(batch, d0)[:_PROBE_POINTS]
                        weights = [feed[w] for w, _, _, _ in self.layers]
                        biases = [None if b is None else feed[b] for _, b, _, _ in self.layers]
                        per_trial.append(directional_jets(weights, biases, self.activation, points, vector, order))
                    cache[key] = [np.concatenate([t[m] for t in per_trial]) for m in range(order + 1)]
                return cache[key]

            for order in range(0, _MAX_ORDER + 1):
                for word in itertools.combinations_with_replacement(range(d0), order):
                    candidate = _partial(word, jets)
                    scale = max(1.0, float(np.max(np.abs(candidate))))
                    if float(np.max(np.abs(values - candidate))) <= _MATCH_TOLERANCE * scale:
                        network = tr.Network(self.layers, tuple(sx.sym(("col", name, c)) for c in range(d0)), self.activation)
                        unit = lambda axis: tuple(1.0 if c == axis else 0.0 for c in range(d0))  # noqa: E731
                        return sx.net(network, tuple(unit(axis) for axis in word))
        return None


def plan_spec_from_text(text: str, parameter_names, loss: int | None = None, constants: dict | None = None,
                        retained=()) -> tuple[PlanSpec, list, list]:
    """(plan description, parameter (name, shape) list, data (name, shape) list) of the program `text`.

    parameter_names   the inputs that are trained, in gradient-output order (tensor_trace.rs:4562-4573);
    loss              id of the loss node (default: the last node);
    constants         {node id: array} for `constant[dense]` nodes;
    retained          names of data inputs bound once and kept on the device.
    Raises UnsupportedOperationError when the program is not a recognised PINN loss."""
    nodes = parse(text)
    parameter_names = list(parameter_names)
    recogniser = _Recogniser(nodes, parameter_names, dict(constants or {}))
    loss = len(nodes) - 1 if loss is None else int(loss)
    if not 0 <= loss < len(nodes):
        raise _refuse(f"loss node %{loss} does not exist")
    terms = recogniser.loss_terms(loss)
    value = tr.LossValue(terms, 0.0, recogniser.dtype)
    parameters = [(name, tuple(recogniser.inputs[name][1].shape)) for name in parameter_names]
    data = [(name, tuple(recogniser.inputs[name][1].shape), name in set(retained)) for name in recogniser.data_names]
    spec = tr.build_plan_spec(value, parameters, data, recogniser.dtype)
    return spec, parameters, [(name, shape) for name, shape, _ in data]
