"""Tensor IR subset of the reference — TEST INFRASTRUCTURE (literal oracle).

A restatement, for the ops a tanh-MLP PDE-residual loss produces, of the
reference's `TensorIr` builder (crates/quabla-core/src/tensor_ir.rs): nodes
with an op, a shape, a dtype and a weak flag (:821-826), weak Python scalars
that adopt the strong dtype through an explicit `Cast` (:6922-7005), result
dtype and weakness derived from the value operands (:7029-7074).

Ops: input, scalar_constant, constant, cast, add, sub, mul, div, matmul, sum,
sum_axis, mean, mean_axis, reshape, transpose, broadcast, powi, unary (tanh,
sin, cos, exp, log1p, expm1, erf, erfc, tan), slice, pad_slice, concat, and the two ops the reference's
composite activations are built from: greater (a comparison with a Bool result, tensor_ir.rs Greater) and
where (a selection by a Bool condition, tensor_ir.rs Where).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

F32, F64, BOOL = "f32", "f64", "bool"
UNARY_KINDS = ("tanh", "sin", "cos", "exp", "log1p", "expm1", "erf", "erfc", "tan")


@dataclass
class Node:
    op: str
    inputs: tuple      # operand node ids
    attrs: tuple       # op-specific static attributes
    shape: tuple
    dtype: str
    weak: bool


def broadcast_shape(a: tuple, b: tuple) -> tuple:
    out = []
    for i in range(1, max(len(a), len(b)) + 1):
        x = a[-i] if i <= len(a) else 1
        y = b[-i] if i <= len(b) else 1
        if x != y and x != 1 and y != 1:
            raise ValueError(f"cannot broadcast {a} and {b}")
        out.append(max(x, y))
    return tuple(reversed(out))


class Graph:
    """An append-only node list; node ids are positions (tensor_ir.rs:829-832)."""

    def __init__(self) -> None:
        self.nodes: list[Node] = []
        self.input_ids: dict[str, int] = {}

    # -- raw push -------------------------------------------------------------
    def push(self, op, inputs, attrs, shape, dtype, weak) -> int:
        self.nodes.append(Node(op, tuple(inputs), tuple(attrs), tuple(int(s) for s in shape), dtype, bool(weak)))
        return len(self.nodes) - 1

    def node(self, i: int) -> Node:
        return self.nodes[i]

    def shape(self, i: int) -> tuple:
        return self.nodes[i].shape

    def push_derived(self, op, inputs, attrs, shape) -> int:
        """dtype of the first value operand; weak only if every operand is weak
        (push_derived, tensor_ir.rs:7029-7074)."""
        dtype = self.nodes[inputs[0]].dtype
        weak = True
        for i in inputs:
            if self.nodes[i].dtype != dtype:
                raise TypeError(f"{op} operands have mismatched dtypes")
            weak = weak and self.nodes[i].weak
        return self.push(op, inputs, attrs, shape, dtype, weak)

    # -- leaves ---------------------------------------------------------------
    def input(self, name: str, shape, dtype: str) -> int:
        if name in self.input_ids:
            raise ValueError(f"duplicate input {name!r}")
        i = self.push("input", (), (name,), shape, dtype, False)
        self.input_ids[name] = i
        return i

    def scalar_constant(self, value: float) -> int:
        """A weak float64 scalar, what a Python number becomes."""
        return self.push("scalar_constant", (), (float(value),), (), F64, True)

    def constant_like(self, value: float, dtype: str, weak: bool) -> int:
        return self.push("scalar_constant", (), (float(value),), (), dtype, weak)

    def constant(self, array, dtype: str) -> int:
        array = np.asarray(array, dtype=np.float64)
        return self.push("constant", (), (array,), array.shape, dtype, False)

    # -- coercion -------------------------------------------------------------
    def cast(self, i: int, dtype: str) -> int:
        node = self.nodes[i]
        if node.dtype == dtype and not node.weak:
            return i
        return self.push("cast", (i,), (), node.shape, dtype, False)

    def _coerce(self, operands: list[int]) -> list[int]:
        strong = None
        for i in operands:
            node = self.nodes[i]
            if node.weak:
                continue
            if strong is not None and strong != node.dtype:
                raise TypeError("operands have mismatched dtypes; convert one of them explicitly with astype")
            strong = node.dtype
        if strong is None:
            return operands
        return [i if self.nodes[i].dtype == strong else self.cast(i, strong) for i in operands]

    def _binary(self, op: str, a: int, b: int) -> int:
        shape = broadcast_shape(self.shape(a), self.shape(b))
        a, b = self._coerce([a, b])
        return self.push_derived(op, (a, b), (), shape)

    # -- arithmetic -----------------------------------------------------------
    def add(self, a, b):
        return self._binary("add", a, b)

    def sub(self, a, b):
        return self._binary("sub", a, b)

    def mul(self, a, b):
        return self._binary("mul", a, b)

    def div(self, a, b):
        return self._binary("div", a, b)

    def greater(self, a: int, b: int) -> int:
        """a > b elementwise; the result is a strong Bool node."""
        shape = broadcast_shape(self.shape(a), self.shape(b))
        a, b = self._coerce([a, b])
        return self.push("greater", (a, b), (), shape, BOOL, False)

    def where(self, condition: int, on_true: int, on_false: int) -> int:
        """where_select: the value operands are coerced like a binary op's; the condition is Bool."""
        if self.nodes[condition].dtype != BOOL:
            raise TypeError("where needs a Bool condition")
        on_true, on_false = self._coerce([on_true, on_false])
        shape = broadcast_shape(self.shape(condition), broadcast_shape(self.shape(on_true), self.shape(on_false)))
        dtype = self.nodes[on_true].dtype
        weak = self.nodes[on_true].weak and self.nodes[on_false].weak
        return self.push("where", (condition, on_true, on_false), (), shape, dtype, weak)

    def powi(self, a: int, exponent: int) -> int:
        return self.push_derived("powi", (a,), (int(exponent),), self.shape(a))

    def unary(self, a: int, kind: str) -> int:
        if kind not in UNARY_KINDS:
            raise ValueError(kind)
        return self.push_derived("unary", (a,), (kind,), self.shape(a))

    def matmul(self, a: int, b: int) -> int:
        sa, sb = self.shape(a), self.shape(b)
        if len(sa) < 2 or len(sb) < 2 or sa[-1] != sb[-2]:
            raise ValueError(f"matmul of {sa} and {sb}")
        batch = broadcast_shape(sa[:-2], sb[:-2])
        a, b = self._coerce([a, b])
        return self.push_derived("matmul", (a, b), (), batch + (sa[-2], sb[-1]))

    # -- reductions -------------------------------------------------------------
    def sum(self, a: int) -> int:
        return self.push_derived("sum", (a,), (), ())

    def mean(self, a: int) -> int:
        return self.push_derived("mean", (a,), (), ())

    def _axis(self, a: int, axis: int) -> int:
        rank = len(self.shape(a))
        if not -rank <= axis < rank:
            raise ValueError(f"axis {axis} for rank {rank}")
        return axis % rank

    def sum_axis(self, a: int, axis: int) -> int:
        axis = self._axis(a, axis)
        shape = self.shape(a)
        return self.push_derived("sum_axis", (a,), (axis,), shape[:axis] + shape[axis + 1:])

    def mean_axis(self, a: int, axis: int) -> int:
        axis = self._axis(a, axis)
        shape = self.shape(a)
        return self.push_derived("mean_axis", (a,), (axis,), shape[:axis] + shape[axis + 1:])

    # -- data movement ------------------------------------------------------------
    def reshape(self, a: int, shape) -> int:
        shape = tuple(int(s) for s in shape)
        if int(np.prod(shape, dtype=np.int64)) != int(np.prod(self.shape(a), dtype=np.int64)):
            raise ValueError(f"cannot reshape {self.shape(a)} to {shape}")
        return self.push_derived("reshape", (a,), (), shape)

    def transpose(self, a: int, axes=None) -> int:
        rank = len(self.shape(a))
        axes = tuple(reversed(range(rank))) if axes is None else tuple(int(x) % rank for x in axes)
        shape = tuple(self.shape(a)[x] for x in axes)
        return self.push_derived("transpose", (a,), (axes,), shape)

    def broadcast_to(self, a: int, shape) -> int:
        shape = tuple(int(s) for s in shape)
        if broadcast_shape(self.shape(a), shape) != shape:
            raise ValueError(f"cannot broadcast {self.shape(a)} to {shape}")
        return self.push_derived("broadcast", (a,), (), shape)

    def slice(self, a: int, axis: int, start: int, length: int) -> int:
        axis = self._axis(a, axis)
        shape = list(self.shape(a))
        if start < 0 or start + length > shape[axis]:
            raise ValueError("slice out of range")
        shape[axis] = length
        return self.push_derived("slice", (a,), (axis, int(start), int(length)), shape)

    def pad_slice(self, a: int, shape, axis: int, start: int) -> int:
        """Zeros of `shape` with `a` placed at `start` along `axis` (the VJP of slice)."""
        return self.push_derived("pad_slice", (a,), (int(axis), int(start)), tuple(shape))

    def concat(self, items: list[int], axis: int) -> int:
        items = self._coerce(list(items))
        axis = self._axis(items[0], axis)
        shape = list(self.shape(items[0]))
        shape[axis] = sum(self.shape(i)[axis] for i in items)
        return self.push_derived("concat", tuple(items), (axis,), shape)

    # -- rebuilding -----------------------------------------------------------------
    def rebuild_like(self, node: Node, remap) -> int:
        """Copy `node` with remapped operands, keeping its dtype and weak flag
        (rebuild_like, crates/quabla-core/src/tensor_ir/op/rebuild.rs:14-115)."""
        return self.push(node.op, tuple(remap(i) for i in node.inputs), node.attrs, node.shape, node.dtype, node.weak)
