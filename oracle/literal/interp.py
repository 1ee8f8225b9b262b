"""CPU plan interpreter of the reference — TEST INFRASTRUCTURE (literal oracle).

Every node is computed in float64 and then rounded ONCE to the node dtype
(evaluate_tensor_nodes_fused, crates/quabla-core/src/tensor_ir.rs:7107-7818;
rounding :7794-7797, float32 = `as f32 as f64` :1307-1314).  Sums run
sequentially in index order (:1838-1840), a mean is sum * (1/n) (:2061-2063),
matmul accumulates in float64 (:1639-1656; NumPy's float64 matmul differs from
the reference's i-k-j loop only in the order of the float64 additions).
"""

from __future__ import annotations

import numpy as np

from .ir import F32, Graph

import math

_UNARY = {"tanh": np.tanh, "sin": np.sin, "cos": np.cos, "exp": np.exp, "log1p": np.log1p, "expm1": np.expm1,
          "tan": np.tan, "erf": np.vectorize(math.erf, otypes=[np.float64]),
          "erfc": np.vectorize(math.erfc, otypes=[np.float64])}


def _round(value: np.ndarray, dtype: str) -> np.ndarray:
    value = np.asarray(value, dtype=np.float64)
    if dtype == F32:  # Bool nodes hold 0.0 / 1.0 and need no rounding
        return value.astype(np.float32).astype(np.float64)
    return value


def _sequential_sum(a: np.ndarray, axis=None) -> np.ndarray:
    if axis is None:
        flat = a.reshape(-1)
        return np.cumsum(flat)[-1] if flat.size else np.float64(0.0)
    return np.take(np.cumsum(a, axis=axis), -1, axis=axis)


def _powi(x: np.ndarray, n: int) -> np.ndarray:
    # f64::powi: repeated multiplication (tensor_ir.rs:2072-2079).
    invert = n < 0
    e = -n if invert else n
    result = np.ones_like(x)
    base = x.copy()
    while e:
        if e & 1:
            result = result * base
        base = base * base
        e >>= 1
    return 1.0 / result if invert else result


def evaluate(graph: Graph, inputs: dict, outputs: list) -> list:
    """Values of `outputs` (node ids) as float64 arrays holding dtype-rounded numbers."""
    needed = [False] * len(graph.nodes)
    pending = list(outputs)
    while pending:
        i = pending.pop()
        if not needed[i]:
            needed[i] = True
            pending.extend(graph.node(i).inputs)
    values: list = [None] * len(graph.nodes)
    for i, node in enumerate(graph.nodes):
        if not needed[i]:
            continue
        op = node.op
        x = [values[j] for j in node.inputs]
        if op == "input":
            v = np.asarray(inputs[node.attrs[0]], dtype=np.float64).reshape(node.shape)
        elif op == "scalar_constant":
            v = np.float64(node.attrs[0])
        elif op == "constant":
            v = node.attrs[0]
        elif op == "cast":
            v = x[0]
        elif op == "add":
            v = x[0] + x[1]
        elif op == "sub":
            v = x[0] - x[1]
        elif op == "mul":
            v = x[0] * x[1]
        elif op == "div":
            v = x[0] / x[1]
        elif op == "greater":
            v = np.asarray(np.asarray(x[0]) > np.asarray(x[1]), dtype=np.float64)
        elif op == "where":
            v = np.where(np.asarray(x[0]) != 0.0, x[1], x[2])
        elif op == "powi":
            v = _powi(np.asarray(x[0], dtype=np.float64), node.attrs[0])
        elif op == "unary":
            v = _UNARY[node.attrs[0]](x[0])
        elif op == "matmul":
            v = np.matmul(x[0], x[1])
        elif op == "sum":
            v = _sequential_sum(np.asarray(x[0]))
        elif op == "mean":
            a = np.asarray(x[0])
            v = _sequential_sum(a) * (1.0 / a.size)
        elif op == "sum_axis":
            v = _sequential_sum(np.asarray(x[0]), node.attrs[0])
        elif op == "mean_axis":
            a = np.asarray(x[0])
            v = _sequential_sum(a, node.attrs[0]) * (1.0 / a.shape[node.attrs[0]])
        elif op == "reshape":
            v = np.reshape(x[0], node.shape)
        elif op == "transpose":
            v = np.transpose(x[0], node.attrs[0])
        elif op == "broadcast":
            v = np.broadcast_to(x[0], node.shape)
        elif op == "slice":
            axis, start, length = node.attrs
            v = np.take(x[0], np.arange(start, start + length), axis=axis)
        elif op == "pad_slice":
            axis, start = node.attrs
            v = np.zeros(node.shape)
            index = [slice(None)] * len(node.shape)
            index[axis] = slice(start, start + np.shape(x[0])[axis])
            v[tuple(index)] = x[0]
        elif op == "concat":
            v = np.concatenate([np.asarray(a) for a in x], axis=node.attrs[0])
        else:
            raise NotImplementedError(op)
        v = _round(v, node.dtype)
        if v.shape != node.shape:
            v = v.reshape(node.shape)
        values[i] = v
    return [values[o] for o in outputs]
